/*
 * samq.h — C ABI of the B200 (sm_100a) W8A8 quantized-linear engine.
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream handle
 * (passed as void*, i.e. a cudaStream_t / CUstream), allocates nothing, never
 * synchronises, never throws and returns an int status: 0 on success, a
 * negative SAMQ_ERR_* value otherwise.  samq_last_error_string() returns a
 * thread-local description of the last failure on the calling thread.
 *
 * The reference project exposes its native path as a pybind11 torch extension
 * named `qgemm` (quant/qgemm/kernels/bindings.cpp:98-134) with three calls:
 * `sym_quant`, `matmul` and `sym_dequant`.  The functions below replace those
 * three calls (and the PyTorch fake-quant functions of
 * RTN_quantization/per_tensor_channel_group.py that the model path really
 * runs) with real int8 arithmetic.  Each declaration cites what it replaces.
 *
 * Conventions (same as the reference's native code, quant/qgemm/include/gemm_int8.h:5-9):
 *   A / X  : [M, K] row-major, K contiguous ("K-major")
 *   W      : [N, K] row-major, K contiguous (i.e. the nn.Linear weight as stored)
 *   C / Y  : [M, N] row-major
 */
#ifndef SAMQ_H_
#define SAMQ_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
#define SAMQ_OK                 0
#define SAMQ_ERR_BAD_ARG       -1   /* null pointer, negative size, unknown enum      */
#define SAMQ_ERR_UNSUPPORTED   -2   /* shape / dtype / granularity not implemented    */
#define SAMQ_ERR_ALIGNMENT     -3   /* pointer or leading dimension not aligned       */
#define SAMQ_ERR_CUDA          -4   /* a CUDA runtime / driver call failed            */
#define SAMQ_ERR_WORKSPACE     -5   /* workspace missing or too small                 */
#define SAMQ_ERR_TOO_LARGE     -6   /* size beyond a fixed built-in limit             */

/* ---- enums -------------------------------------------------------------- */
/* element type of a floating tensor */
#define SAMQ_F16   0
#define SAMQ_BF16  1
#define SAMQ_F32   2
/* GEMM output type additionally allows the raw accumulators */
#define SAMQ_I32   3

/* quantization granularity.  For activations these are the reference strings
 * "per_token" | "per_tensor" | "per_group_token"
 * (RTN_quantization/per_tensor_channel_group.py:130-140); for weights
 * "per_channel" | "per_tensor" | "per_group" (:178-192).  A weight row is a
 * "token" of the same arithmetic, so one enum serves both. */
#define SAMQ_GRAN_ROW     0   /* per_token   / per_channel : scale[M]        */
#define SAMQ_GRAN_TENSOR  1   /* per_tensor                : scale[1]        */
#define SAMQ_GRAN_GROUP   2   /* per_group_token/per_group : scale[M, K/g]   */

/* epilogue activation */
#define SAMQ_ACT_NONE  0
#define SAMQ_ACT_GELU  1      /* exact erf GELU (torch.nn.GELU default)       */

/* online Hadamard modes of quarot/utils.py:253-289 */
#define SAMQ_HAD_NONE     0
#define SAMQ_HAD_FULL     1   /* online_full_had : transform over the whole last dim        */
#define SAMQ_HAD_PARTIAL  2   /* online_partial_had : transform across the head axis,
                                 last dim viewed as [K/had_dim, had_dim]                     */

/* Description of the transform applied before quantization.
 *
 * mode FULL over n = K columns follows quarot/hadamard_utils.py:59-80
 * (`matmul_hadU`): n = had_k * 2^p; an in-place Walsh–Hadamard butterfly with
 * strides 1,2,4,... over each contiguous chunk of 2^p columns, then the
 * explicit had_k x had_k (+-1) matrix `hadk` mixes the had_k chunks, then a
 * division by sqrtf(n).  had_k == 1 means n is a power of two and `hadk` is
 * ignored.  All arithmetic is fp32 on the up-cast input, rounded once to the
 * tensor dtype (the `fp32_had` branch of quarot/utils.py:258-259).
 *
 * mode PARTIAL follows quarot/utils.py:263-289: the last dim is viewed as
 * [heads = K / had_dim, had_dim] and the transform (size `heads`) runs over
 * the head axis for every position inside a head, scaled by 1/sqrt(heads).
 *
 * `signs` (optional, [K] int8 of +-1) multiplies column j by signs[j] before
 * the transform: x @ random_hadamard_matrix(n) == hadU(x * signs)
 * (quarot/hadamard_utils.py:86-94; quarot/model_utils.py:146-152,235-240). */
typedef struct samq_hadamard_spec {
    int32_t       mode;      /* SAMQ_HAD_*                                         */
    int32_t       had_k;     /* 1, 12, 20, 28, 36, 40, ... (size of `hadk`)        */
    const float*  hadk;      /* device, [had_k, had_k] row-major, or NULL          */
    int32_t       had_dim;   /* PARTIAL only: width of one head                    */
    const int8_t* signs;     /* device, [K] of +-1, or NULL                        */
} samq_hadamard_spec;

/* Steps that may run inside the quantization kernel before the absmax, replacing separate
 * passes of the encoder block (quarot/model_utils.py:180-198):
 *   row_map   : gather. Output row r is computed from source row row_map[r]; a negative entry
 *               yields a row of zeros — `window_partition` with its zero padding
 *               (quarot/model_utils.py:15-36) or `window_unpartition` (:39-59) as an index map.
 *               M of the call is the number of OUTPUT rows.
 *   ln_weight / ln_bias / ln_eps : LayerNorm over the K columns of the (gathered) source row,
 *               fp32 statistics, result rounded once to `dtype` (norm1 / norm2 of the block).
 *               Padding rows stay zero (the reference pads after the norm).
 *   src_dtype : storage type of x when it differs from `dtype`, or -1. Supported pair:
 *               SAMQ_BF16 storage with dtype SAMQ_F16 (bf16 attention output that the model
 *               casts to fp16 before `proj`). */
typedef struct samq_quant_prologue {
    const int32_t* row_map;    /* device, [M] int32, or NULL                 */
    const void*    ln_weight;  /* device, [K] of `dtype`, or NULL            */
    const void*    ln_bias;    /* device, [K] of `dtype`, or NULL            */
    float          ln_eps;
    int32_t        src_dtype;  /* SAMQ_* or -1                               */
} samq_quant_prologue;

/* ---- library ------------------------------------------------------------ */

/* Library version, major*10000 + minor*100 + patch.  No reference counterpart
 * (the pybind module has no version attribute). */
int samq_version(void);

/* Thread-local message for the last non-zero status returned on this thread. */
const char* samq_last_error_string(void);

/* Number of bytes of zero-initialised-by-the-call workspace the given
 * quantization call needs (0 for ROW and GROUP; 256 for TENSOR, which holds
 * the running absolute maximum).  The caller allocates it. */
size_t samq_quant_workspace_bytes(int granularity);

/* ---- K1: activation / weight quantization -------------------------------
 *
 * Replaces `qgemm.sym_quant` (quant/qgemm/kernels/bindings.cpp:29-48,
 * quant.cu:11-61) plus the torch absmax that feeds it, and restates on the GPU
 *   quantize_activation_per_token_absmax            per_tensor_channel_group.py:53-61
 *   quantize_activation_per_tensor_absmax           :64-72
 *   quantize_activation_per_group_absmax_token_dim  :74-93
 *   quantize_weight_per_channel_absmax              :5-12
 *   quantize_weight_per_tensor_absmax               :14-21
 *   quantize_weight_per_group_absmax_input_features :23-50
 * stopping before the final `mul_(scales)`:
 *     s = max(absmax, 1e-5) / q_max        (in the tensor dtype; q_max = 2^(n_bits-1) - 1)
 *     q = round_half_even(x / s)           (quotient rounded to the tensor dtype first)
 * n_bits is the reference's `n_bits` argument, 2..8; codes of fewer than 8 bits are still
 * stored one per int8 and feed the same int8 GEMM.
 * Optional steps before the absmax, in this order:
 *     x <- x / divisor[col]   (SmoothQuant divisor, RTN_quantization/Smooth.py:39-40),
 *     x <- hadamard(x * signs) (see samq_hadamard_spec), each rounded once to the dtype.
 *
 * x        : [M, K] of `dtype`, row stride `ldx` elements
 * q_out    : [M, K] int8 codes, saturated to [-q_max, q_max], or NULL
 * scale_out: fp32 copy of the dtype-rounded scale: [M] | [1] | [M, K/group], or NULL
 * fq_out   : [M, K] of `dtype`, the fake-quantized value q*s exactly as the
 *            reference function returns it (no saturation), or NULL
 * tx_out   : [M, K] of `dtype`, the transformed but unquantized input, or NULL
 * workspace: see samq_quant_workspace_bytes(); may be NULL when that is 0.
 * Hadamard is only combined with SAMQ_GRAN_ROW. */
int samq_act_quant_i8(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx,
                      const void* divisor, const samq_hadamard_spec* had,
                      int granularity, int group_size, int n_bits,
                      int8_t* q_out, float* scale_out, void* fq_out, void* tx_out,
                      void* workspace, size_t workspace_bytes, void* stream);

/* samq_act_quant_i8 with a prologue (see samq_quant_prologue); `prologue` may be NULL. */
int samq_act_quant_i8_ex(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx,
                         const samq_quant_prologue* prologue,
                         const void* divisor, const samq_hadamard_spec* had,
                         int granularity, int group_size, int n_bits,
                         int8_t* q_out, float* scale_out, void* fq_out, void* tx_out,
                         void* workspace, size_t workspace_bytes, void* stream);

/* Same arithmetic applied to a weight [N, K] (rows = output channels).  Kept as
 * its own symbol because the reference names the weight quantizers separately
 * (per_tensor_channel_group.py:5-50). scale_out: [N] | [1] | [N, K/group]. */
int samq_weight_quant_i8(const void* w, int dtype, int64_t N, int64_t K, int64_t ldw,
                         int granularity, int group_size, int n_bits,
                         int8_t* q_out, float* scale_out, void* fq_out,
                         void* workspace, size_t workspace_bytes, void* stream);

/* Per-tensor activation quantization that allocates nothing and takes no workspace.
 *
 * This entry point has no counterpart in the reference.  It exists for callers that cannot
 * obtain device memory on the path that runs a layer — a plugin living inside a host process
 * that pre-sized its arena, or code executing while the allocator must stay untouched — and
 * therefore cannot supply the 256-byte workspace samq_act_quant_i8 wants for SAMQ_GRAN_TENSOR.
 * The scratch (one partial maximum per 64 rows plus the reduced maximum, 16.4 KB) is a fixed
 * array inside the library image; each GPU that loads the library holds it until exit.
 *
 * Same arithmetic and outputs as samq_act_quant_i8(..., SAMQ_GRAN_TENSOR, ...) without a
 * divisor or Hadamard: q_out [M,K] int8 (or NULL), scale_out [1] fp32 (or NULL), fq_out [M,K]
 * of `dtype` (or NULL).
 *
 * Limits and rules:
 *  - at most 262144 rows (64 rows x 4096 scratch slots); larger M returns SAMQ_ERR_TOO_LARGE;
 *  - the first call on each device looks up the array's device address (no allocation); make
 *    that first call outside any stream capture;
 *  - all calls on a device share the one array, which keeps what the previous call left there.
 *    Nothing in it has to be zeroed (each call overwrites every slot it later reads), but two
 *    calls that overlap on the GPU (different streams, no ordering) race on it: serialise them. */
int samq_act_quant_per_tensor_static(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx, int n_bits,
                                     int8_t* q_out, float* scale_out, void* fq_out, void* stream);

/* ---- K2: int8 GEMM with fused dequant epilogue ---------------------------
 *
 * Replaces `qgemm.matmul` + `qgemm.sym_dequant`
 * (quant/qgemm/kernels/bindings.cpp:7-26,51-91; gemm.cu:6-45; quant.cu:64-97),
 * the orphan `matmul_i8_host` (quant/qgemm/kernels/gemm_int8.cu:4-39) and the
 * float `F.linear` of W8A8Linear.forward (per_tensor_channel_group.py:157-162):
 *
 *   acc[m,n] = sum_k A[m,k] * W[n,k]                      (int32, exact)
 *   y[m,n]   = act( float(acc) * a_scale[m] * w_scale[n] + bias[n] ) + residual[m,n]
 *
 * computed with tcgen05.mma kind::i8 into tensor memory.  With grouped scales
 * (either operand) the int32 partial sum of each group of `group_size`
 * columns of K is scaled on its own and the products are summed in fp32;
 * group_size must then be a multiple of 32 that divides K, with at most 160
 * groups per row (SAMQ_ERR_UNSUPPORTED / SAMQ_ERR_TOO_LARGE otherwise).
 *
 * A        : [M, K] int8, row stride lda bytes (lda % 16 == 0, base 16-byte aligned)
 * W        : [N, K] int8, row stride ldw bytes (same alignment rule)
 * a_scale  : fp32 [M] (ROW) | [1] (TENSOR) | [M, K/group] (GROUP); NULL = 1.0
 * w_scale  : fp32 [N] (ROW) | [1] (TENSOR) | [N, K/group] (GROUP); NULL = 1.0
 * bias     : [N] of `out_dtype` (fp32 when out_dtype is I32/F32), or NULL
 * residual : [M, N] of `out_dtype`, row stride ldr elements, or NULL
 * out      : [M, N] of out_dtype (F16 | BF16 | F32 | I32), row stride ldo elements.
 *            With SAMQ_I32 the raw accumulators are stored and scales, bias,
 *            activation and residual must all be absent.
 * status   : optional device int32; the kernel writes a non-zero code there if
 *            one of its bounded waits ran out (it then returns early instead
 *            of hanging). The caller reads it after synchronising. */
int samq_gemm_i8(const int8_t* A, int64_t lda, const int8_t* W, int64_t ldw,
                 int64_t M, int64_t N, int64_t K,
                 const float* a_scale, int a_gran,
                 const float* w_scale, int w_gran, int group_size,
                 const void* bias, const void* residual, int64_t ldr,
                 int activation, void* out, int out_dtype, int64_t ldo,
                 int32_t* status, void* stream);

/* Self-test of the GEMM kernel's failure path.  The reference reports a failed native call by
 * throwing from `ensure()` (quant/qgemm/include/common.h:16-23) after the fact; a persistent
 * tensor-core pipeline can instead stall (a load that never lands), so every wait inside these
 * kernels is bounded and a kernel that gives up raises `status` and returns on its own.  This
 * entry runs the raw-int32 GEMM (A [M,K], W [N,K] -> out [M,N], M*N <= 2^22) with a stall made
 * on the host side of the launch: the producer warp never loads k-block `skip_kblock` of each
 * CTA's first tile, and waits give up after `wait_limit_cycles` SM cycles (1e5 .. 4e9).  No
 * fault, trap or endless loop is involved: the kernel drains its roles, frees its tensor memory,
 * sets *status = 1 and returns; `out` is then incomplete.  The next samq_gemm_i8 call is unaffected. */
int samq_gemm_i8_stall_selftest(const int8_t* A, int64_t lda, const int8_t* W, int64_t ldw,
                                int64_t M, int64_t N, int64_t K, int32_t* out, int64_t ldo,
                                int skip_kblock, long long wait_limit_cycles, int32_t* status, void* stream);

/* ---- the packed int4 format of the reference's native extension -------------------------------
 *
 * Replace `qgemm.sym_quant`, `qgemm.matmul` and `qgemm.sym_dequant`
 * (quant/qgemm/kernels/bindings.cpp:7-91; quant.cu:11-97; gemm.cu:6-45) with the same data formats:
 * two 4-bit two's-complement codes per byte, element 2j in the low nibble of byte j.
 *
 * samq_sym_quant_i4    : x fp16 [rows, cols] (row stride ldx elements), scale fp16 [rows] ->
 *                        q_packed uint8 [rows, (cols + 1) / 2]:
 *                        q = clamp(round_half_even(half(x / scale[row])), -8, 7)      (quant.cu:11-46)
 * samq_pack_i4 / samq_unpack_i4 : int8 codes in [-8, 7] <-> the packed form (what a weight quantized
 *                        with n_bits = 4 is stored as; widened to int8 on the way into the GEMM)
 * samq_matmul_i4       : C int32 [M, N] = A [M, K] x B [N, K]^T from packed operands [M, K/2], [N, K/2]
 *                        (bindings.cpp:7-26).  The tensor cores have no 4-bit integer kind: the codes are
 *                        widened into `workspace` ((M + N) * round_up(K, 16) bytes, 16-byte aligned) and
 *                        multiplied by the int8 tcgen05 GEMM; the result is exact.
 * samq_sym_dequant_i32 : out fp16 [rows, cols] = (scale_row[m] * scale_col[n]) * half(q[m, n]), every
 *                        product rounded to fp16 as quant.cu:64-80 does (|q| beyond 65504 overflows there
 *                        too; the fused epilogue of samq_gemm_i8 dequantises in fp32 instead). */
int samq_sym_quant_i4(const void* x, const void* scale, int64_t rows, int64_t cols, int64_t ldx, uint8_t* q_packed, void* stream);
int samq_pack_i4(const int8_t* codes, int64_t rows, int64_t cols, int64_t ldc, uint8_t* q_packed, int64_t ldq, void* stream);
int samq_unpack_i4(const uint8_t* q_packed, int64_t rows, int64_t cols, int64_t ldq, int8_t* codes, int64_t ldc, void* stream);
int samq_matmul_i4(const uint8_t* A, const uint8_t* B, int64_t M, int64_t N, int64_t K, void* workspace, size_t workspace_bytes,
                   int32_t* C, int32_t* status, void* stream);
int samq_sym_dequant_i32(const int32_t* q, const void* scale_row, const void* scale_col, int64_t rows, int64_t cols,
                         void* out, void* stream);

/* Process-wide choice between the two implementations of samq_gemm_i8 for row / tensor scales
 * (no reference counterpart: the reference has a single cuBLAS-style path):
 *   NEVER  - one CTA per 128 x 256 output tile;
 *   ALWAYS - CTA pairs (thread-block clusters of two, tcgen05 cta_group::2) per 256 x 256 tile,
 *            each CTA loading half of the W tile;
 *   AUTO   - (the default) pairs when M >= SAMQ_GEMM_PAIR_MIN_ROWS and K >= SAMQ_GEMM_PAIR_MIN_K,
 *            single CTAs otherwise.
 * Both give bit-identical results.  Returns the previous mode, or -1 for an unknown mode. */
#define SAMQ_GEMM_PAIR_NEVER  0
#define SAMQ_GEMM_PAIR_AUTO   1
#define SAMQ_GEMM_PAIR_ALWAYS 2
#define SAMQ_GEMM_PAIR_MIN_ROWS 2048
#define SAMQ_GEMM_PAIR_MIN_K 4096
int samq_gemm_set_pair_mode(int mode);

/* ---- attention-side helpers (the step between qkv and proj) -------------------------------
 *
 * They implement the decomposed relative position bias that the reference applies through
 * `add_decomposed_rel_pos` (quarot/model_utils.py:162-166):
 *   bias[(qh,qw),(kh,kw)] = q . rel_pos_h[qh-kh+H-1] + q . rel_pos_w[qw-kw+W-1].
 * The dot products come in precomputed (one small tensor-core GEMM by the caller) as
 *   rel_all[head, token, j] = q[token, head, :] . table[j, :],  j < 2H-1 : rel_pos_h rows,
 *                                                               then 2W-1 rel_pos_w rows,
 * fp16 or bf16, row pitch rel_pitch >= (2H-1)+(2W-1) elements.  The kernels move data only.
 *
 * samq_attn_window_prep reads q and k in place from the qkv GEMM output `qkv` [tokens, 3*C]
 * (C = heads*head_dim, head_dim and width multiples of 8) and writes, per token and head,
 *   q_aug = [ q*scale | rel_h[kh], kh<H | rel_w[kw], kw<W | 0.. ]   (width columns)
 *   k_aug = [ k       | onehot(kh)      | onehot(kw)      | 0.. ]
 * as [tokens, heads, width], so that softmax(q_aug k_aug^T) v equals the biased attention with
 * no bias tensor.  tokens = windows*H*W in window order; width >= head_dim + H + W.
 *
 * samq_attn_rel_bias writes the explicit bias [images, heads, H*W, H*W] for global attention,
 * where H + W extra columns would not fit a fused attention kernel (H <= 64, W % 8 == 0). */
int samq_attn_window_prep(const void* qkv, const void* rel_all, int dtype, int64_t tokens, int rel_pitch,
                          int H, int W, int num_heads, int head_dim, float scale, int width,
                          void* q_aug, void* k_aug, void* stream);

int samq_attn_rel_bias(const void* rel_all, int dtype, int64_t images, int rel_pitch, int H, int W, int num_heads,
                       void* bias, void* stream);

/* ---- attention on the tensor cores ----------------------------------------
 *
 * Replaces the attention of quarot/model_utils.py:158-170 (`(q * scale) @ k^T`,
 * `add_decomposed_rel_pos`, softmax, `@ v`) for one "unit" of H x W tokens at a time:
 * a whole image (global blocks: W = 64, H * 64 a multiple of 128) or a window
 * (H, W <= 16).  Scores, bias and probabilities never leave the SM (tcgen05.mma kind::f16,
 * scores and the output accumulator in tensor memory, online softmax in fp32).
 *
 * samq_attn_transpose_v : V of every (unit, head) as [head_dim, keys], keys contiguous, from
 *                         qkv [units * H * W, 3C].  keys = H * W for images; for windows the key
 *                         (kh, kw) sits at kh * 16 + kw and the row is zero-padded to a multiple
 *                         of 64.  vt is [units * heads * head_dim, keys].
 * samq_attn_global      : out [units * H * W, C] (same 16-bit dtype) from qkv and
 *                         rel_all [heads, units * H * W, rel_pitch] (see samq_attn_window_prep).
 *                         head_dim 64 or 80.  V is read where the qkv GEMM left it (as the
 *                         MN-major operand of the P V product); `vt` is ignored and may be NULL
 *                         (the argument remains for callers built against the earlier interface,
 *                         which needed samq_attn_transpose_v first).
 * status : optional device int32, set non-zero if a bounded wait inside the kernel ran out. */
int samq_attn_transpose_v(const void* qkv, int dtype, int64_t units, int H, int W, int num_heads, int head_dim,
                          void* vt, void* stream);
int samq_attn_global(const void* qkv, const void* vt, const void* rel_all, int dtype, int64_t units, int rel_pitch,
                     int H, int W, int num_heads, int head_dim, float scale, void* out, int32_t* status, void* stream);

/* Whole windowed attention in one kernel: for every window (H*W tokens, H*W <= 208) and head,
 *   out[w, l, h, :] = softmax_k( scale * q.k + q.rel_pos_h[qh-kh+H-1] + q.rel_pos_w[qw-kw+W-1] ) v
 * with q, k, v read in place from `qkv` [windows*H*W, 3*C] (fp16 or bf16, 16-byte aligned) and
 * `out` [windows*H*W, C] of the same dtype. `rel_table` holds the 2H-1 rows of rel_pos_h followed
 * by the 2W-1 rows of rel_pos_w, [table_rows, head_dim] with table_rows rounded up to a multiple
 * of 8 (extra rows zero). It is the attention between qkv and proj of a
 * windowed block (quarot/model_utils.py:158-170), with the bias never materialised.
 * head_dim 64 or 80 for windows up to 14x14 (16, 32, 64 for windows of up to 16 tokens);
 * other shapes return SAMQ_ERR_UNSUPPORTED. */
int samq_attn_windowed(const void* qkv, int dtype, int64_t windows, int H, int W, int num_heads, int head_dim,
                       const void* rel_table, int table_rows, float scale, void* out, void* stream);

/* The same attention for SAM's 14 x 14 windows on the tensor cores, the default for windowed
 * blocks (replaces quarot/model_utils.py:158-170 on the windows of quarot/model_utils.py:15-36):
 * a persistent tcgen05 kernel walks (window, head) items; Q, K, V are read in place from
 * `qkv` [windows * 196, 3C] by TMA; the products of each query with the two relative-position
 * tables come out of the same MMA as its scores; softmax is exact two-pass in fp32; nothing but
 * `out` [windows * 196, C] is written.
 * rel_table : [56, head_dim] of the qkv dtype: the 27 rows of rel_pos_h, the 27 rows of rel_pos_w,
 *             two zero rows (table_rows must be 56).
 * head_dim 64 or 80; dtype SAMQ_F16 or SAMQ_BF16; qkv, rel_table and out 16-byte aligned.
 * status : optional device int32, set non-zero if a bounded wait inside the kernel ran out. */
int samq_attn_window14(const void* qkv, const void* rel_table, int table_rows, int dtype, int64_t windows,
                       int num_heads, int head_dim, float scale, void* out, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SAMQ_H_ */
