// extern "C" surface of libsamq: argument checks, thread-local error text and dispatch
// into the kernels.  Declarations and the reference interfaces they replace: include/samq.h.
#include "common.cuh"
#include <string.h>
#include <atomic>

namespace samq {

char* error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

int act_quant_dispatch(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx,
                       const samq_quant_prologue* prologue,
                       const void* divisor, const samq_hadamard_spec* had,
                       int gran, int group_size, int n_bits, int8_t* q, float* scale, void* fq, void* tx,
                       void* workspace, size_t workspace_bytes, void* stream);

int act_quant_per_tensor_static_dispatch(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx, int n_bits,
                                         int8_t* q, float* scale, void* fq, void* stream);

int gemm_i8_dispatch(const int8_t* A, int64_t lda, const int8_t* W, int64_t ldw,
                     int64_t M, int64_t N, int64_t K,
                     const float* a_scale, int a_gran, const float* w_scale, int w_gran, int group_size,
                     const void* bias, const void* residual, int64_t ldr, int activation,
                     void* out, int out_dtype, int64_t ldo, int32_t* status, void* stream);

int gemm_i8_pair_dispatch(const int8_t* A, int64_t lda, const int8_t* W, int64_t ldw,
                          int64_t M, int64_t N, int64_t K,
                          const float* a_scale, int a_gran, const float* w_scale, int w_gran, int group_size,
                          const void* bias, const void* residual, int64_t ldr, int activation,
                          void* out, int out_dtype, int64_t ldo, int32_t* status, void* stream);

int gemm_i8_grouped_dispatch(const int8_t* A, int64_t lda, const int8_t* W, int64_t ldw,
                             int64_t M, int64_t N, int64_t K,
                             const float* a_scale, int a_gran, const float* w_scale, int w_gran, int group_size,
                             const void* bias, const void* residual, int64_t ldr, int activation,
                             void* out, int out_dtype, int64_t ldo, int32_t* status, void* stream);

int attn_window_prep_dispatch(const void* qkv, const void* rel_all, int dtype, int64_t tokens, int J,
                              int H, int W, int nh, int d, float scale, int width, void* qa, void* ka, void* stream);

int attn_rel_bias_dispatch(const void* rel_all, int dtype, int64_t images, int J, int H, int W, int nh, void* bias, void* stream);

int attn_transpose_v_dispatch(const void* qkv, int dtype, int64_t units, int H, int W, int heads, int head_dim, void* vt, void* stream);

int attn_global_dispatch(const void* qkv, const void* vt, const void* rel_all, int dtype, int64_t images, int rel_pitch,
                         int H, int W, int heads, int head_dim, float scale, void* out, int32_t* status, void* stream);

int gemm_i8_stall_selftest_dispatch(const int8_t* A, int64_t lda, const int8_t* W, int64_t ldw, int64_t M, int64_t N, int64_t K,
                                    int32_t* out, int64_t ldo, int skip_kblock, long long wait_limit_cycles,
                                    int32_t* status, void* stream);
int sym_quant_i4_dispatch(const void* x, const void* scale, int64_t rows, int64_t cols, int64_t ldx, uint8_t* q, void* stream);
int unpack_i4_dispatch(const uint8_t* q, int64_t rows, int64_t cols, int64_t ldq, int8_t* out, int64_t ldo, void* stream);
int pack_i4_dispatch(const int8_t* codes, int64_t rows, int64_t cols, int64_t ldc, uint8_t* q, int64_t ldq, void* stream);
int sym_dequant_i32_dispatch(const int32_t* q, const void* scale_row, const void* scale_col, int64_t rows, int64_t cols, void* out, void* stream);
int attn_window14_dispatch(const void* qkv, const void* table, int table_rows, int dtype, int64_t windows, int heads, int head_dim,
                           float scale, void* out, int32_t* status, void* stream);
int attn_window_dispatch(const void* qkv, int dtype, int64_t windows, int H, int W, int nh, int d,
                         const void* table, int table_rows, float scale, void* out, void* stream);

}  // namespace samq

namespace {
std::atomic<int> g_gemm_pair_mode{SAMQ_GEMM_PAIR_AUTO};
}

extern "C" {

int samq_version(void) { return 100; }   // 0.1.0

const char* samq_last_error_string(void) { return samq::error_buffer(); }

size_t samq_quant_workspace_bytes(int granularity) {
    return granularity == SAMQ_GRAN_TENSOR ? 256 : 0;
}

int samq_act_quant_i8(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx,
                      const void* divisor, const samq_hadamard_spec* had,
                      int granularity, int group_size, int n_bits,
                      int8_t* q_out, float* scale_out, void* fq_out, void* tx_out,
                      void* workspace, size_t workspace_bytes, void* stream)
{
    return samq::act_quant_dispatch(x, dtype, M, K, ldx, nullptr, divisor, had, granularity, group_size, n_bits,
                                    q_out, scale_out, fq_out, tx_out, workspace, workspace_bytes, stream);
}

int samq_act_quant_i8_ex(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx,
                         const samq_quant_prologue* prologue,
                         const void* divisor, const samq_hadamard_spec* had,
                         int granularity, int group_size, int n_bits,
                         int8_t* q_out, float* scale_out, void* fq_out, void* tx_out,
                         void* workspace, size_t workspace_bytes, void* stream)
{
    return samq::act_quant_dispatch(x, dtype, M, K, ldx, prologue, divisor, had, granularity, group_size, n_bits,
                                    q_out, scale_out, fq_out, tx_out, workspace, workspace_bytes, stream);
}

int samq_weight_quant_i8(const void* w, int dtype, int64_t N, int64_t K, int64_t ldw,
                         int granularity, int group_size, int n_bits,
                         int8_t* q_out, float* scale_out, void* fq_out,
                         void* workspace, size_t workspace_bytes, void* stream)
{
    return samq::act_quant_dispatch(w, dtype, N, K, ldw, nullptr, nullptr, nullptr, granularity, group_size, n_bits,
                                    q_out, scale_out, fq_out, nullptr, workspace, workspace_bytes, stream);
}

int samq_act_quant_per_tensor_static(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx, int n_bits,
                                     int8_t* q_out, float* scale_out, void* fq_out, void* stream)
{
    return samq::act_quant_per_tensor_static_dispatch(x, dtype, M, K, ldx, n_bits, q_out, scale_out, fq_out, stream);
}

int samq_attn_window_prep(const void* qkv, const void* rel_all, int dtype, int64_t tokens, int rel_pitch,
                          int H, int W, int num_heads, int head_dim, float scale, int width,
                          void* q_aug, void* k_aug, void* stream)
{
    return samq::attn_window_prep_dispatch(qkv, rel_all, dtype, tokens, rel_pitch, H, W, num_heads, head_dim, scale,
                                           width, q_aug, k_aug, stream);
}

int samq_attn_windowed(const void* qkv, int dtype, int64_t windows, int H, int W, int num_heads, int head_dim,
                       const void* rel_table, int table_rows, float scale, void* out, void* stream)
{
    return samq::attn_window_dispatch(qkv, dtype, windows, H, W, num_heads, head_dim, rel_table, table_rows, scale, out, stream);
}

int samq_attn_window14(const void* qkv, const void* rel_table, int table_rows, int dtype, int64_t windows,
                       int num_heads, int head_dim, float scale, void* out, int32_t* status, void* stream)
{
    return samq::attn_window14_dispatch(qkv, rel_table, table_rows, dtype, windows, num_heads, head_dim, scale, out, status, stream);
}

int samq_attn_rel_bias(const void* rel_all, int dtype, int64_t images, int rel_pitch, int H, int W, int num_heads,
                       void* bias, void* stream)
{
    return samq::attn_rel_bias_dispatch(rel_all, dtype, images, rel_pitch, H, W, num_heads, bias, stream);
}

int samq_attn_transpose_v(const void* qkv, int dtype, int64_t units, int H, int W, int num_heads, int head_dim,
                          void* vt, void* stream)
{
    return samq::attn_transpose_v_dispatch(qkv, dtype, units, H, W, num_heads, head_dim, vt, stream);
}

int samq_attn_global(const void* qkv, const void* vt, const void* rel_all, int dtype, int64_t images, int rel_pitch,
                     int H, int W, int num_heads, int head_dim, float scale, void* out, int32_t* status, void* stream)
{
    return samq::attn_global_dispatch(qkv, vt, rel_all, dtype, images, rel_pitch, H, W, num_heads, head_dim, scale, out,
                                      status, stream);
}

int samq_gemm_i8(const int8_t* A, int64_t lda, const int8_t* W, int64_t ldw,
                 int64_t M, int64_t N, int64_t K,
                 const float* a_scale, int a_gran,
                 const float* w_scale, int w_gran, int group_size,
                 const void* bias, const void* residual, int64_t ldr,
                 int activation, void* out, int out_dtype, int64_t ldo,
                 int32_t* status, void* stream)
{
    if (a_gran == SAMQ_GRAN_GROUP || w_gran == SAMQ_GRAN_GROUP)
        return samq::gemm_i8_grouped_dispatch(A, lda, W, ldw, M, N, K, a_scale, a_gran, w_scale, w_gran, group_size,
                                              bias, residual, ldr, activation, out, out_dtype, ldo, status, stream);
    const int mode = g_gemm_pair_mode.load(std::memory_order_relaxed);
    // CTA pairs pay off on long reductions (operand traffic dominates; measured +1.5 % at
    // K = 5120, -4 % at K = 1280 where the epilogue hand-off across the pair costs more) and
    // once there are enough 256-row tiles to fill the device
    if (mode == SAMQ_GEMM_PAIR_ALWAYS ||
        (mode == SAMQ_GEMM_PAIR_AUTO && M >= SAMQ_GEMM_PAIR_MIN_ROWS && K >= SAMQ_GEMM_PAIR_MIN_K))
        return samq::gemm_i8_pair_dispatch(A, lda, W, ldw, M, N, K, a_scale, a_gran, w_scale, w_gran, group_size,
                                           bias, residual, ldr, activation, out, out_dtype, ldo, status, stream);
    return samq::gemm_i8_dispatch(A, lda, W, ldw, M, N, K, a_scale, a_gran, w_scale, w_gran, group_size,
                                  bias, residual, ldr, activation, out, out_dtype, ldo, status, stream);
}

int samq_gemm_i8_stall_selftest(const int8_t* A, int64_t lda, const int8_t* W, int64_t ldw, int64_t M, int64_t N, int64_t K,
                                int32_t* out, int64_t ldo, int skip_kblock, long long wait_limit_cycles,
                                int32_t* status, void* stream)
{
    return samq::gemm_i8_stall_selftest_dispatch(A, lda, W, ldw, M, N, K, out, ldo, skip_kblock, wait_limit_cycles, status, stream);
}

int samq_sym_quant_i4(const void* x, const void* scale, int64_t rows, int64_t cols, int64_t ldx, uint8_t* q_packed, void* stream)
{
    return samq::sym_quant_i4_dispatch(x, scale, rows, cols, ldx, q_packed, stream);
}

int samq_unpack_i4(const uint8_t* q_packed, int64_t rows, int64_t cols, int64_t ldq, int8_t* codes, int64_t ldc, void* stream)
{
    return samq::unpack_i4_dispatch(q_packed, rows, cols, ldq, codes, ldc, stream);
}

int samq_pack_i4(const int8_t* codes, int64_t rows, int64_t cols, int64_t ldc, uint8_t* q_packed, int64_t ldq, void* stream)
{
    return samq::pack_i4_dispatch(codes, rows, cols, ldc, q_packed, ldq, stream);
}

int samq_matmul_i4(const uint8_t* A, const uint8_t* B, int64_t M, int64_t N, int64_t K, void* workspace, size_t workspace_bytes,
                   int32_t* C, int32_t* status, void* stream)
{
    if (K <= 0 || (K & 1)) return samq::fail(SAMQ_ERR_BAD_ARG, "K=%lld must be positive and even (two codes per byte)", (long long)K);
    if (M < 0 || N <= 0) return samq::fail(SAMQ_ERR_BAD_ARG, "bad shape M=%lld N=%lld", (long long)M, (long long)N);
    const int64_t Kp = (K + 15) / 16 * 16;                       // rows of the widened operands stay 16-byte aligned
    const size_t need = (size_t)(M + N) * (size_t)Kp;
    if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15))
        return samq::fail(SAMQ_ERR_WORKSPACE, "the int4 matmul needs %zu bytes of 16-byte aligned workspace ((M + N) * K rounded up to 16)", need);
    int8_t* a8 = static_cast<int8_t*>(workspace);
    int8_t* b8 = a8 + (size_t)M * Kp;
    int rc = samq::unpack_i4_dispatch(A, M, K, K / 2, a8, Kp, stream);
    if (rc != SAMQ_OK) return rc;
    rc = samq::unpack_i4_dispatch(B, N, K, K / 2, b8, Kp, stream);
    if (rc != SAMQ_OK) return rc;
    return samq_gemm_i8(a8, Kp, b8, Kp, M, N, K, nullptr, SAMQ_GRAN_ROW, nullptr, SAMQ_GRAN_ROW, 0, nullptr, nullptr, 0,
                        SAMQ_ACT_NONE, C, SAMQ_I32, N, status, stream);
}

int samq_sym_dequant_i32(const int32_t* q, const void* scale_row, const void* scale_col, int64_t rows, int64_t cols,
                         void* out, void* stream)
{
    return samq::sym_dequant_i32_dispatch(q, scale_row, scale_col, rows, cols, out, stream);
}

int samq_gemm_set_pair_mode(int mode)
{
    if (mode < SAMQ_GEMM_PAIR_NEVER || mode > SAMQ_GEMM_PAIR_ALWAYS) return -1;
    return g_gemm_pair_mode.exchange(mode, std::memory_order_relaxed);
}

}  // extern "C"
