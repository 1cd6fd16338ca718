// K2 — W8A8 GEMM on 5th-generation tensor cores (sm_100a) with a fused dequant epilogue.
//
//   acc[m,n] = sum_k A[m,k] * W[n,k]                          int8 x int8 -> int32
//   y[m,n]   = act(float(acc) * a_scale[m] * w_scale[n] + bias[n]) + residual[m,n]
//
// Replaces the three-kernel chain of the reference's native path
// (quant/qgemm/kernels/gemm.cu:6-45 or gemm_int8.cu:4-39, then quant.cu:64-97)
// and the float F.linear of W8A8Linear.forward
// (RTN_quantization/per_tensor_channel_group.py:157-162).
//
// Structure: a persistent kernel, one CTA per SM, 10 warps:
//   warp 0      TMA producer: cp.async.bulk.tensor loads of a 128x128-byte A tile and a
//               256x128-byte W tile per stage (both K-major, 128-byte swizzle), 4 stages.
//   warp 1      allocates tensor memory and issues tcgen05.mma.kind::i8 (M=128, N=256, K=32),
//               4 per stage, accumulating int32 in TMEM; tcgen05.commit releases the stage.
//   warps 2..9  epilogue: tcgen05.ld the 128x256 int32 accumulator (two warps per TMEM lane
//               quadrant, 128 columns each), dequantise, bias, GELU, residual, store.
// The accumulator is double buffered (2 x 256 TMEM columns) so the epilogue of tile i
// overlaps the MMAs of tile i+1.  Every mbarrier wait is bounded: when a wait runs out the
// kernel raises a status word and winds down instead of hanging.
#include "common.cuh"
#include "tcgen05.cuh"
#include <string.h>
#include <type_traits>

namespace samq {

namespace {

constexpr int BM = 128;            // rows of A per tile   (UMMA M)
constexpr int BN = 256;            // rows of W per tile   (UMMA N)
constexpr int BK = 128;            // bytes (= int8 elements) of K per stage: one 128B swizzle row
constexpr int UK = 32;             // K of one tcgen05.mma for 8-bit operands
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK;   // 16 KiB
constexpr int B_BYTES = BN * BK;   // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_WARPS = 8;
constexpr int THREADS = 64 + EPI_WARPS * 32;
constexpr int ACC_BUFS = 2;
constexpr int TMEM_COLS = ACC_BUFS * BN;       // 512: all of tensor memory

struct __align__(8) Control {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_full[ACC_BUFS];
    uint64_t acc_empty[ACC_BUFS];
    uint32_t tmem_base;
    uint32_t abort_flag;
};

constexpr int EPI_PARAM_FLOATS = ACC_BUFS * 2 * BN;      // w_scale and bias per accumulator buffer
constexpr int STAGING_BYTES = 32 * 64;                   // per epilogue warp: 32 rows x 64 bytes (64-byte swizzle)
constexpr size_t SMEM_BYTES = 1024 /*alignment slack*/ + (size_t)STAGES * STAGE_BYTES +
                              (size_t)EPI_WARPS * STAGING_BYTES +
                              EPI_PARAM_FLOATS * sizeof(float) + sizeof(Control);

using namespace sm100;

// Instruction descriptor for kind::i8: D = S32 (2) in bits [4,6); A, B = signed 8-bit (1) in
// [7,10) and [10,13); both operands K-major (bits 15, 16 = 0); N >> 3 in [17,23); M >> 4 in [24,29).
constexpr uint32_t kInstrDesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

// Exact (erf) GELU, x * Phi(x), with one exp2 and no division:  for z = |x| / sqrt(2),
// 0.5 * erfc(z) = 2^Q(z) with Q a degree-6 polynomial fitted on [0, 4.3] (beyond that the tail is
// below 1e-9); Phi(x) = 1 - 2^Q for x >= 0 and 2^Q otherwise.  Absolute error of the result
// < 4e-7, relative < 2e-5 — two orders below fp16 resolution — at a third of erff's cost, which
// matters because the epilogue of a K = 1280 tile has only ~20 issue slots per output.
__device__ __forceinline__ float gelu_erf(float x) {
    const float z = fminf(fabsf(x) * 0.70710678118654752440f, 4.3f);
    float q = 2.868852462e-04f;
    q = fmaf(q, z, -4.492766690e-03f);
    q = fmaf(q, z, 3.266510367e-02f);
    q = fmaf(q, z, -1.514675319e-01f);
    q = fmaf(q, z, -9.173173308e-01f);
    q = fmaf(q, z, -1.628102660e+00f);
    q = fmaf(q, z, -9.999881387e-01f);
    float h;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(h) : "f"(q));
    const float phi = (x >= 0.f) ? 1.0f - h : h;
    return x * phi;
}

template <typename OutT> struct OutOps;
template <> struct OutOps<__half> {
    static __device__ __forceinline__ float up(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half down(float v) { return __float2half_rn(v); }
};
template <> struct OutOps<__nv_bfloat16> {
    static __device__ __forceinline__ float up(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 down(float v) { return __float2bfloat16_rn(v); }
};
template <> struct OutOps<float> {
    static __device__ __forceinline__ float up(float v) { return v; }
    static __device__ __forceinline__ float down(float v) { return v; }
};

struct GemmParams {
    int M, N, K;
    const float* a_scale; int a_stride;       // stride 0 = one scale for the tensor
    const float* w_scale; int w_stride;
    const void* bias;
    const void* residual; int64_t ldr;
    void* out; int64_t ldo;
    int activation;
    int vec_ok;                                // rows of out/residual are 16-byte aligned
    int tma_store;                             // out is described by map_out: store through shared memory + TMA
    int32_t* status;
};

// OutT = __half | __nv_bfloat16 | float | int32_t (raw accumulators)
template <typename OutT>
__global__ void __launch_bounds__(THREADS, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_out, const GemmParams p)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
    uint8_t* tiles = smem_raw + pad;                                   // 1024-byte aligned
    uint8_t* staging = tiles + (size_t)STAGES * STAGE_BYTES;            // 1024-byte aligned too
    float* epi_params = reinterpret_cast<float*>(staging + (size_t)EPI_WARPS * STAGING_BYTES);
    Control* ctl = reinterpret_cast<Control*>(epi_params + EPI_PARAM_FLOATS);
    volatile uint32_t* abort_flag = &ctl->abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int m_blocks = (p.M + BM - 1) / BM;
    const int n_blocks = (p.N + BN - 1) / BN;
    const int k_blocks = (p.K + BK - 1) / BK;
    const int num_tiles = m_blocks * n_blocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(smem_u32(&ctl->full[s]), 1); mbar_init(smem_u32(&ctl->empty[s]), 1); }
        for (int b = 0; b < ACC_BUFS; ++b) { mbar_init(smem_u32(&ctl->acc_full[b]), 1); mbar_init(smem_u32(&ctl->acc_empty[b]), EPI_WARPS); }
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        if (p.tma_store) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_out) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&ctl->tmem_base)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile / n_blocks) * BM;
                const int n0 = (tile % n_blocks) * BN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort_flag)) { ok = false; break; }
                    const uint32_t bar = smem_u32(&ctl->full[stage]);
                    const uint32_t sa = smem_u32(tiles + (size_t)stage * STAGE_BYTES);
                    mbar_expect_tx(bar, STAGE_BYTES);
                    tma_load_2d(sa, &map_a, bar, kb * BK, m0);
                    tma_load_2d(sa + A_BYTES, &map_w, bar, kb * BK, n0);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                // let copies that are already in flight land before the CTA retires
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000LL) { }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            int acc = 0; uint32_t acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                if (!mbar_wait(smem_u32(&ctl->acc_empty[acc]), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(smem_u32(&ctl->full[stage]), phase, abort_flag)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t sa = smem_u32(tiles + (size_t)stage * STAGE_BYTES);
                    const uint64_t adesc = make_smem_desc(sa);
                    const uint64_t bdesc = make_smem_desc(sa + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UK; ++k) {
                        // advancing K by 32 bytes inside the 128-byte swizzle row: +2 in the (addr >> 4) field
                        mma_i8(tmem_d, adesc + (uint64_t)(k * (UK >> 4)), bdesc + (uint64_t)(k * (UK >> 4)),
                               kInstrDesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    tcgen05_commit(smem_u32(&ctl->empty[stage]));       // frees the stage when the MMAs retire
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                tcgen05_commit(smem_u32(&ctl->acc_full[acc]));           // accumulator complete
                if (++acc == ACC_BUFS) { acc = 0; acc_phase ^= 1u; }
            }
        }
    } else {
        // ---------------- epilogue ----------------
        const int ew = warp - 2;                  // 0..7
        const int quad = warp & 3;                // TMEM lane quadrant this warp may read
        const int half_n = ew >> 2;               // which 128 columns of the 256
        const int epi_tid = threadIdx.x - 64;     // 0..255
        int acc = 0; uint32_t acc_phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
            const int m0 = (tile / n_blocks) * BM;
            const int n0 = (tile % n_blocks) * BN;
            float* ws = epi_params + acc * 2 * BN;
            float* bs = ws + BN;
            if constexpr (!std::is_same<OutT, int32_t>::value) {
                const int n = n0 + epi_tid;
                float wv = 1.0f, bv = 0.0f;
                if (n < p.N) {
                    if (p.w_scale != nullptr) wv = p.w_scale[(int64_t)n * p.w_stride];
                    if (p.bias != nullptr) bv = OutOps<OutT>::up(reinterpret_cast<const OutT*>(p.bias)[n]);
                }
                ws[epi_tid] = wv; bs[epi_tid] = bv;
                asm volatile("bar.sync 1, %0;" ::"r"(EPI_WARPS * 32) : "memory");
            }
            // after a failed wait keep visiting the named barrier above so no warp is left behind
            if (ok && !mbar_wait(smem_u32(&ctl->acc_full[acc]), acc_phase, abort_flag)) ok = false;
            if (!ok) continue;
            tcgen05_fence_after();
            const int row = m0 + quad * 32 + lane;
            const bool row_ok = row < p.M;
            float a_s = 1.0f;
            if constexpr (!std::is_same<OutT, int32_t>::value) {
                if (p.a_scale != nullptr && row_ok) a_s = p.a_scale[(int64_t)row * p.a_stride];
            }
            const uint32_t stage_addr = smem_u32(staging + (size_t)ew * STAGING_BYTES);
            uint8_t* stage_ptr = staging + (size_t)ew * STAGING_BYTES;
            const int rr = quad * 32 + lane;                       // row inside the tile
            const uint32_t swz = (uint32_t)((lane >> 1) & 3);     // 64-byte swizzle: 16-byte slot ^= bits [7:8] of the offset
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                const int col0 = half_n * 128 + c * 32;
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN + col0), r);
                tmem_ld_wait();
                const int n_first = n0 + col0;
                if (n_first >= p.N) continue;                       // warp-uniform
                const int n_valid = min(32, p.N - n_first);
                constexpr int PER16 = 16 / (int)sizeof(OutT);       // elements per 16-byte vector
                constexpr int NVEC = 32 / PER16;                    // 16-byte vectors per 32 columns: 4 or 8
                uint4 packed[NVEC];
                if constexpr (std::is_same<OutT, int32_t>::value) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) packed[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                } else {
                    float y[32];
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const float4 w4 = *reinterpret_cast<const float4*>(ws + col0 + j);
                        const float4 b4 = *reinterpret_cast<const float4*>(bs + col0 + j);
                        y[j + 0] = fmaf(__int2float_rn((int)r[j + 0]) * a_s, w4.x, b4.x);
                        y[j + 1] = fmaf(__int2float_rn((int)r[j + 1]) * a_s, w4.y, b4.y);
                        y[j + 2] = fmaf(__int2float_rn((int)r[j + 2]) * a_s, w4.z, b4.z);
                        y[j + 3] = fmaf(__int2float_rn((int)r[j + 3]) * a_s, w4.w, b4.w);
                    }
                    if (p.activation == SAMQ_ACT_GELU) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) y[j] = gelu_erf(y[j]);
                    }
                    if (p.residual != nullptr && row_ok) {
                        const OutT* res = reinterpret_cast<const OutT*>(p.residual) + (int64_t)row * p.ldr + n_first;
                        if (p.vec_ok && n_valid == 32) {
#pragma unroll
                            for (int j = 0; j < NVEC; ++j) {
                                OutT tmp[PER16];
                                *reinterpret_cast<uint4*>(tmp) = *reinterpret_cast<const uint4*>(res + j * PER16);
#pragma unroll
                                for (int e = 0; e < PER16; ++e) y[j * PER16 + e] += OutOps<OutT>::up(tmp[e]);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) if (j < n_valid) y[j] += OutOps<OutT>::up(res[j]);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < NVEC; ++j) {
                        OutT tmp[PER16];
#pragma unroll
                        for (int e = 0; e < PER16; ++e) tmp[e] = OutOps<OutT>::down(y[j * PER16 + e]);
                        packed[j] = *reinterpret_cast<const uint4*>(tmp);
                    }
                }
                if (p.tma_store) {
                    // rows of 64 bytes per box: 32 columns of a 2-byte type, 16 columns of a 4-byte type
#pragma unroll
                    for (int part = 0; part < NVEC / 4; ++part) {
                        if (lane == 0) bulk_wait_read0();            // the previous box has left shared memory
                        __syncwarp();
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            *reinterpret_cast<uint4*>(stage_ptr + lane * 64 + (((uint32_t)j ^ swz) << 4)) = packed[part * 4 + j];
                        fence_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_2d(&map_out, stage_addr, n_first + part * (64 / (int)sizeof(OutT)), m0 + quad * 32);
                            bulk_commit();
                        }
                    }
                } else if (row_ok) {
                    OutT* o = reinterpret_cast<OutT*>(p.out) + (int64_t)row * p.ldo + n_first;
                    if (p.vec_ok && n_valid == 32) {
#pragma unroll
                        for (int j = 0; j < NVEC; ++j) reinterpret_cast<uint4*>(o)[j] = packed[j];
                    } else {
                        const OutT* src = reinterpret_cast<const OutT*>(packed);
#pragma unroll
                        for (int j = 0; j < 32; ++j) if (j < n_valid) o[j] = src[j];
                    }
                }
            }
            (void)rr;
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctl->acc_empty[acc]));
            if (++acc == ACC_BUFS) { acc = 0; acc_phase ^= 1u; }
        }
    }

    if (warp >= 2 && lane == 0 && p.tma_store) bulk_wait0();          // this thread's TMA stores have completed
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && ctl->abort_flag != 0 && p.status != nullptr) atomicExch(p.status, 1);
}

// ---- host side -----------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(ptr);
    }();
    return fn;
}

// [rows, K] int8 row-major with row stride ld bytes; box = box_rows x 128 bytes, 128-byte swizzle, zero fill.
int make_operand_map(CUtensorMap* map, const int8_t* base, int64_t rows, int64_t K, int64_t ld, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return fail(SAMQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SAMQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return SAMQ_OK;
}

int sm_count() {
    static thread_local int cached_dev = -1;
    static thread_local int cached = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev != cached_dev) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached = n; cached_dev = dev;
    }
    return cached;
}

// [M, N] output with row stride ldo elements of esize bytes; box = 32 rows x 64 bytes, 64-byte swizzle.
int make_out_map(CUtensorMap* map, void* base, int64_t M, int64_t N, int64_t ldo, int esize) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return fail(SAMQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
    cuuint64_t strides[1] = {(cuuint64_t)(ldo * esize)};
    cuuint32_t box[2] = {(cuuint32_t)(64 / esize), 32u};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, esize == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, base, dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                    CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SAMQ_ERR_CUDA, "cuTensorMapEncodeTiled (output) failed with CUresult %d", (int)r);
    return SAMQ_OK;
}

template <typename OutT>
int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mo, const GemmParams& p, cudaStream_t st) {
    SAMQ_CUDA_TRY(cudaFuncSetAttribute(gemm_i8_kernel<OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
    const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
    const int grid = tiles < sm_count() ? tiles : sm_count();
    gemm_i8_kernel<OutT><<<grid, THREADS, SMEM_BYTES, st>>>(ma, mw, mo, p);
    SAMQ_CUDA_TRY(cudaGetLastError());
    return SAMQ_OK;
}

}  // namespace

int gemm_i8_dispatch(const int8_t* A, int64_t lda, const int8_t* W, int64_t ldw,
                     int64_t M, int64_t N, int64_t K,
                     const float* a_scale, int a_gran, const float* w_scale, int w_gran, int group_size,
                     const void* bias, const void* residual, int64_t ldr, int activation,
                     void* out, int out_dtype, int64_t ldo, int32_t* status, void* stream)
{
    if (M < 0 || N <= 0 || K <= 0) return fail(SAMQ_ERR_BAD_ARG, "bad GEMM shape M=%lld N=%lld K=%lld",
                                               (long long)M, (long long)N, (long long)K);
    if (M == 0) return SAMQ_OK;
    if (A == nullptr || W == nullptr || out == nullptr) return fail(SAMQ_ERR_BAD_ARG, "A, W and out must not be null");
    if (M > 2147483647LL - BM || N > 2147483647LL - BN || K > 2147483647LL - BK)
        return fail(SAMQ_ERR_TOO_LARGE, "GEMM dimension exceeds 2^31");
    if (lda < K || ldw < K || ldo < N) return fail(SAMQ_ERR_BAD_ARG, "leading dimension smaller than the row");
    if ((lda & 15) || (ldw & 15) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
        return fail(SAMQ_ERR_ALIGNMENT, "A and W need 16-byte aligned bases and row strides (lda=%lld ldw=%lld)",
                    (long long)lda, (long long)ldw);
    if (activation != SAMQ_ACT_NONE && activation != SAMQ_ACT_GELU) return fail(SAMQ_ERR_BAD_ARG, "unknown activation %d", activation);
    if (a_gran == SAMQ_GRAN_GROUP || w_gran == SAMQ_GRAN_GROUP)
        return fail(SAMQ_ERR_UNSUPPORTED, "grouped scales are handled by the grouped GEMM entry (group_size=%d)", group_size);
    if ((a_gran != SAMQ_GRAN_ROW && a_gran != SAMQ_GRAN_TENSOR) || (w_gran != SAMQ_GRAN_ROW && w_gran != SAMQ_GRAN_TENSOR))
        return fail(SAMQ_ERR_BAD_ARG, "unknown scale granularity");
    if (out_dtype == SAMQ_I32 && (a_scale || w_scale || bias || residual || activation != SAMQ_ACT_NONE))
        return fail(SAMQ_ERR_BAD_ARG, "raw int32 output takes no scales, bias, activation or residual");
    if (residual != nullptr && ldr < N) return fail(SAMQ_ERR_BAD_ARG, "ldr smaller than N");

    CUtensorMap ma, mw;
    int rc = make_operand_map(&ma, A, M, K, lda, BM);
    if (rc != SAMQ_OK) return rc;
    rc = make_operand_map(&mw, W, N, K, ldw, BN);
    if (rc != SAMQ_OK) return rc;

    GemmParams p;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.a_scale = a_scale; p.a_stride = (a_gran == SAMQ_GRAN_ROW) ? 1 : 0;
    p.w_scale = w_scale; p.w_stride = (w_gran == SAMQ_GRAN_ROW) ? 1 : 0;
    p.bias = bias; p.residual = residual; p.ldr = ldr;
    p.out = out; p.ldo = ldo; p.activation = activation; p.status = status;
    const size_t esz = (out_dtype == SAMQ_F16 || out_dtype == SAMQ_BF16) ? 2 : 4;
    p.vec_ok = ((reinterpret_cast<uintptr_t>(out) & 15) == 0) && ((ldo * esz) % 16 == 0) &&
               (residual == nullptr || (((reinterpret_cast<uintptr_t>(residual) & 15) == 0) && ((ldr * esz) % 16 == 0)));
    // the coalesced path: tiles leave through shared memory and TMA stores, which need a 16-byte
    // aligned base and row pitch; anything else takes direct per-thread stores
    CUtensorMap mo;
    memset(&mo, 0, sizeof(mo));
    p.tma_store = 0;
    if (((reinterpret_cast<uintptr_t>(out) & 15) == 0) && ((ldo * esz) % 16 == 0)) {
        rc = make_out_map(&mo, out, M, N, ldo, (int)esz);
        if (rc != SAMQ_OK) return rc;
        p.tma_store = 1;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (out_dtype) {
    case SAMQ_F16:  return launch_gemm<__half>(ma, mw, mo, p, st);
    case SAMQ_BF16: return launch_gemm<__nv_bfloat16>(ma, mw, mo, p, st);
    case SAMQ_F32:  return launch_gemm<float>(ma, mw, mo, p, st);
    case SAMQ_I32:  return launch_gemm<int32_t>(ma, mw, mo, p, st);
    default: return fail(SAMQ_ERR_BAD_ARG, "unknown out_dtype %d", out_dtype);
    }
}

}  // namespace samq
