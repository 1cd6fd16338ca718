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
#include <cuda.h>
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
constexpr long long WAIT_LIMIT_CYCLES = 4000000000LL;   // about 2 s

struct __align__(8) Control {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_full[ACC_BUFS];
    uint64_t acc_empty[ACC_BUFS];
    uint32_t tmem_base;
    uint32_t abort_flag;
};

constexpr int EPI_PARAM_FLOATS = ACC_BUFS * 2 * BN;      // w_scale and bias per accumulator buffer
constexpr size_t SMEM_BYTES = 1024 /*alignment slack*/ + (size_t)STAGES * STAGE_BYTES +
                              EPI_PARAM_FLOATS * sizeof(float) + sizeof(Control);

// ---- PTX wrappers ------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait. Returns false when the limit ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 255u) == 0) {
            if (*abort_flag != 0) return false;
            if (clock64() - t0 > WAIT_LIMIT_CYCLES) { *abort_flag = 1; return false; }
        }
    }
    return true;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after()  { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for a K-major operand tile whose rows are 128 bytes wide and
// stored with the 128-byte swizzle (what TMA writes with CU_TENSOR_MAP_SWIZZLE_128B):
// start address >> 4 in bits [0,14); leading byte offset (unused for this layout) = 1 in [16,30);
// stride byte offset = 1024 B (8 rows) >> 4 in [32,46); descriptor version 1 in [46,48);
// layout type 2 (128-byte swizzle) in [61,64).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    uint64_t d = (uint64_t)((smem_addr >> 4) & 0x3FFFu);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor for kind::i8: D = S32 (2) in bits [4,6); A, B = signed 8-bit (1) in
// [7,10) and [10,13); both operands K-major (bits 15, 16 = 0); N >> 3 in [17,23); M >> 4 in [24,29).
constexpr uint32_t kInstrDesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f)); }

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
    int32_t* status;
};

// OutT = __half | __nv_bfloat16 | float | int32_t (raw accumulators)
template <typename OutT>
__global__ void __launch_bounds__(THREADS, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const GemmParams p)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
    uint8_t* tiles = smem_raw + pad;                                   // 1024-byte aligned
    float* epi_params = reinterpret_cast<float*>(tiles + (size_t)STAGES * STAGE_BYTES);
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
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                const int col0 = half_n * 128 + c * 32;
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN + col0), r);
                tmem_ld_wait();
                const int n_first = n0 + col0;
                if (!row_ok || n_first >= p.N) continue;
                const int n_valid = min(32, p.N - n_first);
                if constexpr (std::is_same<OutT, int32_t>::value) {
                    int32_t* o = reinterpret_cast<int32_t*>(p.out) + (int64_t)row * p.ldo + n_first;
                    if (p.vec_ok && n_valid == 32) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            reinterpret_cast<uint4*>(o)[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) if (j < n_valid) o[j] = (int32_t)r[j];
                    }
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
                    OutT* o = reinterpret_cast<OutT*>(p.out) + (int64_t)row * p.ldo + n_first;
                    const OutT* res = p.residual != nullptr
                        ? reinterpret_cast<const OutT*>(p.residual) + (int64_t)row * p.ldr + n_first : nullptr;
                    constexpr int PER16 = 16 / (int)sizeof(OutT);
                    if (p.vec_ok && n_valid == 32) {
#pragma unroll
                        for (int j = 0; j < 32; j += PER16) {
                            OutT tmp[PER16];
                            if (res != nullptr) {
                                *reinterpret_cast<uint4*>(tmp) = *reinterpret_cast<const uint4*>(res + j);
#pragma unroll
                                for (int e = 0; e < PER16; ++e) y[j + e] += OutOps<OutT>::up(tmp[e]);
                            }
#pragma unroll
                            for (int e = 0; e < PER16; ++e) tmp[e] = OutOps<OutT>::down(y[j + e]);
                            *reinterpret_cast<uint4*>(o + j) = *reinterpret_cast<const uint4*>(tmp);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (j < n_valid) {
                                float v = y[j];
                                if (res != nullptr) v += OutOps<OutT>::up(res[j]);
                                o[j] = OutOps<OutT>::down(v);
                            }
                        }
                    }
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctl->acc_empty[acc]));
            if (++acc == ACC_BUFS) { acc = 0; acc_phase ^= 1u; }
        }
    }

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

template <typename OutT>
int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mw, const GemmParams& p, cudaStream_t st) {
    SAMQ_CUDA_TRY(cudaFuncSetAttribute(gemm_i8_kernel<OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
    const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
    const int grid = tiles < sm_count() ? tiles : sm_count();
    gemm_i8_kernel<OutT><<<grid, THREADS, SMEM_BYTES, st>>>(ma, mw, p);
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
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (out_dtype) {
    case SAMQ_F16:  return launch_gemm<__half>(ma, mw, p, st);
    case SAMQ_BF16: return launch_gemm<__nv_bfloat16>(ma, mw, p, st);
    case SAMQ_F32:  return launch_gemm<float>(ma, mw, p, st);
    case SAMQ_I32:  return launch_gemm<int32_t>(ma, mw, p, st);
    default: return fail(SAMQ_ERR_BAD_ARG, "unknown out_dtype %d", out_dtype);
    }
}

}  // namespace samq
