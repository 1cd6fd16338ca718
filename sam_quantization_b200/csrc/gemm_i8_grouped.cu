// K2 variant for grouped scales: per_group weights
// (quantize_weight_per_group_absmax_input_features, RTN_quantization/per_tensor_channel_group.py:23-50)
// and / or per_group_token activations (:74-93).  The scale changes every `group_size` columns of
// K, so dequantisation cannot wait for the end of the K loop:
//
//   y[m,n] = act( sum_g  float(acc_g[m,n]) * a_scale[m, g] * w_scale[n, g]  + bias[n] ) + residual[m,n]
//   acc_g[m,n] = sum over the K columns of group g of A[m,k] * W[n,k]            (int32, exact)
//
// Same pipeline as gemm_i8_kernel (TMA producer warp, tcgen05.mma issuer warp, 8 epilogue warps,
// every wait bounded).  Tile 128 x 128 with four 128-column TMEM accumulators and six operand stages:
// the MMA warp accumulates one group into the next free accumulator and publishes it; the epilogue
// warps drain it into fp32 registers (64 running sums per thread), scaled by that group's scales,
// while the MMAs of the following groups run.  group_size must be a multiple of 32 (one tcgen05.mma
// covers 32 columns of K; a 128-column stage may hold up to four groups), at most 160 groups per row.
// The weight scales of the next group are fetched into a small per-warp ring in shared memory while the
// current group drains; the int32 -> fp32 conversion is an integer add (exact for groups of up to 256
// columns); a per-token activation scale multiplies the sum once at the end of the tile.
// SAMQ_GROUPED_BN = 256 builds the 128 x 256-tile variant (two accumulators, four stages, 128 running
// sums per thread): it needs a third less operand traffic but measured no faster (0.80 against
// 0.82-0.94 POP/s at group 128), the drain being bound by the latency of the tensor-memory loads, which
// more registers per thread leave less room to overlap.
#include "gemm_common.cuh"

namespace samq {

using namespace sm100;
using namespace gemm;

namespace {

#ifndef SAMQ_GROUPED_BN
#define SAMQ_GROUPED_BN 128
#endif
constexpr int BM = 128;
constexpr int BN = SAMQ_GROUPED_BN;            // 128: four accumulators, six stages; 256: two accumulators, four stages
constexpr int UK = 32;
constexpr int STAGES = BN == 128 ? 6 : 4;
constexpr int A_BYTES = BM * BK;               // 16 KiB
constexpr int B_BYTES = BN * BK;               // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_WARPS = 8;                   // two per TMEM lane quadrant, BN / 2 columns each
constexpr int CPW = BN / 2;                    // accumulator columns per epilogue warp
constexpr int THREADS = 64 + EPI_WARPS * 32;
constexpr int ACC_BUFS = 512 / BN;
constexpr int TMEM_COLS = ACC_BUFS * BN;       // 512
constexpr int MAX_GROUPS = 160;                // K = 5120 in groups of 32
constexpr int STAGING_BYTES = 32 * 64;
constexpr int RING_FLOATS = 2 * CPW;           // per epilogue warp: the weight scales of two consecutive groups

struct __align__(8) Control {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_full[ACC_BUFS];
    uint64_t acc_empty[ACC_BUFS];
    uint32_t tmem_base;
    uint32_t abort_flag;
};

constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES + (size_t)EPI_WARPS * STAGING_BYTES +
                              (size_t)EPI_WARPS * RING_FLOATS * sizeof(float) + (size_t)BN * sizeof(float) + sizeof(Control);

constexpr uint32_t kInstrDesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ void tmem_ld16x(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}

__device__ __forceinline__ void tmem_ld_chunk(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld16x(taddr, r); }
__device__ __forceinline__ void tmem_ld_chunk(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld32(taddr, r); }

struct GroupedParams {
    int M, N, K;
    int groups;                 // K / group_size
    int units_per_group;        // group_size / 32: tcgen05.mma instructions per group
    int a_grouped;              // the activation scale changes with the group
    const float* a_scale; int a_row_stride, a_group_stride;    // a_scale[m * a_row_stride + g * a_group_stride]
    const float* w_scale; int w_row_stride, w_group_stride;
    const void* bias;
    const void* residual; int64_t ldr;
    void* out; int64_t ldo;
    int activation;
    int vec_ok;
    int tma_store;
    int32_t* status;
};

template <typename OutT>
__global__ void __launch_bounds__(THREADS, 1)
gemm_i8_grouped_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                       const __grid_constant__ CUtensorMap map_out, const GroupedParams p)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
    uint8_t* tiles = smem_raw + pad;
    uint8_t* staging = tiles + (size_t)STAGES * STAGE_BYTES;
    float* rings = reinterpret_cast<float*>(staging + (size_t)EPI_WARPS * STAGING_BYTES);     // [EPI_WARPS][2][CPW]
    float* biases = rings + EPI_WARPS * RING_FLOATS;                                           // [BN]
    Control* ctl = reinterpret_cast<Control*>(biases + BN);
    volatile uint32_t* abort_flag = &ctl->abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int m_blocks = (p.M + BM - 1) / BM;
    const int n_blocks = (p.N + BN - 1) / BN;
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
    const int total_units = p.groups * p.units_per_group;          // K / 32
    const int k_blocks = (total_units + BK / UK - 1) / (BK / UK);

    if (warp == 0) {
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
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000LL) { }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            int acc = 0; uint32_t acc_phase = 0;
            bool ok = true;
            // The issuing thread must hand the tensor core an MMA every few tens of clocks, so the common
            // case (groups that are whole 128-column stages) keeps the four MMAs of a stage unrolled and free of
            // bookkeeping; groups of 32, 64 or 96 columns take the step-by-step loop below.
            const bool whole_stages = (p.units_per_group & (BK / UK - 1)) == 0;
            const int kb_per_group = p.units_per_group / (BK / UK);
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                if (whole_stages) {
                    for (int g = 0; g < p.groups && ok; ++g) {
                        if (!mbar_wait(smem_u32(&ctl->acc_empty[acc]), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                        tcgen05_fence_after();
                        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
                        for (int kb = 0; kb < kb_per_group; ++kb) {
                            if (!mbar_wait(smem_u32(&ctl->full[stage]), phase, abort_flag)) { ok = false; break; }
                            tcgen05_fence_after();
                            const uint32_t sa = smem_u32(tiles + (size_t)stage * STAGE_BYTES);
                            const uint64_t adesc = make_smem_desc(sa);
                            const uint64_t bdesc = make_smem_desc(sa + A_BYTES);
#pragma unroll
                            for (int k = 0; k < BK / UK; ++k)
                                mma_i8(tmem_d, adesc + (uint64_t)(k * (UK >> 4)), bdesc + (uint64_t)(k * (UK >> 4)),
                                       kInstrDesc, (kb | k) != 0 ? 1u : 0u);
                            tcgen05_commit(smem_u32(&ctl->empty[stage]));
                            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                        }
                        if (!ok) break;
                        tcgen05_commit(smem_u32(&ctl->acc_full[acc]));       // this group's partial sums are complete
                        if (++acc == ACC_BUFS) { acc = 0; acc_phase ^= 1u; }
                    }
                    continue;
                }
                int unit = 0;                                   // 32-column steps of K issued for this tile
                uint64_t adesc = 0, bdesc = 0;
                for (int g = 0; g < p.groups && ok; ++g) {
                    if (!mbar_wait(smem_u32(&ctl->acc_empty[acc]), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
                    for (int u = 0; u < p.units_per_group; ++u) {
                        const int k = unit & (BK / UK - 1);
                        if (k == 0) {                            // first step of a stage: its operands must have landed
                            if (!mbar_wait(smem_u32(&ctl->full[stage]), phase, abort_flag)) { ok = false; break; }
                            tcgen05_fence_after();
                            const uint32_t sa = smem_u32(tiles + (size_t)stage * STAGE_BYTES);
                            adesc = make_smem_desc(sa);
                            bdesc = make_smem_desc(sa + A_BYTES);
                        }
                        mma_i8(tmem_d, adesc + (uint64_t)(k * (UK >> 4)), bdesc + (uint64_t)(k * (UK >> 4)), kInstrDesc, u != 0 ? 1u : 0u);
                        ++unit;
                        if ((unit & (BK / UK - 1)) == 0 || unit == total_units) {   // last step that reads this stage
                            tcgen05_commit(smem_u32(&ctl->empty[stage]));
                            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                        }
                    }
                    if (!ok) break;
                    tcgen05_commit(smem_u32(&ctl->acc_full[acc]));       // this group's partial sums are complete
                    if (++acc == ACC_BUFS) { acc = 0; acc_phase ^= 1u; }
                }
            }
        }
    } else {
        const int ew = warp - 2;
        const int quad = warp & 3;
        const int half_n = ew >> 2;               // which half of the tile's columns
        const int epi_tid = threadIdx.x - 64;
        int acc = 0; uint32_t acc_phase = 0;
        bool ok = true;
        const uint32_t stage_addr = smem_u32(staging + (size_t)ew * STAGING_BYTES);
        uint8_t* stage_ptr = staging + (size_t)ew * STAGING_BYTES;
        float* ring = rings + ew * RING_FLOATS;
        const uint32_t swz = (uint32_t)((lane >> 1) & 3);
        const bool magic_ok = p.units_per_group <= 8;     // |acc| < 2^22: the integer-add conversion is exact
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
            const int m0 = (tile / n_blocks) * BM;
            const int n0 = (tile % n_blocks) * BN;
            // the bias of this tile; the first barrier keeps slow warps of the previous tile from seeing it change
            asm volatile("bar.sync 1, %0;" ::"r"(EPI_WARPS * 32) : "memory");
            if (epi_tid < BN) {
                const int n = n0 + epi_tid;
                biases[epi_tid] = (n < p.N && p.bias != nullptr) ? OutOps<OutT>::up(reinterpret_cast<const OutT*>(p.bias)[n]) : 0.f;
            }
            asm volatile("bar.sync 1, %0;" ::"r"(EPI_WARPS * 32) : "memory");

            const int row = m0 + quad * 32 + lane;
            const bool row_ok = row < p.M;
            // weight scales of group g for this warp's columns: lane l fetches columns l, l+32, ...
            auto fetch_w = [&](int g, float (&w)[CPW / 32]) {
#pragma unroll
                for (int i = 0; i < CPW / 32; ++i) {
                    const int n = n0 + half_n * CPW + i * 32 + lane;
                    w[i] = (n < p.N && p.w_scale != nullptr) ? p.w_scale[(int64_t)n * p.w_row_stride + (int64_t)g * p.w_group_stride] : 1.0f;
                }
            };
            {
                float w0[CPW / 32];
                fetch_w(0, w0);
                __syncwarp();
#pragma unroll
                for (int i = 0; i < CPW / 32; ++i) ring[i * 32 + lane] = w0[i];
                __syncwarp();
            }
            float2 y2[CPW / 2];
#pragma unroll
            for (int j = 0; j < CPW / 2; ++j) y2[j] = make_float2(0.f, 0.f);
            // a per-token (or per-tensor) activation scale is the same for every group: it multiplies the sum once
            float a_row = 1.0f;
            if (!p.a_grouped && p.a_scale != nullptr && row_ok) a_row = p.a_scale[(int64_t)row * p.a_row_stride];
            float a_s = 1.0f;
            if (p.a_grouped && p.a_scale != nullptr && row_ok) a_s = p.a_scale[(int64_t)row * p.a_row_stride];
            for (int g = 0; g < p.groups; ++g) {
                // next group's scales travel while this group drains
                float wn[CPW / 32];
#pragma unroll
                for (int i = 0; i < CPW / 32; ++i) wn[i] = 1.f;
                float a_next = 1.0f;
                if (g + 1 < p.groups) {
                    fetch_w(g + 1, wn);
                    if (p.a_grouped && p.a_scale != nullptr && row_ok) a_next = p.a_scale[(int64_t)row * p.a_row_stride + (int64_t)(g + 1) * p.a_group_stride];
                }
                if (ok && !mbar_wait(smem_u32(&ctl->acc_full[acc]), acc_phase, abort_flag)) ok = false;
                if (!ok) break;
                tcgen05_fence_after();
                const float2 a2 = make_float2(a_s, a_s);
                const uint32_t tmem_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN + half_n * CPW);
                const float* ws = ring + (g & 1) * CPW;
                const float2 k2 = make_float2(-12582912.0f, -12582912.0f);
                // 64 columns per warp: two 32-column loads; 128 columns per warp: eight 16-column loads (register budget)
                constexpr int CH = CPW == 64 ? 32 : 16;
#pragma unroll
                for (int c = 0; c < CPW / CH; ++c) {
                    uint32_t r[CH];
                    tmem_ld_chunk(tmem_row + (uint32_t)(c * CH), r);
                    tmem_ld_wait();
                    if (c == CPW / CH - 1) {                    // the accumulator is in registers: hand the buffer back
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&ctl->acc_empty[acc]));
                    }
#pragma unroll
                    for (int j = 0; j < CH; j += 4) {
                        const float4 w4 = *reinterpret_cast<const float4*>(ws + c * CH + j);
                        float2 wlo = make_float2(w4.x, w4.y), whi = make_float2(w4.z, w4.w);
                        if (p.a_grouped) { wlo = __fmul2_rn(wlo, a2); whi = __fmul2_rn(whi, a2); }
                        float2 flo, fhi;
                        if (magic_ok) {
                            // 1.5 * 2^23 + acc is exact in fp32 and its bit pattern is 0x4B400000 + acc
                            flo = __fadd2_rn(make_float2(__uint_as_float(r[j + 0] + 0x4B400000u), __uint_as_float(r[j + 1] + 0x4B400000u)), k2);
                            fhi = __fadd2_rn(make_float2(__uint_as_float(r[j + 2] + 0x4B400000u), __uint_as_float(r[j + 3] + 0x4B400000u)), k2);
                        } else {
                            flo = make_float2(__int2float_rn((int)r[j + 0]), __int2float_rn((int)r[j + 1]));
                            fhi = make_float2(__int2float_rn((int)r[j + 2]), __int2float_rn((int)r[j + 3]));
                        }
                        const int q = (c * CH + j) >> 1;
                        y2[q] = __ffma2_rn(flo, wlo, y2[q]);
                        y2[q + 1] = __ffma2_rn(fhi, whi, y2[q + 1]);
                    }
                }
                if (++acc == ACC_BUFS) { acc = 0; acc_phase ^= 1u; }
                // publish the next group's weight scales (every lane has finished reading this group's)
                __syncwarp();
#pragma unroll
                for (int i = 0; i < CPW / 32; ++i) ring[((g + 1) & 1) * CPW + i * 32 + lane] = wn[i];
                __syncwarp();
                a_s = a_next;
            }
            if (!ok) continue;                       // keep visiting the named barriers

            // ---- finish the tile: bias, activation, residual, store ----
#pragma unroll
            for (int c = 0; c < CPW / 32; ++c) {
                const int col0 = half_n * CPW + c * 32;
                const int n_first = n0 + col0;
                if (n_first >= p.N) continue;
                const int n_valid = min(32, p.N - n_first);
                constexpr int PER16 = 16 / (int)sizeof(OutT);
                constexpr int NVEC = 32 / PER16;
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    const float2 t = y2[(c * 32 + j) >> 1];
                    v[j] = fmaf(t.x, a_row, biases[col0 + j]);
                    v[j + 1] = fmaf(t.y, a_row, biases[col0 + j + 1]);
                }
                if (p.activation == SAMQ_ACT_GELU) gelu32(v);
                if (p.residual != nullptr && row_ok) {
                    const OutT* res = reinterpret_cast<const OutT*>(p.residual) + (int64_t)row * p.ldr + n_first;
                    if (p.vec_ok && n_valid == 32) {
#pragma unroll
                        for (int j = 0; j < NVEC; ++j) {
                            OutT tmp[PER16];
                            *reinterpret_cast<uint4*>(tmp) = *reinterpret_cast<const uint4*>(res + j * PER16);
#pragma unroll
                            for (int e = 0; e < PER16; ++e) v[j * PER16 + e] += OutOps<OutT>::up(tmp[e]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) if (j < n_valid) v[j] += OutOps<OutT>::up(res[j]);
                    }
                }
                uint4 packed[NVEC];
                OutOps<OutT>::pack32(v, packed);
                if (p.tma_store) {
#pragma unroll
                    for (int part = 0; part < NVEC / 4; ++part) {
                        if (lane == 0) bulk_wait_read0();
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
                    const OutT* src = reinterpret_cast<const OutT*>(packed);
#pragma unroll
                    for (int j = 0; j < 32; ++j) if (j < n_valid) o[j] = src[j];
                }
            }
        }
    }

    if (warp >= 2 && lane == 0 && p.tma_store) bulk_wait0();
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && ctl->abort_flag != 0 && p.status != nullptr) atomicExch(p.status, 1);
}

template <typename OutT>
int launch_grouped(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mo, const GroupedParams& p, cudaStream_t st) {
    SAMQ_CUDA_TRY(cudaFuncSetAttribute(gemm_i8_grouped_kernel<OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
    const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
    const int grid = tiles < sm_count() ? tiles : sm_count();
    gemm_i8_grouped_kernel<OutT><<<grid, THREADS, SMEM_BYTES, st>>>(ma, mw, mo, p);
    SAMQ_CUDA_TRY(cudaGetLastError());
    return SAMQ_OK;
}

}  // namespace

int gemm_i8_grouped_dispatch(const int8_t* A, int64_t lda, const int8_t* W, int64_t ldw,
                             int64_t M, int64_t N, int64_t K,
                             const float* a_scale, int a_gran, const float* w_scale, int w_gran, int group_size,
                             const void* bias, const void* residual, int64_t ldr, int activation,
                             void* out, int out_dtype, int64_t ldo, int32_t* status, void* stream)
{
    if (M < 0 || N <= 0 || K <= 0) return fail(SAMQ_ERR_BAD_ARG, "bad GEMM shape M=%lld N=%lld K=%lld",
                                               (long long)M, (long long)N, (long long)K);
    if (M == 0) return SAMQ_OK;
    if (A == nullptr || W == nullptr || out == nullptr) return fail(SAMQ_ERR_BAD_ARG, "A, W and out must not be null");
    if (group_size <= 0 || K % group_size != 0) return fail(SAMQ_ERR_BAD_ARG, "group_size %d must divide K=%lld", group_size, (long long)K);
    if (group_size % UK != 0)
        return fail(SAMQ_ERR_UNSUPPORTED, "the grouped GEMM needs group_size to be a multiple of %d (got %d)", UK, group_size);
    const int64_t groups = K / group_size;
    if (groups > MAX_GROUPS) return fail(SAMQ_ERR_TOO_LARGE, "K / group_size = %lld exceeds %d groups", (long long)groups, MAX_GROUPS);
    if (M > 2147483647LL - BM || N > 2147483647LL - BN) return fail(SAMQ_ERR_TOO_LARGE, "GEMM dimension exceeds 2^31");
    if (lda < K || ldw < K || ldo < N) return fail(SAMQ_ERR_BAD_ARG, "leading dimension smaller than the row");
    if ((lda & 15) || (ldw & 15) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
        return fail(SAMQ_ERR_ALIGNMENT, "A and W need 16-byte aligned bases and row strides (lda=%lld ldw=%lld)",
                    (long long)lda, (long long)ldw);
    if (activation != SAMQ_ACT_NONE && activation != SAMQ_ACT_GELU) return fail(SAMQ_ERR_BAD_ARG, "unknown activation %d", activation);
    if (out_dtype == SAMQ_I32) return fail(SAMQ_ERR_UNSUPPORTED, "raw int32 output is not defined for grouped scales");
    if (residual != nullptr && ldr < N) return fail(SAMQ_ERR_BAD_ARG, "ldr smaller than N");

    CUtensorMap ma, mw, mo;
    int rc = make_operand_map(&ma, A, M, K, lda, BM);
    if (rc != SAMQ_OK) return rc;
    rc = make_operand_map(&mw, W, N, K, ldw, BN);
    if (rc != SAMQ_OK) return rc;

    GroupedParams p;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.groups = (int)groups; p.units_per_group = group_size / UK;
    p.a_grouped = (a_gran == SAMQ_GRAN_GROUP) ? 1 : 0;
    p.a_scale = a_scale; p.w_scale = w_scale;
    p.a_row_stride = (a_gran == SAMQ_GRAN_GROUP) ? (int)groups : (a_gran == SAMQ_GRAN_ROW ? 1 : 0);
    p.a_group_stride = (a_gran == SAMQ_GRAN_GROUP) ? 1 : 0;
    p.w_row_stride = (w_gran == SAMQ_GRAN_GROUP) ? (int)groups : (w_gran == SAMQ_GRAN_ROW ? 1 : 0);
    p.w_group_stride = (w_gran == SAMQ_GRAN_GROUP) ? 1 : 0;
    p.bias = bias; p.residual = residual; p.ldr = ldr;
    p.out = out; p.ldo = ldo; p.activation = activation; p.status = status;
    const size_t esz = (out_dtype == SAMQ_F16 || out_dtype == SAMQ_BF16) ? 2 : 4;
    p.vec_ok = (((reinterpret_cast<uintptr_t>(out) & 15) == 0) && ((ldo * esz) % 16 == 0) &&
                (residual == nullptr || (((reinterpret_cast<uintptr_t>(residual) & 15) == 0) && ((ldr * esz) % 16 == 0)))) ? 1 : 0;
    memset(&mo, 0, sizeof(mo));
    p.tma_store = 0;
    if (((reinterpret_cast<uintptr_t>(out) & 15) == 0) && ((ldo * esz) % 16 == 0)) {
        rc = make_out_map(&mo, out, M, N, ldo, (int)esz);
        if (rc != SAMQ_OK) return rc;
        p.tma_store = 1;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (out_dtype) {
    case SAMQ_F16:  return launch_grouped<__half>(ma, mw, mo, p, st);
    case SAMQ_BF16: return launch_grouped<__nv_bfloat16>(ma, mw, mo, p, st);
    case SAMQ_F32:  return launch_grouped<float>(ma, mw, mo, p, st);
    default: return fail(SAMQ_ERR_BAD_ARG, "unknown out_dtype %d", out_dtype);
    }
}

}  // namespace samq
