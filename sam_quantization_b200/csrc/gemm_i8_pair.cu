// K2 on CTA pairs: the same W8A8 GEMM + fused epilogue as gemm_i8.cu, with two CTAs of a
// thread-block cluster sharing every W tile (tcgen05 cta_group::2).
//
// A pair owns a 256 x 256 output tile.  Each CTA loads its own 128 rows of A and only HALF of the
// W tile (128 of its 256 rows) per 128-byte k-block — 32 KiB per stage instead of 48, six stages —
// and the leader CTA issues tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 32), which reads A and
// W from both CTAs' shared memory and leaves each CTA's 128 x 256 int32 accumulator in its own
// tensor memory.  Per SM the operand traffic from L2 drops by a third, which is what limits the
// single-CTA kernel on its long-K shapes.  No load is multicast: every CTA fetches exactly the
// bytes it stores.  Barriers: the leader's `full` barrier counts the bytes of both CTAs' loads;
// MMA completion is committed to the `empty` / `acc_full` barriers of both CTAs; both CTAs'
// epilogue warps report to the leader's `acc_empty` barrier.  Every wait is bounded as in gemm_i8.cu.
#include "gemm_common.cuh"

namespace samq {

using namespace sm100;
using namespace gemm;

namespace {

constexpr int BM = 128;            // rows of A per tile   (UMMA M)
constexpr int BN = 256;            // rows of W per tile   (UMMA N)
constexpr int UK = 32;             // K of one tcgen05.mma for 8-bit operands
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK;   // 16 KiB
constexpr int BNH = BN / 2;         // rows of W each CTA of the pair loads
constexpr int B_BYTES = BNH * BK;  // 16 KiB
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


// Instruction descriptor for kind::i8: D = S32 (2) in bits [4,6); A, B = signed 8-bit (1) in
// [7,10) and [10,13); both operands K-major (bits 15, 16 = 0); N >> 3 in [17,23); M >> 4 in [24,29).
constexpr uint32_t kInstrDesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);

struct PairParams {
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

// OutT = __half | __nv_bfloat16 | float | int32_t (raw accumulators); GELU / RES compile the
// activation and the residual add in or out of the epilogue
template <typename OutT, bool GELU, bool RES>
__global__ void __launch_bounds__(THREADS, 1)
gemm_i8_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_out, const PairParams p)
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
    const uint32_t rank = cluster_ctarank();                         // 0 = leader of the pair
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int m_blocks = (p.M + 2 * BM - 1) / (2 * BM);               // 256-row tiles, one per pair
    const int n_blocks = (p.N + BN - 1) / BN;
    const int k_blocks = (p.K + BK - 1) / BK;
    const int num_tiles = m_blocks * n_blocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(smem_u32(&ctl->full[s]), 1); mbar_init(smem_u32(&ctl->empty[s]), 1); }
        for (int b = 0; b < ACC_BUFS; ++b) { mbar_init(smem_u32(&ctl->acc_full[b]), 1); mbar_init(smem_u32(&ctl->acc_empty[b]), 2 * EPI_WARPS); }
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        if (p.tma_store) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_out) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&ctl->tmem_base)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();                                                  // both CTAs' barriers exist before any remote arrival
    tcgen05_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
                const int m0 = (tile / n_blocks) * (2 * BM) + (int)rank * BM;     // this CTA's rows of A
                const int n0 = (tile % n_blocks) * BN + (int)rank * BNH;          // this CTA's rows of W
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort_flag)) { ok = false; break; }
                    const uint32_t bar = smem_u32(&ctl->full[stage]);
                    const uint32_t leader_bar = map_to_cta(bar, 0);
                    const uint32_t sa = smem_u32(tiles + (size_t)stage * STAGE_BYTES);
                    if (rank == 0) mbar_expect_tx(bar, 2 * STAGE_BYTES);          // bytes of both CTAs
                    tma_load_2d_pair(sa, &map_a, leader_bar, kb * BK, m0);
                    tma_load_2d_pair(sa + A_BYTES, &map_w, leader_bar, kb * BK, n0);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            // every stage has been handed back: no completion from the leader's MMA thread can
            // still be on its way to this CTA's barriers when the CTA retires
            for (int s = 0; s < STAGES && ok; ++s) {
                if (!mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort_flag)) ok = false;
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (!ok) {
                // let copies that are already in flight land before the CTA retires
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000LL) { }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0 && rank == 0) {
            int stage = 0; uint32_t phase = 0;
            int acc = 0; uint32_t acc_phase = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
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
                        mma_i8_pair(tmem_d, adesc + (uint64_t)(k * (UK >> 4)), bdesc + (uint64_t)(k * (UK >> 4)),
                                    kInstrDesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    // frees the stage in both CTAs when the MMAs retire
                    tcgen05_commit_pair(map_to_cta(smem_u32(&ctl->empty[stage]), 0));
                    tcgen05_commit_pair(map_to_cta(smem_u32(&ctl->empty[stage]), 1));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                tcgen05_commit_pair(map_to_cta(smem_u32(&ctl->acc_full[acc]), 0));   // accumulators complete in both CTAs
                tcgen05_commit_pair(map_to_cta(smem_u32(&ctl->acc_full[acc]), 1));
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
        for (int tile = pair; tile < num_tiles; tile += num_pairs) {
            const int m0 = (tile / n_blocks) * (2 * BM) + (int)rank * BM;
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
            if constexpr (RES) {
                // pull this warp's 32 x 128 residual block towards L2 while the MMAs of the tile run
                const int prow = m0 + quad * 32 + lane;
                if (prow < p.M) {
                    const char* rp = reinterpret_cast<const char*>(p.residual) +
                                     ((int64_t)prow * p.ldr + n0 + half_n * 128) * (int64_t)sizeof(OutT);
#pragma unroll
                    for (int b = 0; b < (int)(128 * sizeof(OutT)); b += 128)
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(rp + b));
                }
            }
            // the row's activation scale does not depend on the accumulator: fetch it before waiting for the MMAs
            const int row = m0 + quad * 32 + lane;
            const bool row_ok = row < p.M;
            float a_s = 1.0f;
            if constexpr (!std::is_same<OutT, int32_t>::value) {
                if (p.a_scale != nullptr && row_ok) a_s = p.a_scale[(int64_t)row * p.a_stride];
            }
            // after a failed wait keep visiting the named barrier above so no warp is left behind
            if (ok && !mbar_wait(smem_u32(&ctl->acc_full[acc]), acc_phase, abort_flag)) ok = false;
            if (!ok) continue;
            tcgen05_fence_after();
            const uint32_t stage_addr = smem_u32(staging + (size_t)ew * STAGING_BYTES);
            uint8_t* stage_ptr = staging + (size_t)ew * STAGING_BYTES;
            const int rr = quad * 32 + lane;                       // row inside the tile
            const uint32_t swz = (uint32_t)((lane >> 1) & 3);     // 64-byte swizzle: 16-byte slot ^= bits [7:8] of the offset
            // The accumulator is read 32 columns at a time; the load of chunk c+1 is in flight while
            // chunk c is dequantised and stored, and the buffer is handed back to the MMA warp as soon
            // as the last chunk sits in registers.
            const uint32_t tmem_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN + half_n * 128);
            uint32_t rbuf[2][32];
            tmem_ld32(tmem_row, rbuf[0]);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int col0 = half_n * 128 + c * 32;
                uint32_t (&r)[32] = rbuf[c & 1];
                tmem_ld_wait();
                if (c + 1 < 4) {
                    tmem_ld32(tmem_row + (uint32_t)((c + 1) * 32), rbuf[(c + 1) & 1]);
                } else {
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&ctl->acc_empty[acc]), 0));   // the leader's barrier
                }
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
                    dequant32(r, a_s, ws + col0, bs + col0, y);
                    if constexpr (GELU) gelu32(y);
                    if constexpr (RES) {
                        const OutT* res_base = reinterpret_cast<const OutT*>(p.residual);
                        if (p.tma_store && p.vec_ok && n_valid == 32) {
                            // coalesced: the warp reads its 32 x 32 residual block row-segment by
                            // row-segment (16 bytes per lane, whole rows per instruction group), parks
                            // it in the staging buffer in the swizzled layout, and every lane then
                            // picks up its own row from there
                            constexpr int SEG = 32 / PER16;                      // 16-byte segments per row: 4 or 8
                            constexpr int ROWS_PER_LD = 32 / SEG;                // rows covered by one warp-wide load
                            uint4 seg[SEG];
#pragma unroll
                            for (int k = 0; k < SEG; ++k) {
                                const int rrow = k * ROWS_PER_LD + lane / SEG;
                                const int grow = m0 + quad * 32 + rrow;
                                seg[k] = grow < p.M
                                    ? *reinterpret_cast<const uint4*>(res_base + (int64_t)grow * p.ldr + n_first + (lane % SEG) * PER16)
                                    : make_uint4(0, 0, 0, 0);
                            }
                            if (lane == 0) bulk_wait_read0();                    // staging is free again
                            __syncwarp();
#pragma unroll
                            for (int part = 0; part < SEG / 4; ++part) {
                                // a staging pass holds 64 bytes per row: all of a 2-byte row, half of a 4-byte row
#pragma unroll
                                for (int k = 0; k < SEG; ++k) {
                                    const int rrow = k * ROWS_PER_LD + lane / SEG;
                                    const int sg = lane % SEG;
                                    if (sg / 4 == part)
                                        *reinterpret_cast<uint4*>(stage_ptr + rrow * 64 +
                                            ((((uint32_t)(sg & 3)) ^ (uint32_t)((rrow >> 1) & 3)) << 4)) = seg[k];
                                }
                                __syncwarp();
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    OutT tmp[PER16];
                                    *reinterpret_cast<uint4*>(tmp) = *reinterpret_cast<const uint4*>(stage_ptr + lane * 64 + (((uint32_t)j ^ swz) << 4));
#pragma unroll
                                    for (int e = 0; e < PER16; ++e) y[(part * 4 + j) * PER16 + e] += OutOps<OutT>::up(tmp[e]);
                                }
                                __syncwarp();
                            }
                        } else if (row_ok) {
                            const OutT* res = res_base + (int64_t)row * p.ldr + n_first;
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
                    }
                    OutOps<OutT>::pack32(y, packed);
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
            if (++acc == ACC_BUFS) { acc = 0; acc_phase ^= 1u; }
        }
    }

    if (warp >= 2 && lane == 0 && p.tma_store) bulk_wait0();          // this thread's TMA stores have completed
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    __syncwarp();
    cluster_sync();                                   // no remote arrival or MMA read of the peer is still in flight
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && ctl->abort_flag != 0 && p.status != nullptr) atomicExch(p.status, 1);
}

template <typename OutT, bool GELU, bool RES>
int launch_gemm_variant(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mo, const PairParams& p, cudaStream_t st) {
    auto kernel = gemm_i8_pair_kernel<OutT, GELU, RES>;
    SAMQ_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
    const int tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + BN - 1) / BN);
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(THREADS); cfg.dynamicSmemBytes = SMEM_BYTES; cfg.stream = st;
    cfg.attrs = attr; cfg.numAttrs = 1;
    // how many pairs the device can hold at once (GPCs with an odd number of SMs leave one out)
    static thread_local int pairs_cached[64] = {0};
    int dev = 0;
    SAMQ_CUDA_TRY(cudaGetDevice(&dev));
    int max_pairs = (dev >= 0 && dev < 64) ? pairs_cached[dev] : 0;
    if (max_pairs == 0) {
        cfg.gridDim = dim3(2 * (sm_count() / 2));
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) { (void)cudaGetLastError(); n = sm_count() / 2 - 4; }
        max_pairs = n;
        if (dev >= 0 && dev < 64) pairs_cached[dev] = n;
    }
    const int pairs = tiles < max_pairs ? tiles : max_pairs;
    cfg.gridDim = dim3(2 * pairs);
    SAMQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, ma, mw, mo, p));
    return SAMQ_OK;
}

template <typename OutT>
int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mo, const PairParams& p, cudaStream_t st) {
    if constexpr (std::is_same<OutT, int32_t>::value) {
        return launch_gemm_variant<OutT, false, false>(ma, mw, mo, p, st);
    } else {
        const bool gelu = p.activation == SAMQ_ACT_GELU, res = p.residual != nullptr;
        if (gelu && res) return launch_gemm_variant<OutT, true, true>(ma, mw, mo, p, st);
        if (gelu) return launch_gemm_variant<OutT, true, false>(ma, mw, mo, p, st);
        if (res) return launch_gemm_variant<OutT, false, true>(ma, mw, mo, p, st);
        return launch_gemm_variant<OutT, false, false>(ma, mw, mo, p, st);
    }
}

}  // namespace

int gemm_i8_pair_dispatch(const int8_t* A, int64_t lda, const int8_t* W, int64_t ldw,
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
    rc = make_operand_map(&mw, W, N, K, ldw, BNH);
    if (rc != SAMQ_OK) return rc;

    PairParams p;
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
