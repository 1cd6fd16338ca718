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
#include "gemm_common.cuh"

namespace samq {

using namespace sm100;
using namespace gemm;

namespace {

constexpr int BM = 128;            // rows of A per tile   (UMMA M)
constexpr int BN = 256;            // rows of W per tile   (UMMA N)
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


// Instruction descriptor for kind::i8: D = S32 (2) in bits [4,6); A, B = signed 8-bit (1) in
// [7,10) and [10,13); both operands K-major (bits 15, 16 = 0); N >> 3 in [17,23); M >> 4 in [24,29).
constexpr uint32_t kInstrDesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

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
    long long wait_limit;                      // cycles a pipeline wait may take before the kernel gives up
    int skip_kblock;                           // self-test only: the producer never loads this k-block of its first tile (-1: none)
};

// OutT = __half | __nv_bfloat16 | float | int32_t (raw accumulators); GELU / RES compile the
// activation and the residual add in or out of the epilogue
template <typename OutT, bool GELU, bool RES>
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
                    if (!mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort_flag, p.wait_limit)) { ok = false; break; }
                    const uint32_t bar = smem_u32(&ctl->full[stage]);
                    const uint32_t sa = smem_u32(tiles + (size_t)stage * STAGE_BYTES);
                    if (!(kb == p.skip_kblock && tile == (int)blockIdx.x)) {      // the self-test leaves one stage unfilled
                        mbar_expect_tx(bar, STAGE_BYTES);
                        tma_load_2d(sa, &map_a, bar, kb * BK, m0);
                        tma_load_2d(sa + A_BYTES, &map_w, bar, kb * BK, n0);
                    }
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
                if (!mbar_wait(smem_u32(&ctl->acc_empty[acc]), acc_phase ^ 1u, abort_flag, p.wait_limit)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(smem_u32(&ctl->full[stage]), phase, abort_flag, p.wait_limit)) { ok = false; break; }
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
            // the row's activation scale does not depend on the accumulator: fetch it before waiting for the
            // MMAs, so that its latency is not added to the epilogue (a warp issues in order)
            const int row = m0 + quad * 32 + lane;
            const bool row_ok = row < p.M;
            float a_s = 1.0f;
            if constexpr (!std::is_same<OutT, int32_t>::value) {
                if (p.a_scale != nullptr && row_ok) a_s = p.a_scale[(int64_t)row * p.a_stride];
            }
            // The residual block of a 32-column chunk is read coalesced (16 bytes per lane, whole row segments
            // per instruction group) one chunk ahead of its use: chunk 0 before the wait for the MMAs, chunk
            // c + 1 while chunk c is dequantised, so that the L2 latency is never on the epilogue's path.
            constexpr int PER16_R = 16 / (int)sizeof(OutT);         // elements per 16-byte vector
            constexpr int SEG = 32 / PER16_R;                       // 16-byte segments per 32-column row: 4 or 8
            constexpr int ROWS_PER_LD = 32 / SEG;                   // rows covered by one warp-wide load
            constexpr int NSEG = RES ? SEG : 1;
            uint4 seg[2][NSEG];
            auto res_chunk_fast = [&](int c) -> bool {              // warp-uniform: the chunk takes the coalesced route
                return p.tma_store && p.vec_ok && n0 + half_n * 128 + c * 32 + 32 <= p.N;
            };
            auto load_res = [&](int c, uint4 (&sg)[NSEG]) {
                const OutT* res_base = reinterpret_cast<const OutT*>(p.residual);
                const int n_first = n0 + half_n * 128 + c * 32;
#pragma unroll
                for (int k = 0; k < NSEG; ++k) {
                    const int grow = m0 + quad * 32 + k * ROWS_PER_LD + lane / SEG;
                    sg[k] = grow < p.M
                        ? *reinterpret_cast<const uint4*>(res_base + (int64_t)grow * p.ldr + n_first + (lane % SEG) * PER16_R)
                        : make_uint4(0, 0, 0, 0);
                }
            };
            if constexpr (RES) {
                if (res_chunk_fast(0)) load_res(0, seg[0]);
            }
            // after a failed wait keep visiting the named barrier above so no warp is left behind
            if (ok && !mbar_wait(smem_u32(&ctl->acc_full[acc]), acc_phase, abort_flag, p.wait_limit)) ok = false;
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
                    if constexpr (RES) {
                        if (res_chunk_fast(c + 1)) load_res(c + 1, seg[(c + 1) & 1]);
                    }
                } else {
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&ctl->acc_empty[acc]));
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
                        if (res_chunk_fast(c)) {
                            // the block fetched one chunk ago is parked in the staging buffer in the swizzled
                            // layout, and every lane then picks up its own row from there
                            uint4 (&sgc)[NSEG] = seg[c & 1];
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
                                            ((((uint32_t)(sg & 3)) ^ (uint32_t)((rrow >> 1) & 3)) << 4)) = sgc[k];
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
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && ctl->abort_flag != 0 && p.status != nullptr) atomicExch(p.status, 1);
}

template <typename OutT, bool GELU, bool RES>
int launch_gemm_variant(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mo, const GemmParams& p, cudaStream_t st) {
    SAMQ_CUDA_TRY(cudaFuncSetAttribute(gemm_i8_kernel<OutT, GELU, RES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
    const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
    const int grid = tiles < sm_count() ? tiles : sm_count();
    gemm_i8_kernel<OutT, GELU, RES><<<grid, THREADS, SMEM_BYTES, st>>>(ma, mw, mo, p);
    SAMQ_CUDA_TRY(cudaGetLastError());
    return SAMQ_OK;
}

template <typename OutT>
int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mo, const GemmParams& p, cudaStream_t st) {
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

// skip_kblock / wait_limit_cycles: see samq_gemm_i8_stall_selftest; the product entry passes -1 / 0.
static int gemm_i8_run(const int8_t* A, int64_t lda, const int8_t* W, int64_t ldw,
                       int64_t M, int64_t N, int64_t K,
                       const float* a_scale, int a_gran, const float* w_scale, int w_gran, int group_size,
                       const void* bias, const void* residual, int64_t ldr, int activation,
                       void* out, int out_dtype, int64_t ldo, int32_t* status, void* stream,
                       int skip_kblock, long long wait_limit_cycles);

int gemm_i8_dispatch(const int8_t* A, int64_t lda, const int8_t* W, int64_t ldw,
                     int64_t M, int64_t N, int64_t K,
                     const float* a_scale, int a_gran, const float* w_scale, int w_gran, int group_size,
                     const void* bias, const void* residual, int64_t ldr, int activation,
                     void* out, int out_dtype, int64_t ldo, int32_t* status, void* stream)
{
    return gemm_i8_run(A, lda, W, ldw, M, N, K, a_scale, a_gran, w_scale, w_gran, group_size, bias, residual, ldr, activation,
                       out, out_dtype, ldo, status, stream, -1, 0);
}

int gemm_i8_stall_selftest_dispatch(const int8_t* A, int64_t lda, const int8_t* W, int64_t ldw, int64_t M, int64_t N, int64_t K,
                                    int32_t* out, int64_t ldo, int skip_kblock, long long wait_limit_cycles,
                                    int32_t* status, void* stream)
{
    if (status == nullptr) return fail(SAMQ_ERR_BAD_ARG, "the stall self-test reports through the status word: it must not be null");
    if (skip_kblock < 0 || skip_kblock >= (K + BK - 1) / BK)
        return fail(SAMQ_ERR_BAD_ARG, "skip_kblock %d is not a k-block of K=%lld", skip_kblock, (long long)K);
    if (wait_limit_cycles < 100000 || wait_limit_cycles > WAIT_LIMIT_CYCLES)
        return fail(SAMQ_ERR_BAD_ARG, "wait_limit_cycles must lie between 1e5 and %lld", WAIT_LIMIT_CYCLES);
    if (M * N > (int64_t)1 << 22) return fail(SAMQ_ERR_TOO_LARGE, "the stall self-test is meant for a small GEMM");
    return gemm_i8_run(A, lda, W, ldw, M, N, K, nullptr, SAMQ_GRAN_ROW, nullptr, SAMQ_GRAN_ROW, 0, nullptr, nullptr, 0,
                       SAMQ_ACT_NONE, out, SAMQ_I32, ldo, status, stream, skip_kblock, wait_limit_cycles);
}

static int gemm_i8_run(const int8_t* A, int64_t lda, const int8_t* W, int64_t ldw,
                       int64_t M, int64_t N, int64_t K,
                       const float* a_scale, int a_gran, const float* w_scale, int w_gran, int group_size,
                       const void* bias, const void* residual, int64_t ldr, int activation,
                       void* out, int out_dtype, int64_t ldo, int32_t* status, void* stream,
                       int skip_kblock, long long wait_limit_cycles)
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
    p.skip_kblock = skip_kblock;
    p.wait_limit = wait_limit_cycles > 0 ? wait_limit_cycles : WAIT_LIMIT_CYCLES;
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
