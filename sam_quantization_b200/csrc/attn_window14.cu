// Windowed attention of SAM's encoder blocks (14 x 14-token windows) with the decomposed relative
// position bias, on the 5th-generation tensor cores: the `(q * scale) @ k^T + rel_pos -> softmax
// -> @ v` of quarot/model_utils.py:158-170 over the windows of quarot/model_utils.py:15-36, read
// straight from the qkv GEMM output [windows * 196, 3C] and written as [windows * 196, C].
//
// A persistent kernel, one CTA per SM, walks (window, head) items.  Everything an item needs
// stays on chip:
//   * Q [196 x D], K [196 x D] and V [196 x D] arrive by TMA as 16-element-wide column strips
//     (32-byte swizzle), so D = 80 costs no padding.  K and V are the same kind of tile: K is
//     consumed K-major (keys are the N rows of S = Q K^T), V MN-major (keys are the K rows of
//     O = P V), which is what makes a separate V transpose unnecessary.
//   * The two relative-position tables (27 + 27 rows, [56 x D]) sit once per CTA in the rows
//     200..255 of the K buffer, so the SAME product S = Q [K; tables]^T (M128 N256 K=D) yields
//     the 196 scores of a query in TMEM columns 0..195 and its 54 table products q . R[j] in
//     columns 200..253.  A softmax thread (one query row = one TMEM lane) picks
//     rel_h[kh] = T[qh - kh + 13] and rel_w[kw] = T[27 + qw - kw + 13] into registers.
//   * 196 keys fit one score buffer, so the softmax is exact two-pass (row maximum, then
//     2^(t - max), sum, P as bf16/fp16 into shared memory in the operand layout): no running maximum.
//   * A window has two query tiles (rows 0..127 and 128..195), each with its own 256-column
//     score buffer and its own group of four softmax warps; O = P V is accumulated into the
//     first D columns of the tile's own score buffer once its P has been extracted.
// Roles (320 threads): warps 0-3 softmax of tile A, warps 4-6 softmax of tile B (warp 7 has no
// valid row), warp 8 TMA producer, warp 9 tcgen05.mma issuer.  Loads of item i+1 overlap the
// softmax of item i (V double-buffered; Q / K are free again as soon as the score products ran).
// Every wait is bounded; a wait that runs out sets the abort flag, the roles drain, and the
// status word is set.
#include "attn_common.cuh"

namespace samq {

using namespace sm100;
using namespace attn;

namespace {

constexpr int WS = 14;                  // window side
constexpr int WL = WS * WS;             // 196 tokens per window
constexpr int NREL = 2 * WS - 1;        // 27 rows per relative-position table
constexpr int KEYS_PAD = 208;           // keys rounded up to whole 16-key MMA steps
constexpr int KSTEPS_PV = KEYS_PAD / 16;
constexpr int SCOLS = 256;              // score buffer: keys 0..195, table products at TAB_COL..TAB_COL+53
constexpr int TAB_COL = 200;
constexpr int TAB_ROWS = 56;            // 27 + 27 table rows and two zero rows
constexpr int QROWS = 200;              // Q rows fetched per window (196 valid)
constexpr int PB_ROWS = 72;             // P rows kept for the second query tile (68 valid)
constexpr int W14_THREADS = 320;
constexpr int TMEM_COLS_W14 = 512;

struct W14Control {
    uint64_t tab_full, qk_full, qk_empty, v_full[2], v_empty[2], s_full[2], s_empty[2], p_full[2], o_full[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
};

template <int D> struct W14Smem {
    static constexpr int NA = D / 16;                       // 16-element (32-byte) strips per row
    static constexpr int Q_ATOM = QROWS * 32;
    static constexpr int K_ATOM = SCOLS * 32;
    static constexpr int V_ATOM = KEYS_PAD * 32;
    static constexpr int PA_ATOM = 128 * 32;
    static constexpr int PB_ATOM = PB_ROWS * 32;
    static constexpr int Q_BYTES = NA * Q_ATOM;
    static constexpr int K_BYTES = NA * K_ATOM;
    static constexpr int V_BYTES = NA * V_ATOM;
    static constexpr int PA_BYTES = KSTEPS_PV * PA_ATOM;
    static constexpr int PB_USED = KSTEPS_PV * PB_ATOM;
    static constexpr int SCRATCH_W6 = 54 * 32 * 4;          // table products of the warp that owns only 8 P rows
    static constexpr int PB_BYTES = PB_USED + ((SCRATCH_W6 + 255) / 256) * 256;
    static constexpr int Q_OFF = 0;
    static constexpr int K_OFF = Q_OFF + Q_BYTES;
    static constexpr int V_OFF = K_OFF + K_BYTES;
    static constexpr int PA_OFF = V_OFF + 2 * V_BYTES;
    static constexpr int PB_OFF = PA_OFF + PA_BYTES;
    static constexpr int CTL_OFF = PB_OFF + PB_BYTES;
    static constexpr int TOTAL = 1024 + CTL_OFF + (int)sizeof(W14Control) + 64;
    static_assert(Q_BYTES % 256 == 0 && K_BYTES % 256 == 0 && V_BYTES % 256 == 0 && PA_BYTES % 256 == 0, "swizzle atoms must stay 256-byte aligned");
    static_assert(TOTAL <= 227 * 1024, "shared memory budget");
};

struct W14Params {
    void* out;                 // [windows * 196, C]
    int64_t items;             // windows * heads
    int heads;
    float scale;
    int32_t* status;
};

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
}

template <typename T, int D>
__global__ void __launch_bounds__(W14_THREADS, 1)
attn_window14_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                     const __grid_constant__ CUtensorMap map_tab, const W14Params p)
{
    using SM = W14Smem<D>;
    constexpr int NA = SM::NA;
    extern __shared__ uint8_t w14_smem_raw[];
    const uint32_t raw_addr = smem_u32(w14_smem_raw);
    const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
    uint8_t* base = w14_smem_raw + pad;
    W14Control* ctl = reinterpret_cast<W14Control*>(base + SM::CTL_OFF);
    volatile uint32_t* abort_flag = &ctl->abort_flag;
    const uint32_t q_s = smem_u32(base + SM::Q_OFF), k_s = smem_u32(base + SM::K_OFF), v_s = smem_u32(base + SM::V_OFF);
    const uint32_t pa_s = smem_u32(base + SM::PA_OFF), pb_s = smem_u32(base + SM::PB_OFF);

    // a CTA of this launch already gave up on a wait: do not start more work
    if (p.status != nullptr && *reinterpret_cast<volatile int32_t*>(p.status) != 0) return;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int C = p.heads * D;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&ctl->tab_full), 1);
        mbar_init(smem_u32(&ctl->qk_full), 1);
        mbar_init(smem_u32(&ctl->qk_empty), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&ctl->v_full[s]), 1);
            mbar_init(smem_u32(&ctl->v_empty[s]), 1);
            mbar_init(smem_u32(&ctl->s_full[s]), 1);
            mbar_init(smem_u32(&ctl->o_full[s]), 1);
        }
        mbar_init(smem_u32(&ctl->s_empty[0]), 4);
        mbar_init(smem_u32(&ctl->s_empty[1]), 3);
        mbar_init(smem_u32(&ctl->p_full[0]), 4);
        mbar_init(smem_u32(&ctl->p_full[1]), 3);
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_kv) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_tab) : "memory");
    }
    // the V rows 196..207 are never written by a load but are multiplied by P = 0: keep them finite
    for (int i = threadIdx.x; i < 2 * NA * (KEYS_PAD - WL) * 8; i += W14_THREADS) {
        const int buf_atom = i / ((KEYS_PAD - WL) * 8), rem = i - buf_atom * ((KEYS_PAD - WL) * 8);
        reinterpret_cast<uint32_t*>(base + SM::V_OFF + buf_atom * SM::V_ATOM + WL * 32)[rem] = 0u;
    }
    fence_async_smem();
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&ctl->tmem_base)), "r"((uint32_t)TMEM_COLS_W14) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;

    if (warp == 8) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            const uint32_t tbar = smem_u32(&ctl->tab_full);
            mbar_expect_tx(tbar, NA * TAB_ROWS * 32);
#pragma unroll
            for (int a = 0; a < NA; ++a) tma_load_2d(k_s + a * SM::K_ATOM + TAB_COL * 32, &map_tab, tbar, a * 16, 0);
            bool ok = true;
            int it = 0;
            for (int64_t item = blockIdx.x; item < p.items && ok; item += gridDim.x, ++it) {
                const int head = (int)(item % p.heads);
                const int row0 = (int)(item / p.heads) * WL;
                if (it > 0 && !mbar_wait(smem_u32(&ctl->qk_empty), (uint32_t)((it - 1) & 1), abort_flag)) { ok = false; break; }
                const uint32_t qbar = smem_u32(&ctl->qk_full);
                mbar_expect_tx(qbar, NA * (QROWS + WL) * 32);
#pragma unroll
                for (int a = 0; a < NA; ++a) tma_load_2d(q_s + a * SM::Q_ATOM, &map_q, qbar, head * D + a * 16, row0);
#pragma unroll
                for (int a = 0; a < NA; ++a) tma_load_2d(k_s + a * SM::K_ATOM, &map_kv, qbar, C + head * D + a * 16, row0);
                const int vb = it & 1;
                if (it >= 2 && !mbar_wait(smem_u32(&ctl->v_empty[vb]), (uint32_t)(((it >> 1) - 1) & 1), abort_flag)) { ok = false; break; }
                const uint32_t vbar = smem_u32(&ctl->v_full[vb]);
                mbar_expect_tx(vbar, NA * WL * 32);
#pragma unroll
                for (int a = 0; a < NA; ++a)
                    tma_load_2d(v_s + vb * SM::V_BYTES + a * SM::V_ATOM, &map_kv, vbar, 2 * C + head * D + a * 16, row0);
            }
            if (!ok) {
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000LL) { }          // let copies in flight land before the CTA retires
            }
        }
    } else if (warp == 9) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc_s = f16_idesc(AtOps<T>::kFormat, 128, SCOLS);
            constexpr uint32_t idesc_o = f16_idesc(AtOps<T>::kFormat, 128, D) | (1u << 16);      // B (= V) is MN-major
            bool ok = mbar_wait(smem_u32(&ctl->tab_full), 0, abort_flag);
            int it = 0;
            for (int64_t item = blockIdx.x; item < p.items && ok; item += gridDim.x, ++it) {
                const uint32_t ph = (uint32_t)(it & 1);
                if (!mbar_wait(smem_u32(&ctl->qk_full), ph, abort_flag)) { ok = false; break; }
                for (int b = 0; b < 2 && ok; ++b) {
                    // the tile's score buffer holds the previous item's O until its softmax warps have read it
                    if (it > 0 && !mbar_wait(smem_u32(&ctl->s_empty[b]), ph ^ 1u, abort_flag)) { ok = false; break; }
                    tcgen05_fence_after();
#pragma unroll
                    for (int a = 0; a < NA; ++a)
                        mma_f16(tmem_base + (uint32_t)(b * SCOLS), desc_sw32_k(q_s + a * SM::Q_ATOM + b * 128 * 32),
                                desc_sw32_k(k_s + a * SM::K_ATOM), idesc_s, a != 0 ? 1u : 0u);
                    tcgen05_commit(smem_u32(&ctl->s_full[b]));
                }
                if (!ok) break;
                tcgen05_commit(smem_u32(&ctl->qk_empty));                // Q and K may be refilled
                const int vb = it & 1;
                if (!mbar_wait(smem_u32(&ctl->v_full[vb]), (uint32_t)((it >> 1) & 1), abort_flag)) { ok = false; break; }
                for (int b = 0; b < 2 && ok; ++b) {
                    if (!mbar_wait(smem_u32(&ctl->p_full[b]), ph, abort_flag)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t pbase = b == 0 ? pa_s : pb_s;
                    const uint32_t patom = b == 0 ? SM::PA_ATOM : SM::PB_ATOM;
#pragma unroll
                    for (int ks = 0; ks < KSTEPS_PV; ++ks)
                        mma_f16(tmem_base + (uint32_t)(b * SCOLS), desc_sw32_k(pbase + ks * patom),
                                desc_sw32_mn(v_s + vb * SM::V_BYTES + ks * 512, SM::V_ATOM), idesc_o, ks != 0 ? 1u : 0u);
                    tcgen05_commit(smem_u32(&ctl->o_full[b]));
                }
                if (!ok) break;
                tcgen05_commit(smem_u32(&ctl->v_empty[vb]));             // this V buffer may be refilled
            }
        }
    } else if (warp != 7) {
        // ---------------- softmax + output ----------------
        const int b = warp >> 2;                                   // query tile
        const int wq = warp & 3;
        const int row = wq * 32 + lane;                            // row in the tile = TMEM lane
        const int lq = b * 128 + row;                              // query index inside the window
        const bool valid_q = lq < WL;
        const int lqc = valid_q ? lq : WL - 1;
        const int qh = lqc / WS, qw = lqc - qh * WS;
        const uint32_t lane_base = tmem_base + ((uint32_t)(wq * 32) << 16) + (uint32_t)(b * SCOLS);
        const float c = p.scale * LOG2E;
        const float2 c2 = make_float2(c, c);
        // private scratch for the 54 table products of this warp's rows: inside the warp's own P rows
        // (value j of lane l: strip j / 8, the warp's 1 KB slab of that strip), or, for the warp that owns
        // only 8 P rows, behind the P buffer
        uint8_t* p_base = base + (b == 0 ? SM::PA_OFF : SM::PB_OFF);
        const int p_atom = b == 0 ? SM::PA_ATOM : SM::PB_ATOM;
        auto scratch = [&](int j) -> float* {
            if (b == 1 && wq == 2) return reinterpret_cast<float*>(base + SM::PB_OFF + SM::PB_USED) + j * 32 + lane;
            return reinterpret_cast<float*>(p_base + (j >> 3) * p_atom + wq * 1024 + (j & 7) * 128) + lane;
        };
        const bool writes_p = (b == 0) || row < PB_ROWS;
        uint8_t* prow = p_base + row * 32;
        const uint32_t sw = (uint32_t)((row >> 2) & 1);            // 32-byte swizzle: chunk index XOR bit 7 of the address
        bool ok = true;
        int it = 0;
        for (int64_t item = blockIdx.x; item < p.items; item += gridDim.x, ++it) {
            const uint32_t ph = (uint32_t)(it & 1);
            if (ok && !mbar_wait(smem_u32(&ctl->s_full[b]), ph, abort_flag)) ok = false;
            if (!ok) break;
            tcgen05_fence_after();
            // ---- the query's products with the relative-position tables ----
            {
                uint32_t t0[32], t1[16], t2[8];
                tmem_ld32(lane_base + (uint32_t)TAB_COL, t0);
                tmem_ld16(lane_base + (uint32_t)(TAB_COL + 32), t1);
                tmem_ld8(lane_base + (uint32_t)(TAB_COL + 48), t2);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) *scratch(j) = __uint_as_float(t0[j]) * LOG2E;
#pragma unroll
                for (int j = 0; j < 16; ++j) *scratch(32 + j) = __uint_as_float(t1[j]) * LOG2E;
#pragma unroll
                for (int j = 0; j < 6; ++j) *scratch(48 + j) = __uint_as_float(t2[j]) * LOG2E;
            }
            __syncwarp();
            float bh[WS], bw[WS];
#pragma unroll
            for (int k = 0; k < WS; ++k) {
                bh[k] = *scratch(qh + (WS - 1) - k);
                bw[k] = *scratch(NREL + qw + (WS - 1) - k);
            }
            __syncwarp();                                          // the scratch is dead: P may overwrite it

            // ---- pass 1: row maximum of t = s * scale * log2e + (rel_h + rel_w) * log2e ----
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int ch = 0; ch < 7; ++ch) {
                uint32_t s[32];
                tmem_ld32(lane_base + (uint32_t)(ch * 32), s);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    const int k = ch * 32 + j;
                    if (k < WL) {
                        const int kh = k / WS, kw = k - kh * WS;
                        const float2 t = __fadd2_rn(__ffma2_rn(make_float2(__uint_as_float(s[j]), __uint_as_float(s[j + 1])), c2,
                                                               make_float2(bh[kh], bh[kh])), make_float2(bw[kw], bw[kw + 1]));
                        mx0 = fmaxf(mx0, t.x);
                        mx1 = fmaxf(mx1, t.y);
                    }
                }
            }
            const float m = fmaxf(mx0, mx1);
#pragma unroll
            for (int k = 0; k < WS; ++k) bh[k] -= m;

            // ---- pass 2: p = 2^(t - m), row sum, P into shared memory (16 keys = one 32-byte strip row) ----
            float2 ls0 = make_float2(0.f, 0.f), ls1 = make_float2(0.f, 0.f);
#pragma unroll
            for (int ch = 0; ch < 7; ++ch) {
                uint32_t s[32];
                tmem_ld32(lane_base + (uint32_t)(ch * 32), s);
                tmem_ld_wait();
                uint32_t pk[16];
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    const int k = ch * 32 + j;
                    if (k < WL) {
                        const int kh = k / WS, kw = k - kh * WS;
                        const float2 e = __fadd2_rn(__ffma2_rn(make_float2(__uint_as_float(s[j]), __uint_as_float(s[j + 1])), c2,
                                                               make_float2(bh[kh], bh[kh])), make_float2(bw[kw], bw[kw + 1]));
                        const float2 pr = make_float2(ex2(e.x), ex2(e.y));
                        if (j & 2) ls1 = __fadd2_rn(ls1, pr); else ls0 = __fadd2_rn(ls0, pr);
                        pk[j >> 1] = AtOps<T>::pack(pr.x, pr.y);
                    } else {
                        pk[j >> 1] = 0u;                           // keys 196..207 do not exist
                    }
                }
                if (writes_p) {
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const int strip = ch * 2 + half;
                        if (strip < KSTEPS_PV) {
                            uint8_t* dst = prow + strip * p_atom;
                            *reinterpret_cast<uint4*>(dst + ((0u ^ sw) << 4)) = make_uint4(pk[half * 8 + 0], pk[half * 8 + 1], pk[half * 8 + 2], pk[half * 8 + 3]);
                            *reinterpret_cast<uint4*>(dst + ((1u ^ sw) << 4)) = make_uint4(pk[half * 8 + 4], pk[half * 8 + 5], pk[half * 8 + 6], pk[half * 8 + 7]);
                        }
                    }
                }
            }
            const float2 lsum2 = __fadd2_rn(ls0, ls1);
            const float inv_l = 1.0f / (lsum2.x + lsum2.y);
            fence_async_smem();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctl->p_full[b]));

            // ---- output: O = P V sits in the first D columns of the tile's score buffer ----
            if (!mbar_wait(smem_u32(&ctl->o_full[b]), ph, abort_flag)) { ok = false; break; }
            tcgen05_fence_after();
            const int64_t token = (item / p.heads) * WL + lq;
            T* orow = reinterpret_cast<T*>(p.out) + token * (int64_t)C + (int)(item % p.heads) * D;
#pragma unroll
            for (int cc = 0; cc < D / 16; ++cc) {
                uint32_t o[16];
                tmem_ld16(lane_base + (uint32_t)(cc * 16), o);
                tmem_ld_wait();
                uint32_t w[8];
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    w[e] = AtOps<T>::pack(__uint_as_float(o[2 * e]) * inv_l, __uint_as_float(o[2 * e + 1]) * inv_l);
                if (valid_q) {
                    *reinterpret_cast<uint4*>(orow + cc * 16) = make_uint4(w[0], w[1], w[2], w[3]);
                    *reinterpret_cast<uint4*>(orow + cc * 16 + 8) = make_uint4(w[4], w[5], w[6], w[7]);
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctl->s_empty[b]));       // the score buffer may be overwritten
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    if (warp == 9) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS_W14) : "memory");
    }
    if (threadIdx.x == 0 && ctl->abort_flag != 0 && p.status != nullptr) atomicExch(p.status, 1);
}

// bf16 / fp16 [rows, cols] row-major, box = box_rows x 16 elements (32 bytes), 32-byte swizzle
int make_strip_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t pitch_elems, int box_rows, bool bf16) {
    gemm::EncodeTiledFn fn = gemm::encode_tiled_fn();
    if (fn == nullptr) return fail(SAMQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)(pitch_elems * 2)};
    cuuint32_t box[2] = {16u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base),
                    dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SAMQ_ERR_CUDA, "cuTensorMapEncodeTiled (32-byte strips) failed with CUresult %d", (int)r);
    return SAMQ_OK;
}

template <typename T, int D>
int launch_w14(const void* qkv, const void* table, const W14Params& p, int64_t windows, cudaStream_t st) {
    const bool bf16 = std::is_same<T, __nv_bfloat16>::value;
    const int C = p.heads * D;
    const int64_t tokens = windows * WL;
    CUtensorMap mq, mkv, mt;
    int rc = make_strip_map(&mq, qkv, tokens, 3 * C, 3 * C, QROWS, bf16);
    if (rc != SAMQ_OK) return rc;
    rc = make_strip_map(&mkv, qkv, tokens, 3 * C, 3 * C, WL, bf16);
    if (rc != SAMQ_OK) return rc;
    rc = make_strip_map(&mt, table, TAB_ROWS, D, D, TAB_ROWS, bf16);
    if (rc != SAMQ_OK) return rc;
    auto kernel = attn_window14_kernel<T, D>;
    SAMQ_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, W14Smem<D>::TOTAL));
    const int64_t grid = p.items < gemm::sm_count() ? p.items : gemm::sm_count();
    kernel<<<(unsigned)grid, W14_THREADS, W14Smem<D>::TOTAL, st>>>(mq, mkv, mt, p);
    SAMQ_CUDA_TRY(cudaGetLastError());
    return SAMQ_OK;
}

}  // namespace

int attn_window14_dispatch(const void* qkv, const void* table, int table_rows, int dtype, int64_t windows, int heads, int head_dim,
                           float scale, void* out, int32_t* status, void* stream)
{
    if (qkv == nullptr || table == nullptr || out == nullptr) return fail(SAMQ_ERR_BAD_ARG, "null pointer");
    if (windows < 0 || heads <= 0) return fail(SAMQ_ERR_BAD_ARG, "bad shape windows=%lld heads=%d", (long long)windows, heads);
    if (table_rows != TAB_ROWS)
        return fail(SAMQ_ERR_BAD_ARG, "the table must hold the 27 + 27 rows of both relative-position tables padded to %d rows (got %d)", TAB_ROWS, table_rows);
    if ((reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(table) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
        return fail(SAMQ_ERR_ALIGNMENT, "qkv, table and out must be 16-byte aligned");
    if (dtype != SAMQ_F16 && dtype != SAMQ_BF16) return fail(SAMQ_ERR_UNSUPPORTED, "attention takes fp16 or bf16");
    if (windows * (int64_t)WL > 2147483647LL) return fail(SAMQ_ERR_TOO_LARGE, "too many tokens");
    if (windows == 0) return SAMQ_OK;
    W14Params p;
    p.out = out; p.items = windows * heads; p.heads = heads; p.scale = scale; p.status = status;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool bf = dtype == SAMQ_BF16;
    switch (head_dim) {
    case 64: return bf ? launch_w14<__nv_bfloat16, 64>(qkv, table, p, windows, st) : launch_w14<__half, 64>(qkv, table, p, windows, st);
    case 80: return bf ? launch_w14<__nv_bfloat16, 80>(qkv, table, p, windows, st) : launch_w14<__half, 80>(qkv, table, p, windows, st);
    default: return fail(SAMQ_ERR_UNSUPPORTED, "the 14 x 14 window attention kernel is built for head_dim 64 and 80 (got %d)", head_dim);
    }
}

}  // namespace samq
