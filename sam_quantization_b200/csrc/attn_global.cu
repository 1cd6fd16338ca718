// Global (full-image) attention of SAM's encoder blocks with the decomposed relative position
// bias, on the 5th-generation tensor cores.  It replaces, for the 64 x 64-token global blocks,
// the `(q * scale) @ k^T + rel_pos -> softmax -> @ v` of quarot/model_utils.py:158-170 without
// ever writing the [heads, L, L] score or bias tensors to memory.
//
//   bias[(qh,qw),(kh,kw)] = rel_h[q, qh - kh + H - 1] + rel_w[q, qw - kw + W - 1]
//
// where rel_h / rel_w are the dot products of the query with the relative-position tables (one
// small GEMM done by the caller: rel_all[head, token, j]).  The key axis is walked one key ROW
// at a time (W = 64 keys per block), so inside a block the rel_h term is one scalar per query
// and the rel_w terms are the same 64 values in every block: they live in registers.
//
// One CTA owns 128 queries of one (image, head); two CTAs are resident per SM so that one's
// softmax overlaps the other's matrix products.  Roles (192 threads):
//   warps 0-3  softmax: thread r owns query row r (= TMEM lane r).  Per key block: load the 64
//              scores from tensor memory, t = s * scale * log2e + bias, row maximum, p = 2^(t - m),
//              row sum, P as bf16/fp16 into shared memory in the 128-byte-swizzled operand layout.
//              A block is one pass with the maximum m in use and no maximum taken; only when a row
//              sum shows that some p passed 2^8 (p stays below 2^14 otherwise) is m raised, the pass
//              repeated from the scores still in tensor memory, and the output accumulator rescaled
//              in place.
//   warp 4     TMA producer: Q once, then per block the K rows and the V rows of the same keys, both
//              straight from qkv (two stages).
//   warp 5     MMA issuer: S = Q K^T (M128 N64 K=D) into one of two score buffers, and
//              O += P V (M128 N=D K64), both tcgen05.mma kind::f16 with fp32 accumulation.
// V is consumed MN-major, as D / 16 strips of [64 keys x 16 values] in the 32-byte swizzle: no transposed
// copy of V exists (attn_transpose_v below is kept for callers that want V^T for another purpose).
// Every wait is bounded; a wait that runs out sets the abort flag, the roles drain, and the
// status word is set.
#include "attn_common.cuh"

namespace samq {

using namespace sm100;
using namespace attn;

namespace {

constexpr int BQ = 128;                 // queries per CTA
constexpr int BKEY = 64;                // keys per block = one row of the key grid
constexpr int AT_THREADS = 192;        // 4 softmax warps, the TMA warp, the MMA warp
constexpr int TMEM_COLS_AT = 256;       // S0 at 0, S1 at 64, O at 128
constexpr int O_COL = 128;

struct AttnControl {
    uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], s_empty[2], p_full, pv_done;
    uint32_t tmem_base;
    uint32_t abort_flag;
};

struct AttnParams {
    const void* rel_all;     // [heads, tokens, rel_pitch]
    void* out;               // [tokens, C]
    int64_t tokens;          // units * L
    int rel_pitch;
    int H, W, L, heads, qtiles;   // token grid of one attention unit (image or window), L = H * W
    int nblocks;             // 64-key blocks per unit
    float scale;
    int32_t* status;
};

template <int D> struct AtSmem {
    static constexpr int NATOM = (D + 63) / 64;            // 128-byte swizzle rows per operand row
    static constexpr int Q_BYTES = NATOM * BQ * 128;
    static constexpr int K_BYTES = NATOM * BKEY * 128;
    static constexpr int DV = D;
    static constexpr int V_STRIP = BKEY * 32;              // one strip of V: 64 keys x 16 values (32 bytes), 32-byte swizzle
    static constexpr int VT_BYTES = (D / 16) * V_STRIP;    // D / 16 strips
    static constexpr int STAGE_BYTES = K_BYTES + VT_BYTES;
    static constexpr int P_BYTES = BQ * 128;
    static constexpr int TOTAL = 1024 + Q_BYTES + 2 * STAGE_BYTES + P_BYTES + (int)sizeof(AttnControl) + 64;
};

// WINDOW = false: one unit is an image of H x 64 tokens, a key block is one key row.
// WINDOW = true : one unit is a window of H x W tokens (H, W <= 16); keys are addressed as
//                 [H, 16] with the columns W..15 of every row (and rows >= H) absent: TMA fills
//                 them with zeros through a 4-D view of qkv, their bias is -inf, and a key block
//                 is four key rows.
template <typename T, int D, bool WINDOW>
__global__ void __launch_bounds__(AT_THREADS, 2)
attn_global_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_vt, const AttnParams p)
{
    using SM = AtSmem<D>;
    static_assert(D % 16 == 0 && D <= 128, "head_dim must be a multiple of 16 up to 128");
    extern __shared__ uint8_t at_smem_raw[];
    const uint32_t raw_addr = smem_u32(at_smem_raw);
    const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
    uint8_t* q_tile = at_smem_raw + pad;                                 // 1024-byte aligned, like every tile below
    uint8_t* stages = q_tile + SM::Q_BYTES;
    uint8_t* p_tile = stages + 2 * SM::STAGE_BYTES;
    AttnControl* ctl = reinterpret_cast<AttnControl*>(p_tile + SM::P_BYTES);
    volatile uint32_t* abort_flag = &ctl->abort_flag;

    // a CTA of this launch already gave up on a wait: do not start more work
    if (p.status != nullptr && *reinterpret_cast<volatile int32_t*>(p.status) != 0) return;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qt = blockIdx.x % p.qtiles;
    const int bh = blockIdx.x / p.qtiles;
    const int head = bh % p.heads;
    const int image = bh / p.heads;                                      // the attention unit: image or window
    const int C = p.heads * D;
    const int64_t token0 = (int64_t)image * p.L + (int64_t)qt * BQ;      // first query row of this CTA in qkv
    const int nblocks = p.nblocks;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&ctl->q_full), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&ctl->k_full[s]), 1); mbar_init(smem_u32(&ctl->k_empty[s]), 1);
            mbar_init(smem_u32(&ctl->v_full[s]), 1); mbar_init(smem_u32(&ctl->v_empty[s]), 1);
            mbar_init(smem_u32(&ctl->s_full[s]), 1);  mbar_init(smem_u32(&ctl->s_empty[s]), 4);
        }
        mbar_init(smem_u32(&ctl->p_full), 4);
        mbar_init(smem_u32(&ctl->pv_done), 1);
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_vt) : "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&ctl->tmem_base)), "r"((uint32_t)TMEM_COLS_AT) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;

    if (warp == 4) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            const uint32_t qbar = smem_u32(&ctl->q_full);
            mbar_expect_tx(qbar, SM::Q_BYTES);
#pragma unroll
            for (int a = 0; a < SM::NATOM; ++a)
                tma_load_2d(smem_u32(q_tile + a * BQ * 128), &map_q, qbar, head * D + a * 64, (int)token0);
            // K rows are released as soon as their score product has run, V rows only after the
            // P V product two blocks later: K is fetched first and runs further ahead
            bool ok = true;
            auto load_k = [&](int i) -> bool {
                const int st = i & 1;
                if (!mbar_wait(smem_u32(&ctl->k_empty[st]), ((i >> 1) & 1) ^ 1u, abort_flag)) return false;
                const uint32_t bar = smem_u32(&ctl->k_full[st]);
                uint8_t* sb = stages + st * SM::STAGE_BYTES;
                mbar_expect_tx(bar, SM::K_BYTES);
#pragma unroll
                for (int a = 0; a < SM::NATOM; ++a) {
                    if (WINDOW) tma_load_4d(smem_u32(sb + a * BKEY * 128), &map_k, bar, C + head * D + a * 64, 0, 4 * i, image);
                    else tma_load_2d(smem_u32(sb + a * BKEY * 128), &map_k, bar, C + head * D + a * 64, image * p.L + i * BKEY);
                }
                return true;
            };
            auto load_v = [&](int i) -> bool {
                const int st = i & 1;
                if (!mbar_wait(smem_u32(&ctl->v_empty[st]), ((i >> 1) & 1) ^ 1u, abort_flag)) return false;
                const uint32_t bar = smem_u32(&ctl->v_full[st]);
                const uint32_t vdst = smem_u32(stages + st * SM::STAGE_BYTES + SM::K_BYTES);
                mbar_expect_tx(bar, SM::VT_BYTES);
#pragma unroll
                for (int a = 0; a < D / 16; ++a) {              // V straight from qkv, 16 values of the head width per strip
                    if (WINDOW) tma_load_4d(vdst + a * SM::V_STRIP, &map_vt, bar, 2 * C + head * D + a * 16, 0, 4 * i, image);
                    else tma_load_2d(vdst + a * SM::V_STRIP, &map_vt, bar, 2 * C + head * D + a * 16, image * p.L + i * BKEY);
                }
                return true;
            };
            for (int i = 0; i < nblocks && ok; ++i) {
                ok = load_k(i);
                if (ok && i >= 1) ok = load_v(i - 1);
            }
            if (ok) ok = load_v(nblocks - 1);
            if (!ok) {
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000LL) { }          // let copies in flight land before the CTA retires
            }
        }
    } else if (warp == 5) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc_s = f16_idesc(AtOps<T>::kFormat, BQ, BKEY);
            constexpr uint32_t idesc_o = f16_idesc(AtOps<T>::kFormat, BQ, SM::DV) | (1u << 16);   // B (= V) is MN-major
            bool ok = mbar_wait(smem_u32(&ctl->q_full), 0, abort_flag);
            auto issue_s = [&](int j) -> bool {
                const int st = j & 1;
                const uint32_t ph = (uint32_t)((j >> 1) & 1);
                if (!mbar_wait(smem_u32(&ctl->k_full[st]), ph, abort_flag)) return false;
                if (!mbar_wait(smem_u32(&ctl->s_empty[st]), ph ^ 1u, abort_flag)) return false;
                tcgen05_fence_after();
                const uint32_t kb = smem_u32(stages + st * SM::STAGE_BYTES);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    // 16 elements = 32 bytes along K: +2 in the descriptor's (address >> 4) field; a new
                    // 128-byte swizzle row group every 64 elements
                    const uint64_t adesc = make_smem_desc(smem_u32(q_tile) + (ks >> 2) * BQ * 128) + (uint64_t)((ks & 3) * 2);
                    const uint64_t bdesc = make_smem_desc(kb + (ks >> 2) * BKEY * 128) + (uint64_t)((ks & 3) * 2);
                    mma_f16(tmem_base + (uint32_t)(st * BKEY), adesc, bdesc, idesc_s, ks != 0 ? 1u : 0u);
                }
                tcgen05_commit(smem_u32(&ctl->k_empty[st]));          // the K rows may be refilled
                tcgen05_commit(smem_u32(&ctl->s_full[st]));
                return true;
            };
            if (ok) ok = issue_s(0);
            for (int i = 0; i < nblocks && ok; ++i) {
                if (i + 1 < nblocks && !issue_s(i + 1)) { ok = false; break; }
                if (!mbar_wait(smem_u32(&ctl->v_full[i & 1]), (uint32_t)((i >> 1) & 1), abort_flag)) { ok = false; break; }
                if (!mbar_wait(smem_u32(&ctl->p_full), (uint32_t)(i & 1), abort_flag)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t vb = smem_u32(stages + (i & 1) * SM::STAGE_BYTES + SM::K_BYTES);
#pragma unroll
                for (int ks = 0; ks < BKEY / 16; ++ks) {
                    const uint64_t adesc = make_smem_desc(smem_u32(p_tile)) + (uint64_t)(ks * 2);
                    const uint64_t bdesc = desc_sw32_mn(vb + (uint32_t)(ks * 512), (uint32_t)SM::V_STRIP);   // 16 keys = 512 bytes of a strip
                    mma_f16(tmem_base + (uint32_t)O_COL, adesc, bdesc, idesc_o, (i | ks) != 0 ? 1u : 0u);
                }
                tcgen05_commit(smem_u32(&ctl->v_empty[i & 1]));       // the V rows may be refilled
                tcgen05_commit(smem_u32(&ctl->pv_done));              // P may be overwritten, O is current
            }
        }
    } else {
        // ---------------- softmax + output ----------------
        const int row = warp * 32 + lane;                          // query row in the tile = TMEM lane
        const int lq = qt * BQ + row;                              // query index inside the unit
        const bool valid_q = lq < p.L;                             // the last tile of a window runs past its tokens
        const int lqc = valid_q ? lq : p.L - 1;
        const int qh = lqc / p.W, qw = lqc - qh * p.W;
        const T* rel = reinterpret_cast<const T*>(p.rel_all) +
                       ((int64_t)head * p.tokens + (int64_t)image * p.L + lqc) * p.rel_pitch;
        const int rows_h = 2 * p.H - 1;
        // rel_w term of the key columns, times log2(e); -inf for absent columns
        constexpr int NRW = WINDOW ? 16 : BKEY;
        float rwl[NRW];
#pragma unroll
        for (int j = 0; j < NRW; ++j)
            rwl[j] = j < p.W ? AtOps<T>::up(rel + rows_h + (qw - j + p.W - 1)) * LOG2E : -INFINITY;
        const float c = p.scale * LOG2E;
        const float2 c2 = make_float2(c, c);
        float m_used = 0.f, l_sum = 0.f;             // the first block replaces this provisional maximum
        const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
        uint8_t* prow = p_tile + row * 128;
        const uint32_t sw = (uint32_t)(row & 7);
        bool ok = true;
        // rel_h term of the key row(s) of a block: one row for images, four for windows.  The values of
        // block i + 1 are fetched (16-bit, from L2) while block i is processed: a warp issues in order, so a
        // load consumed in the iteration that issues it would stall the whole softmax for its latency.
        constexpr int NRH = WINDOW ? 4 : 1;
        T rh_next[NRH];
        auto fetch_rh = [&](int blk) {
#pragma unroll
            for (int r = 0; r < NRH; ++r) {
                const int kh = NRH * blk + r;
                rh_next[r] = rel[kh < p.H ? (qh - kh + p.H - 1) : 0];
            }
        };
        fetch_rh(0);
        for (int i = 0; i < nblocks; ++i) {
            // (-inf for rows beyond the window)
            float rhv[NRH];
#pragma unroll
            for (int r = 0; r < NRH; ++r) {
                const int kh = NRH * i + r;
                rhv[r] = kh < p.H ? AtOps<T>::up(&rh_next[r]) * LOG2E : -INFINITY;
            }
            if (i + 1 < nblocks) fetch_rh(i + 1);
            if (!mbar_wait(smem_u32(&ctl->s_full[i & 1]), (uint32_t)((i >> 1) & 1), abort_flag)) { ok = false; break; }
            tcgen05_fence_after();
            // One pass over the block's 64 scores with a given reference maximum:
            //   e = s * scale * log2e + (rel_h + rel_w) * log2e - m_ref,  p = 2^e,
            // two columns per instruction; leaves P packed in pk and returns the row sum.  `row_max` is the
            // same walk without the exponentials: it returns max e.
            uint32_t pk[BKEY / 2];
            auto walk = [&](auto with_exp, float m_ref) -> float {
                constexpr bool EXP = decltype(with_exp)::value;
                uint32_t s0[32], s1[32];
                tmem_ld32(lane_base + (uint32_t)((i & 1) * BKEY), s0);
                tmem_ld32(lane_base + (uint32_t)((i & 1) * BKEY + 32), s1);
                float2 off[NRH];
#pragma unroll
                for (int r = 0; r < NRH; ++r) { const float v = rhv[r] - m_ref; off[r] = make_float2(v, v); }
                tmem_ld_wait();
                float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // independent chains
                float2 ls2[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    // column j of the first half and column 32 + j of the second
                    const float2 w0 = make_float2(rwl[j % NRW], rwl[(j + 1) % NRW]);
                    const float2 w1 = make_float2(rwl[(32 + j) % NRW], rwl[(33 + j) % NRW]);
                    const float2 b0 = __fadd2_rn(w0, off[WINDOW ? (j >> 4) : 0]);
                    const float2 b1 = __fadd2_rn(w1, off[WINDOW ? 2 + (j >> 4) : 0]);
                    const float2 e0 = __ffma2_rn(make_float2(__uint_as_float(s0[j]), __uint_as_float(s0[j + 1])), c2, b0);
                    const float2 e1 = __ffma2_rn(make_float2(__uint_as_float(s1[j]), __uint_as_float(s1[j + 1])), c2, b1);
                    const int a = (j >> 1) & 1;
                    if constexpr (EXP) {
                        const float2 p0 = make_float2(ex2(e0.x), ex2(e0.y));
                        const float2 p1 = make_float2(ex2(e1.x), ex2(e1.y));
                        ls2[2 * a] = __fadd2_rn(ls2[2 * a], p0);
                        ls2[2 * a + 1] = __fadd2_rn(ls2[2 * a + 1], p1);
                        pk[j >> 1] = AtOps<T>::pack(p0.x, p0.y);
                        pk[16 + (j >> 1)] = AtOps<T>::pack(p1.x, p1.y);
                    } else {
                        mx[2 * a] = fmaxf(mx[2 * a], fmaxf(e0.x, e0.y));
                        mx[2 * a + 1] = fmaxf(mx[2 * a + 1], fmaxf(e1.x, e1.y));
                    }
                }
                if constexpr (EXP) {
                    const float2 a2 = __fadd2_rn(__fadd2_rn(ls2[0], ls2[1]), __fadd2_rn(ls2[2], ls2[3]));
                    return a2.x + a2.y;
                } else {
                    return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
                }
            };
            auto sweep = [&](float m_ref) -> float { return walk(std::true_type{}, m_ref); };
            auto row_max = [&](float m_ref) -> float { return walk(std::false_type{}, m_ref); };
            // Optimistic pass with the maximum in use and no maximum taken: the row sum bounds the largest
            // p from above (max p <= sum <= 64 max p), so a sum beyond 2^14 (an overflowed one included)
            // tells that some p passed 2^8.  Only then, and on the first block, the true maximum is taken
            // from the scores still in tensor memory, the reference raised and the pass repeated; P stays
            // below 2^14 otherwise, inside the range of either 16-bit type.
            float bsum = 0.f;
            bool raise;
            if (i == 0) {
                raise = true;
            } else {
                bsum = sweep(m_used);
                raise = __any_sync(0xffffffffu, !(bsum <= 16384.0f));
            }
            float alpha = 1.0f;
            if (raise) {                                           // warp-uniform
                const float e_max = row_max(m_used);
                const float m_new = (i == 0) ? m_used + e_max : m_used + fmaxf(e_max, 0.f);
                alpha = (i == 0) ? 0.f : ex2(m_used - m_new);     // nothing has been accumulated before the first block
                m_used = m_new;
                bsum = sweep(m_used);
                l_sum *= alpha;
            }
            l_sum += bsum;
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctl->s_empty[i & 1]));   // the score buffer may be overwritten

            if (i > 0) {
                // the previous P V product has left P and has been added into O
                if (!mbar_wait(smem_u32(&ctl->pv_done), (uint32_t)((i - 1) & 1), abort_flag)) { ok = false; break; }
                tcgen05_fence_after();
                if (raise) {                                       // warp-uniform
#pragma unroll
                    for (int cc = 0; cc < SM::DV / 16; ++cc) {
                        uint32_t o[16];
                        tmem_ld16(lane_base + (uint32_t)(O_COL + cc * 16), o);
                        tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
                        tmem_st16(lane_base + (uint32_t)(O_COL + cc * 16), o);
                    }
                    tmem_st_wait();
                }
            }
            // P row -> shared memory, the layout tcgen05.mma reads with the 128-byte swizzle:
            // 16-byte chunk index XOR (row mod 8)
#pragma unroll
            for (int ch = 0; ch < 8; ++ch)
                *reinterpret_cast<uint4*>(prow + (((uint32_t)ch ^ sw) << 4)) =
                    make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
            fence_async_smem();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctl->p_full));
        }
        if (ok && mbar_wait(smem_u32(&ctl->pv_done), (uint32_t)((nblocks - 1) & 1), abort_flag)) {
            tcgen05_fence_after();
            const float inv_l = 1.0f / l_sum;
            T* orow = reinterpret_cast<T*>(p.out) + (token0 + row) * (int64_t)C + head * D;
#pragma unroll
            for (int cc = 0; cc < D / 16; ++cc) {
                uint32_t o[16];
                tmem_ld16(lane_base + (uint32_t)(O_COL + cc * 16), o);
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
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    if (warp == 5) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS_AT) : "memory");
    }
    if (threadIdx.x == 0 && ctl->abort_flag != 0 && p.status != nullptr) atomicExch(p.status, 1);
}

// V of every (unit, head) as [D, keys] (keys contiguous): the K-major B operand of O += P V.
// Keys are laid out as [H, key_pitch] (key_pitch = W for images; 16 for windows, the columns
// W..15 zero) and padded with zeros to a multiple of 64.  One CTA transposes 64 key slots x D
// values through shared memory; both supported types are 16-bit, so only bits move.
__global__ void __launch_bounds__(256)
transpose_v_kernel(const uint16_t* __restrict__ qkv, int H, int W, int key_pitch, int vt_len, int heads, int D,
                   uint16_t* __restrict__ vt)
{
    __shared__ uint16_t tile[128][BKEY + 2];                        // [dv][key slot], padded against bank conflicts
    const int s0 = blockIdx.x * BKEY;                               // first key slot of this CTA
    const int bh = blockIdx.y;
    const int head = bh % heads, unit = bh / heads;
    const int C = heads * D;
    const int L = H * W;
    const int chunks = D >> 3;                                      // 16-byte chunks per token
    const uint16_t* src = qkv + (int64_t)unit * L * 3 * C + 2 * C + head * D;
    for (int idx = threadIdx.x; idx < BKEY * chunks; idx += blockDim.x) {
        const int slot = idx / chunks, ch = idx - slot * chunks;
        const int kh = (s0 + slot) / key_pitch, kw = (s0 + slot) - kh * key_pitch;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (kh < H && kw < W) v = *reinterpret_cast<const uint4*>(src + (int64_t)(kh * W + kw) * 3 * C + ch * 8);
        const uint16_t* e = reinterpret_cast<const uint16_t*>(&v);
#pragma unroll
        for (int k = 0; k < 8; ++k) tile[ch * 8 + k][slot] = e[k];
    }
    __syncthreads();
    uint16_t* dst = vt + (int64_t)bh * D * vt_len + s0;
    for (int idx = threadIdx.x; idx < D * (BKEY / 2); idx += blockDim.x) {
        const int dv = idx / (BKEY / 2), pr = idx - dv * (BKEY / 2);
        *reinterpret_cast<uint32_t*>(dst + (int64_t)dv * vt_len + pr * 2) = *reinterpret_cast<const uint32_t*>(&tile[dv][pr * 2]);
    }
}

CUtensorMapDataType map_type(bool bf16) { return bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16; }

// bf16 / fp16 [rows, cols] row-major; box = box_rows x 64 elements with the 128-byte swizzle, or
// box_rows x 16 elements with the 32-byte swizzle (strips)
int make_map_16bit(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t pitch_elems, int box_rows, bool bf16,
                   bool strips = false) {
    gemm::EncodeTiledFn fn = gemm::encode_tiled_fn();
    if (fn == nullptr) return fail(SAMQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)(pitch_elems * 2)};
    cuuint32_t box[2] = {strips ? 16u : 64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, map_type(bf16), 2, const_cast<void*>(base),
                    dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    strips ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SAMQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return SAMQ_OK;
}

// qkv [units * H * W, cols] seen as [units, H, W, cols]; box = 64 (or, as strips, 16) columns x 16 key
// columns x 4 key rows of one unit: key columns W..15 and key rows >= H lie outside the view and read as zeros
int make_map_window_keys(CUtensorMap* map, const void* base, int64_t units, int H, int W, int64_t cols, bool bf16, bool strips = false) {
    gemm::EncodeTiledFn fn = gemm::encode_tiled_fn();
    if (fn == nullptr) return fail(SAMQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[4] = {(cuuint64_t)cols, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)units};
    cuuint64_t strides[3] = {(cuuint64_t)(cols * 2), (cuuint64_t)(cols * 2 * W), (cuuint64_t)(cols * 2 * W * H)};
    cuuint32_t box[4] = {strips ? 16u : 64u, 16u, 4u, 1u};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(map, map_type(bf16), 4, const_cast<void*>(base),
                    dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    strips ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SAMQ_ERR_CUDA, "cuTensorMapEncodeTiled (4-D) failed with CUresult %d", (int)r);
    return SAMQ_OK;
}

template <typename T, int D, bool WINDOW>
int launch_attn(const void* qkv, const AttnParams& p, int64_t units, cudaStream_t st) {
    const bool bf16 = std::is_same<T, __nv_bfloat16>::value;
    const int C = p.heads * D;
    CUtensorMap mq, mk, mv;
    int rc = make_map_16bit(&mq, qkv, p.tokens, 3 * C, 3 * C, BQ, bf16);
    if (rc != SAMQ_OK) return rc;
    rc = WINDOW ? make_map_window_keys(&mk, qkv, units, p.H, p.W, 3 * C, bf16)
                : make_map_16bit(&mk, qkv, p.tokens, 3 * C, 3 * C, BKEY, bf16);
    if (rc != SAMQ_OK) return rc;
    // V is read where the qkv GEMM left it, as strips of 16 values: the MN-major B operand of O += P V
    rc = WINDOW ? make_map_window_keys(&mv, qkv, units, p.H, p.W, 3 * C, bf16, true)
                : make_map_16bit(&mv, qkv, p.tokens, 3 * C, 3 * C, BKEY, bf16, true);
    if (rc != SAMQ_OK) return rc;
    auto kernel = attn_global_kernel<T, D, WINDOW>;
    SAMQ_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AtSmem<D>::TOTAL));
    const unsigned grid = (unsigned)(units * p.heads * p.qtiles);
    kernel<<<grid, AT_THREADS, AtSmem<D>::TOTAL, st>>>(mq, mk, mv, p);
    SAMQ_CUDA_TRY(cudaGetLastError());
    return SAMQ_OK;
}

// key slots per unit, padded to whole 64-key blocks
int padded_keys(int H, int W) { return W == BKEY ? H * W : ((H * 16 + BKEY - 1) / BKEY) * BKEY; }

}  // namespace

int attn_transpose_v_dispatch(const void* qkv, int dtype, int64_t units, int H, int W, int heads, int head_dim, void* vt, void* stream)
{
    if (qkv == nullptr || vt == nullptr) return fail(SAMQ_ERR_BAD_ARG, "null pointer");
    if (units < 0 || H <= 0 || W <= 0 || heads <= 0 || head_dim <= 0 || head_dim > 128 || (head_dim & 7) || !(W == BKEY || (W <= 16 && H <= 16)))
        return fail(SAMQ_ERR_BAD_ARG, "bad shape units=%lld H=%d W=%d heads=%d head_dim=%d", (long long)units, H, W, heads, head_dim);
    if ((reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(vt) & 3))
        return fail(SAMQ_ERR_ALIGNMENT, "qkv must be 16-byte aligned");
    if (dtype != SAMQ_F16 && dtype != SAMQ_BF16) return fail(SAMQ_ERR_UNSUPPORTED, "attention helpers take fp16 or bf16");
    if (units == 0) return SAMQ_OK;
    const int vt_len = padded_keys(H, W);
    dim3 grid((unsigned)(vt_len / BKEY), (unsigned)(units * heads));
    transpose_v_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(qkv), H, W, W == BKEY ? BKEY : 16, vt_len, heads, head_dim, static_cast<uint16_t*>(vt));
    SAMQ_CUDA_TRY(cudaGetLastError());
    return SAMQ_OK;
}

int attn_global_dispatch(const void* qkv, const void* vt, const void* rel_all, int dtype, int64_t units, int rel_pitch,
                         int H, int W, int heads, int head_dim, float scale, void* out, int32_t* status, void* stream)
{
    (void)vt;                                   // V is read from qkv; the argument stays for callers built against the earlier interface
    if (qkv == nullptr || rel_all == nullptr || out == nullptr) return fail(SAMQ_ERR_BAD_ARG, "null pointer");
    const bool window = W != BKEY;
    if (window ? !(W <= 16 && H <= 16 && W >= 1 && H >= 1) : ((H * W) % BQ != 0 || H <= 0))
        return fail(SAMQ_ERR_UNSUPPORTED, "the attention kernel takes images of H x %d tokens or windows of at most 16 x 16 (H=%d W=%d)", BKEY, H, W);
    if (units < 0 || heads <= 0 || rel_pitch < 2 * H - 1 + 2 * W - 1)
        return fail(SAMQ_ERR_BAD_ARG, "bad shape units=%lld H=%d W=%d heads=%d rel_pitch=%d", (long long)units, H, W, heads, rel_pitch);
    if ((reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
        return fail(SAMQ_ERR_ALIGNMENT, "qkv and out must be 16-byte aligned");
    if (dtype != SAMQ_F16 && dtype != SAMQ_BF16) return fail(SAMQ_ERR_UNSUPPORTED, "attention takes fp16 or bf16");
    if (units == 0) return SAMQ_OK;
    AttnParams p;
    p.rel_all = rel_all; p.out = out; p.tokens = units * (int64_t)H * W; p.rel_pitch = rel_pitch;
    p.H = H; p.W = W; p.L = H * W; p.heads = heads; p.qtiles = (H * W + BQ - 1) / BQ; p.scale = scale; p.status = status;
    const int vt_len = padded_keys(H, W);
    p.nblocks = vt_len / BKEY;
    if (p.tokens > 2147483647LL) return fail(SAMQ_ERR_TOO_LARGE, "too many tokens");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool bf = dtype == SAMQ_BF16;
#define SAMQ_ATTN(DV)                                                                                                   \
    (window ? (bf ? launch_attn<__nv_bfloat16, DV, true>(qkv, p, units, st)                                  \
                  : launch_attn<__half, DV, true>(qkv, p, units, st))                                        \
            : (bf ? launch_attn<__nv_bfloat16, DV, false>(qkv, p, units, st)                                 \
                  : launch_attn<__half, DV, false>(qkv, p, units, st)))
    switch (head_dim) {
    case 64: return SAMQ_ATTN(64);
    case 80: return SAMQ_ATTN(80);
    default: return fail(SAMQ_ERR_UNSUPPORTED, "the attention kernel is built for head_dim 64 and 80 (got %d)", head_dim);
    }
#undef SAMQ_ATTN
}

}  // namespace samq
