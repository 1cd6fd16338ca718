// Windowed multi-head attention with decomposed relative position bias, one pass over HBM.
//
//   out[w, l, h, :] = softmax_k( scale * q.k + q.Rh[qh-kh+H-1] + q.Rw[qw-kw+W-1] ) v
//
// for the 14x14-token windows of SAM's encoder blocks (the attention between qkv and proj,
// quarot/model_utils.py:158-170 with `add_decomposed_rel_pos`).  q, k, v are read in place from
// the qkv GEMM output [windows*L, 3C]; nothing else touches HBM except the [windows*L, C] result,
// so the kernel's roofline is HBM: (3C + C) * 2 bytes per token.
//
// One CTA per (window, head), one warp per 16-query tile (13 warps for a 14x14 window).  K and V sit in shared memory (rows padded by 16 bytes:
// conflict-free ldmatrix fragment loads); each warp owns 16-query tiles staged in its own small
// buffer; S = Q K^T, the q.table products and the bias itself run on mma.sync.m16n8k16 with the
// whole 16 x L score row-block in registers (L <= 208, so a plain softmax, no online rescaling),
// then P V with V fragments from ldmatrix.trans.
// The windows are far too small for tcgen05's 128-row tiles to pay; the legacy warp-level MMA is
// the right tool for a 196-token problem and the kernel is bound by its memory traffic.
#include "common.cuh"

namespace samq {

namespace {

template <typename T> struct MmaType;
template <> struct MmaType<__half> {
    static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
    }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    }
};
template <> struct MmaType<__nv_bfloat16> {
    static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
    }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    }
};

// ldmatrix: lane l supplies the address of row (l % 8) of matrix (l / 8); every lane receives, per
// matrix, the pair (row l / 4, columns 2 * (l % 4) ..+1) — or its transpose with .trans.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], const void* smem_row) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// 16-byte asynchronous global -> shared copy (no register staging, all copies of a thread in flight at once)
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// B fragments (k16 x n8, "col") of a row-major [n][k] operand for all KT k-steps of key tile `nt`
template <typename T, int KT, int DP>
__device__ __forceinline__ void load_b_frags(uint32_t (&b)[KT][2], const T* base, int nt, int lane) {
    const T* row = base + (nt * 8 + (lane & 7)) * DP + (lane >> 3) * 8;
#pragma unroll
    for (int k = 0; k + 1 < KT; k += 2) {
        uint32_t r[4];
        ldmatrix_x4(r, row + k * 16);
        b[k][0] = r[0]; b[k][1] = r[1]; b[k + 1][0] = r[2]; b[k + 1][1] = r[3];
    }
    if (KT & 1) {
        uint32_t r[2];
        ldmatrix_x2(r, base + (nt * 8 + (lane & 7)) * DP + ((lane >> 3) & 1) * 8 + (KT - 1) * 16);
        b[KT - 1][0] = r[0]; b[KT - 1][1] = r[1];
    }
}

// D: head width (multiple of 16); LP: padded window length (multiple of 16, >= H*W);
// JP: padded number of table rows (multiple of 8, >= 2H-1 + 2W-1).
//
// The bias is applied by the tensor cores too: per query tile the q.table products are scattered
// into a 16 x 32 tile sel[r][kh] = q_r.Rh[qh_r-kh+H-1] (columns 0..15) and
// sel[r][16+kw] = q_r.Rw[qw_r-kw+W-1] (columns 16..31), and the scores get two more k-steps
// against the constant one-hot matrix E[key][.] (row of the key in columns 0..15, column of the key
// in 16..31).  Everything after the q.k product runs in the base-2 domain (log2 e folded into the
// scale and into sel) so that the softmax needs one ex2 per score.
template <typename T, int D, int LP, int JP>
__global__ void __launch_bounds__((LP / 16) * 32, 1)
window_attention_kernel(const T* __restrict__ qkv, int H, int W, int nh,
                        const T* __restrict__ table, float scale, T* __restrict__ out)
{
    constexpr int DP = D + 8;                       // padded row pitch in elements (16 bytes of padding)
    constexpr int EP = 32 + 8;                      // pitch of the one-hot / sel tiles
    constexpr int NT = LP / 8;                      // 8-wide key tiles
    constexpr int KT = D / 16;                      // k-steps over the head width
    extern __shared__ __align__(16) uint8_t smem[];
    T* Ks = reinterpret_cast<T*>(smem);             // [LP][DP]
    T* Vs = Ks + LP * DP;                           // [LP][DP]
    T* Es = Vs + LP * DP;                           // [LP][EP]   one-hot (row | column) of every key
    constexpr int NW = LP / 16;                     // one warp per 16-query tile
    constexpr int NTHR = NW * 32;
    T* Qs = Es + LP * EP;                           // [NW][16][DP]  each warp's query tile
    T* Ss = Qs + NW * 16 * DP;                      // [NW][16][EP]  its sel tile

    const int L = H * W, C = nh * D;
    const int window = blockIdx.x / nh, head = blockIdx.x - window * nh;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tq = lane & 3;
    const T* base = qkv + (int64_t)window * L * 3 * C + head * D;
    const int rows_h = 2 * H - 1, rows_w = 2 * W - 1;

    // ---- stage K, V (asynchronously) and build E ------------------------------------------------
    constexpr int CH = D / 8;                       // 16-byte chunks per row
    for (int i = tid; i < LP * CH; i += NTHR) {
        const int r = i / CH, c = i - r * CH;
        if (r < L) {
            const T* row = base + (int64_t)r * 3 * C;
            cp_async16(Ks + r * DP + c * 8, row + C + c * 8);
            cp_async16(Vs + r * DP + c * 8, row + 2 * C + c * 8);
        } else {
            *reinterpret_cast<uint4*>(Ks + r * DP + c * 8) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(Vs + r * DP + c * 8) = make_uint4(0, 0, 0, 0);
        }
    }
    const T one = Elem<T>::down(1.0f), zero = Elem<T>::down(0.0f);
    for (int i = tid; i < LP * 32; i += NTHR) {
        const int key = i >> 5, j = i & 31;
        const int kh = key / W, kw = key - kh * W;
        Es[key * EP + j] = (key < L && ((j < 16 && j == kh) || (j >= 16 && j - 16 == kw))) ? one : zero;
    }
    for (int i = tid; i < NW * 16 * EP; i += NTHR) Ss[i] = zero;
    cp_async_wait_all();
    __syncthreads();

    T* my_q = Qs + warp * 16 * DP;
    T* my_sel = Ss + warp * 16 * EP;
    const float kLog2e = 1.4426950408889634f;
    const float scale2 = scale * kLog2e;

    {
        const int tile = warp;
        const int r0 = tile * 16 + g, r1 = r0 + 8;              // the two query rows of this thread
        // ---- Q tile: asynchronous 16-byte copies into this warp's buffer, fragments by ldmatrix ----
        for (int i = lane; i < 16 * CH; i += 32) {
            const int r = i / CH, c = i - r * CH, qr = tile * 16 + r;
            if (qr < L) cp_async16(my_q + r * DP + c * 8, base + (int64_t)qr * 3 * C + c * 8);
            else *reinterpret_cast<uint4*>(my_q + r * DP + c * 8) = make_uint4(0, 0, 0, 0);
        }
        cp_async_wait_all();
        __syncwarp();
        // Q fragments are re-read from the warp's buffer at every use instead of living in 20 registers
        const T* q_row = my_q + ((lane & 7) + ((lane >> 3) & 1) * 8) * DP + (lane >> 4) * 8;
        // ---- q . table rows, scattered into the sel tile ---------------------------------------------
        const int qh0 = min(r0, L - 1) / W, qw0 = min(r0, L - 1) - qh0 * W;
        const int qh1 = min(r1, L - 1) / W, qw1 = min(r1, L - 1) - qh1 * W;
        float ra[JP / 8][4];
#pragma unroll
        for (int jt = 0; jt < JP / 8; ++jt) ra[jt][0] = ra[jt][1] = ra[jt][2] = ra[jt][3] = 0.f;
#pragma unroll
        for (int k = 0; k < KT; ++k) {
            uint32_t qa[4];
            ldmatrix_x4(qa, q_row + k * 16);
#pragma unroll
            for (int jt = 0; jt < JP / 8; ++jt) {
                uint32_t b[2];                                    // the table is tiny and stays in L1
                b[0] = *reinterpret_cast<const uint32_t*>(table + (jt * 8 + g) * D + k * 16 + 2 * tq);
                b[1] = *reinterpret_cast<const uint32_t*>(table + (jt * 8 + g) * D + k * 16 + 2 * tq + 8);
                MmaType<T>::mma(ra[jt], qa, b);
            }
        }
#pragma unroll
        for (int jt = 0; jt < JP / 8; ++jt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = jt * 8 + 2 * tq + (e & 1);
                const int qh = (e & 2) ? qh1 : qh0, qw = (e & 2) ? qw1 : qw0;
                const int rl = (e & 2) ? g + 8 : g;
                int col = -1;
                if (j < rows_h) { const int kh = qh + (H - 1) - j; if (kh >= 0 && kh < H) col = kh; }
                else if (j < rows_h + rows_w) { const int kw = qw + (W - 1) - (j - rows_h); if (kw >= 0 && kw < W) col = 16 + kw; }
                if (col >= 0) my_sel[rl * EP + col] = Elem<T>::down(ra[jt][e] * kLog2e);
            }
        }
        __syncwarp();
        const T* sel_row = my_sel + ((lane & 7) + ((lane >> 3) & 1) * 8) * EP + (lane >> 4) * 8;
        // ---- S = (Q K^T) * scale * log2(e) + sel E^T ---------------------------------------------------
        // k-step outermost: the NT accumulators are independent, so consecutive MMAs never wait on
        // each other (with the key tile outermost every MMA would depend on the previous one)
        float s[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
        for (int k = 0; k < KT; ++k) {
            uint32_t qa[4];
            ldmatrix_x4(qa, q_row + k * 16);
#pragma unroll
            for (int nt = 0; nt < NT; nt += 2) {
                uint32_t r[4];                                    // B fragments of key tiles nt and nt + 1
                ldmatrix_x4(r, Ks + ((nt + (lane >> 4)) * 8 + (lane & 7)) * DP + k * 16 + ((lane >> 3) & 1) * 8);
                const uint32_t b0[2] = {r[0], r[1]}, b1[2] = {r[2], r[3]};
                MmaType<T>::mma(s[nt], qa, b0);
                MmaType<T>::mma(s[nt + 1], qa, b1);
            }
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) s[nt][e] *= scale2;
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            uint32_t sa[4];
            ldmatrix_x4(sa, sel_row + k * 16);
#pragma unroll
            for (int nt = 0; nt < NT; nt += 2) {
                uint32_t r[4];
                ldmatrix_x4(r, Es + ((nt + (lane >> 4)) * 8 + (lane & 7)) * EP + k * 16 + ((lane >> 3) & 1) * 8);
                const uint32_t b0[2] = {r[0], r[1]}, b1[2] = {r[2], r[3]};
                MmaType<T>::mma(s[nt], sa, b0);
                MmaType<T>::mma(s[nt + 1], sa, b1);
            }
        }
        // ---- softmax over the row block (base 2) -----------------------------------------------------
        float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            if (nt * 8 + 8 > L) {                                 // tiles that contain padding keys
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    if (nt * 8 + 2 * tq + e >= L) { s[nt][e] = -INFINITY; s[nt][2 + e] = -INFINITY; }
                }
            }
            m0 = fmaxf(m0, fmaxf(s[nt][0], s[nt][1]));
            m1 = fmaxf(m1, fmaxf(s[nt][2], s[nt][3]));
        }
        m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 1)); m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 2));
        m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 1)); m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 2));
        float l0 = 0.f, l1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(s[nt][e]) : "f"(s[nt][e] - m0));
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(s[nt][2 + e]) : "f"(s[nt][2 + e] - m1));
                l0 += s[nt][e];
                l1 += s[nt][2 + e];
            }
        }
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
        // ---- O = P V ----------------------------------------------------------------------------
        float o[D / 8][4];
#pragma unroll
        for (int dn = 0; dn < D / 8; ++dn) o[dn][0] = o[dn][1] = o[dn][2] = o[dn][3] = 0.f;
#pragma unroll
        for (int kt = 0; kt < LP / 16; ++kt) {
            uint32_t pa[4];
            pa[0] = MmaType<T>::pack(s[2 * kt][0], s[2 * kt][1]);
            pa[1] = MmaType<T>::pack(s[2 * kt][2], s[2 * kt][3]);
            pa[2] = MmaType<T>::pack(s[2 * kt + 1][0], s[2 * kt + 1][1]);
            pa[3] = MmaType<T>::pack(s[2 * kt + 1][2], s[2 * kt + 1][3]);
#pragma unroll
            for (int dn = 0; dn < D / 8; dn += 2) {
                uint32_t r[4];
                ldmatrix_x4_trans(r, Vs + (kt * 16 + (lane & 15)) * DP + (dn + (lane >> 4)) * 8);
                const uint32_t b0[2] = {r[0], r[1]}, b1[2] = {r[2], r[3]};
                MmaType<T>::mma(o[dn], pa, b0);
                MmaType<T>::mma(o[dn + 1], pa, b1);
            }
        }
        // ---- normalise and store ------------------------------------------------------------------
        const float inv0 = 1.0f / l0, inv1 = 1.0f / l1;
        T* out0 = out + ((int64_t)window * L + r0) * C + head * D;
        T* out1 = out + ((int64_t)window * L + r1) * C + head * D;
#pragma unroll
        for (int dn = 0; dn < D / 8; ++dn) {
            if (r0 < L) *reinterpret_cast<uint32_t*>(out0 + dn * 8 + 2 * tq) = MmaType<T>::pack(o[dn][0] * inv0, o[dn][1] * inv0);
            if (r1 < L) *reinterpret_cast<uint32_t*>(out1 + dn * 8 + 2 * tq) = MmaType<T>::pack(o[dn][2] * inv1, o[dn][3] * inv1);
        }
        __syncwarp();                                   // sel and the Q buffer are rewritten by the next tile
    }
}

template <typename T, int D, int LP, int JP>
int launch_window_attention(const T* qkv, int64_t windows, int H, int W, int nh, const T* table, float scale,
                            T* out, cudaStream_t st)
{
    constexpr int DP = D + 8, EP = 40;
    const size_t smem = ((size_t)(2 * LP + LP) * DP + (size_t)(LP + LP) * EP) * sizeof(T);
    SAMQ_CUDA_TRY(cudaFuncSetAttribute(window_attention_kernel<T, D, LP, JP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    window_attention_kernel<T, D, LP, JP><<<(unsigned)(windows * nh), (LP / 16) * 32, smem, st>>>(qkv, H, W, nh, table, scale, out);
    SAMQ_CUDA_TRY(cudaGetLastError());
    return SAMQ_OK;
}

template <typename T>
int window_attention_typed(const void* qkv, int64_t windows, int H, int W, int nh, int d, const void* table,
                           float scale, void* out, cudaStream_t st)
{
    const int L = H * W, J = 2 * H - 1 + 2 * W - 1;
#define SAMQ_WA(DV, LPV, JPV) \
    return launch_window_attention<T, DV, LPV, JPV>((const T*)qkv, windows, H, W, nh, (const T*)table, scale, (T*)out, st)
    if (H > 16 || W > 16) return fail(SAMQ_ERR_UNSUPPORTED, "windowed attention kernel takes windows of at most 16 x 16 (%dx%d)", H, W);
    if (L <= 16 && J <= 16) {
        if (d == 16) SAMQ_WA(16, 16, 16);
        if (d == 32) SAMQ_WA(32, 16, 16);
        if (d == 64) SAMQ_WA(64, 16, 16);
    }
    if (L <= 208 && J <= 56) {
        if (d == 64) SAMQ_WA(64, 208, 56);
        if (d == 80) SAMQ_WA(80, 208, 56);
    }
#undef SAMQ_WA
    return fail(SAMQ_ERR_UNSUPPORTED, "windowed attention kernel has no variant for window %dx%d, head_dim %d", H, W, d);
}

}  // namespace

int attn_window_dispatch(const void* qkv, int dtype, int64_t windows, int H, int W, int nh, int d,
                         const void* table, int table_rows, float scale, void* out, void* stream)
{
    if (qkv == nullptr || table == nullptr || out == nullptr) return fail(SAMQ_ERR_BAD_ARG, "null pointer");
    if (table_rows < ((2 * H - 1 + 2 * W - 1 + 7) / 8) * 8)
        return fail(SAMQ_ERR_BAD_ARG, "the table needs %d rows (2H-1 + 2W-1 rounded up to 8), got %d",
                    ((2 * H - 1 + 2 * W - 1 + 7) / 8) * 8, table_rows);
    if (windows < 0 || H <= 0 || W <= 0 || nh <= 0 || d <= 0) return fail(SAMQ_ERR_BAD_ARG, "bad shape");
    if (windows * (int64_t)nh > 2147483647LL) return fail(SAMQ_ERR_TOO_LARGE, "too many (window, head) pairs");
    if ((reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(table) & 3) ||
        (reinterpret_cast<uintptr_t>(out) & 3) || (d & 7))
        return fail(SAMQ_ERR_ALIGNMENT, "qkv must be 16-byte aligned and head_dim a multiple of 8");
    if (windows == 0) return SAMQ_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == SAMQ_F16) return window_attention_typed<__half>(qkv, windows, H, W, nh, d, table, scale, out, st);
    if (dtype == SAMQ_BF16) return window_attention_typed<__nv_bfloat16>(qkv, windows, H, W, nh, d, table, scale, out, st);
    return fail(SAMQ_ERR_UNSUPPORTED, "attention kernels take fp16 or bf16");
}

}  // namespace samq
