// Attention-side helpers for the decomposed relative position bias of SAM's encoder
// (the `add_decomposed_rel_pos` call of quarot/model_utils.py:162-166), reading q and k straight
// out of the qkv GEMM's output [tokens, 3C] without any reshaping copy.
//
//   bias[(qh,qw),(kh,kw)] = q . Rh[qh - kh + H - 1] + q . Rw[qw - kw + W - 1]
//
// The dot products of every query with every table row are one small tensor-core GEMM done by
// the caller: rel_all[head, token, j] = q[token, head, :] . table[j, :], j over the 2H-1 rows
// of Rh followed by the 2W-1 rows of Rw (row pitch J).  The kernels here only move data:
//
// window_prep: for windows the bias is folded into the attention inputs.  The query row becomes
//   [ q * scale | rel_h[0..H) | rel_w[0..W) | 0 ... ] and the key row [ k | onehot(kh) | onehot(kw) | 0 ... ],
//   so that q' . k' = scale * q . k + rel_h[kh] + rel_w[kw] and a stock fused attention applies.
//   One warp per token writes the token's whole [heads, width] row with 16-byte stores.
// rel_bias:    for global attention (64 x 64 keys) the explicit bias [images, heads, L, L] is
//   written once with coalesced 16-byte stores; one warp per (token, head) row of L keys.
//
// Both are bound by HBM traffic: window_prep reads 2/3 of qkv and writes 2 * width / d as much;
// rel_bias writes 2 * L bytes per (token, head).
#include "common.cuh"

namespace samq {

namespace {

template <typename T> __device__ __forceinline__ float ld(const T* p) { return Elem<T>::up(*p); }

template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]);
template <> __device__ __forceinline__ uint4 pack8<__half>(const float (&f)[8]) {
    uint4 r; __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return r;
}
template <> __device__ __forceinline__ uint4 pack8<__nv_bfloat16>(const float (&f)[8]) {
    uint4 r; __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return r;
}
template <typename T>
__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
    const T* h = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = Elem<T>::up(h[i]);
}

template <typename T>
__global__ void __launch_bounds__(256)
window_prep_kernel(const T* __restrict__ qkv, const T* __restrict__ rel_all, int64_t tokens, int J,
                   int H, int W, int nh, int d, float scale, int width,
                   T* __restrict__ q_aug, T* __restrict__ k_aug)
{
    const int lane = threadIdx.x & 31;
    const int64_t token = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (token >= tokens) return;
    const int L = H * W, C = nh * d;
    const int l = (int)(token % L), qh = l / W, qw = l - qh * W;
    const int dch = d >> 3;                            // 16-byte chunks holding q / k themselves, per head
    const int rch = (width - d) >> 3;                  // chunks holding the bias terms / one-hot codes
    const T* qrow = qkv + token * 3 * C;
    T* qo = q_aug + token * nh * width;
    T* ko = k_aug + token * nh * width;
    const int rows_h = 2 * H - 1;

    // (1) q * scale and k: the token's C values of each are contiguous in qkv; five chunks per lane
    // are loaded before any is stored so that a warp keeps 5 KB in flight
    const int nchunks = nh * dch;
    for (int c0 = 0; c0 < nchunks; c0 += 5 * 32) {
        uint4 qv[5], kv[5];
#pragma unroll
        for (int i = 0; i < 5; ++i) {
            const int c = c0 + i * 32 + lane;
            if (c < nchunks) {
                qv[i] = *reinterpret_cast<const uint4*>(qrow + c * 8);
                kv[i] = *reinterpret_cast<const uint4*>(qrow + C + c * 8);
            }
        }
#pragma unroll
        for (int i = 0; i < 5; ++i) {
            const int c = c0 + i * 32 + lane;
            if (c < nchunks) {
                const int head = c / dch, part = c - head * dch;
                float f[8];
                unpack8<T>(qv[i], f);
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] *= scale;
                *reinterpret_cast<uint4*>(qo + head * width + part * 8) = pack8<T>(f);
                *reinterpret_cast<uint4*>(ko + head * width + part * 8) = kv[i];
            }
        }
    }
    // (2) the bias terms behind q and the one-hot position codes behind k
    for (int id = lane; id < nh * rch; id += 32) {
        const int head = id / rch, r = id - head * rch;
        const T* rel = rel_all + ((int64_t)head * tokens + token) * J;
        float fq[8], fk[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int j = r * 8 + e;
            float a = 0.f, b = 0.f;
            if (j < H) { a = ld(rel + (qh - j + H - 1)); b = (j == qh) ? 1.f : 0.f; }
            else if (j < H + W) { const int kw = j - H; a = ld(rel + rows_h + (qw - kw + W - 1)); b = (kw == qw) ? 1.f : 0.f; }
            fq[e] = a; fk[e] = b;
        }
        *reinterpret_cast<uint4*>(qo + head * width + d + r * 8) = pack8<T>(fq);
        *reinterpret_cast<uint4*>(ko + head * width + d + r * 8) = pack8<T>(fk);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
rel_bias_kernel(const T* __restrict__ rel_all, int64_t tokens, int J, int H, int W, int nh, T* __restrict__ bias)
{
    __shared__ float th_s[8][64];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int L = H * W;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;     // (token, head)
    if (item >= tokens * nh) return;
    const int head = (int)(item % nh);
    const int64_t token = item / nh;
    const int l = (int)(token % L), qh = l / W, qw = l - qh * W;
    const int64_t image = token / L;
    const T* rel = rel_all + ((int64_t)head * tokens + token) * J;
    const int rows_h = 2 * H - 1;
    // per-key-row terms to shared memory, this lane's 8 per-key-column terms to registers
    for (int kh = lane; kh < H; kh += 32) th_s[warp][kh] = ld(rel + (qh - kh + H - 1));
    __syncwarp();
    const int wch = W >> 3;                            // 16-byte chunks per key row
    T* out = bias + ((image * nh + head) * L + l) * (int64_t)L;
    if (32 % wch == 0) {
        // a lane keeps the same 8 key columns on every pass: their terms are loaded once, and a
        // pass is one shared-memory read, four packed adds, the conversions and a 16-byte store
        const int kw0 = (lane % wch) * 8;
        float2 tw[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
            tw[e] = make_float2(ld(rel + rows_h + (qw - (kw0 + 2 * e) + W - 1)), ld(rel + rows_h + (qw - (kw0 + 2 * e + 1) + W - 1)));
        for (int kh = lane / wch; kh < H; kh += 32 / wch) {
            const float a = th_s[warp][kh];
            const float2 a2 = make_float2(a, a);
            float v[8];
#pragma unroll
            for (int e = 0; e < 4; ++e) { const float2 t = __fadd2_rn(a2, tw[e]); v[2 * e] = t.x; v[2 * e + 1] = t.y; }
            *reinterpret_cast<uint4*>(out + (int64_t)kh * W + kw0) = pack8<T>(v);
        }
        return;
    }
    for (int c0 = lane; c0 < H * wch; c0 += 32) {
        const int kh = c0 / wch, kw0 = (c0 - kh * wch) * 8;
        const float a = th_s[warp][kh];
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = a + ld(rel + rows_h + (qw - (kw0 + e) + W - 1));
        *reinterpret_cast<uint4*>(out + (int64_t)kh * W + kw0) = pack8<T>(v);
    }
}

}  // namespace

int attn_window_prep_dispatch(const void* qkv, const void* rel_all, int dtype, int64_t tokens, int J,
                              int H, int W, int nh, int d, float scale, int width, void* qa, void* ka, void* stream)
{
    if (qkv == nullptr || rel_all == nullptr || qa == nullptr || ka == nullptr) return fail(SAMQ_ERR_BAD_ARG, "null pointer");
    if (tokens < 0 || H <= 0 || W <= 0 || nh <= 0 || d <= 0 || width < d + H + W || J < 2 * H - 1 + 2 * W - 1)
        return fail(SAMQ_ERR_BAD_ARG, "bad shape tokens=%lld H=%d W=%d heads=%d d=%d width=%d J=%d",
                    (long long)tokens, H, W, nh, d, width, J);
    if ((d & 7) || (width & 7)) return fail(SAMQ_ERR_ALIGNMENT, "head_dim and width must be multiples of 8");
    if ((reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(qa) & 15) || (reinterpret_cast<uintptr_t>(ka) & 15))
        return fail(SAMQ_ERR_ALIGNMENT, "qkv, q_aug and k_aug must be 16-byte aligned");
    if (tokens == 0) return SAMQ_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned grid = (unsigned)((tokens + 7) / 8);
    if (dtype == SAMQ_F16)
        window_prep_kernel<__half><<<grid, 256, 0, st>>>((const __half*)qkv, (const __half*)rel_all, tokens, J, H, W, nh, d,
                                                         scale, width, (__half*)qa, (__half*)ka);
    else if (dtype == SAMQ_BF16)
        window_prep_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)qkv, (const __nv_bfloat16*)rel_all, tokens, J,
                                                                H, W, nh, d, scale, width, (__nv_bfloat16*)qa, (__nv_bfloat16*)ka);
    else return fail(SAMQ_ERR_UNSUPPORTED, "attention helpers take fp16 or bf16");
    SAMQ_CUDA_TRY(cudaGetLastError());
    return SAMQ_OK;
}

int attn_rel_bias_dispatch(const void* rel_all, int dtype, int64_t images, int J, int H, int W, int nh, void* bias, void* stream)
{
    if (rel_all == nullptr || bias == nullptr) return fail(SAMQ_ERR_BAD_ARG, "null pointer");
    if (images < 0 || H <= 0 || W <= 0 || nh <= 0 || J < 2 * H - 1 + 2 * W - 1) return fail(SAMQ_ERR_BAD_ARG, "bad shape");
    if (H > 64 || (W & 7)) return fail(SAMQ_ERR_UNSUPPORTED, "the bias kernel needs H <= 64 and W a multiple of 8 (H=%d W=%d)", H, W);
    if ((reinterpret_cast<uintptr_t>(bias) & 15) != 0) return fail(SAMQ_ERR_ALIGNMENT, "bias must be 16-byte aligned");
    if (images == 0) return SAMQ_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t tokens = images * H * W;
    const unsigned grid = (unsigned)((tokens * nh + 7) / 8);
    if (dtype == SAMQ_F16)
        rel_bias_kernel<__half><<<grid, 256, 0, st>>>((const __half*)rel_all, tokens, J, H, W, nh, (__half*)bias);
    else if (dtype == SAMQ_BF16)
        rel_bias_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)rel_all, tokens, J, H, W, nh, (__nv_bfloat16*)bias);
    else return fail(SAMQ_ERR_UNSUPPORTED, "attention helpers take fp16 or bf16");
    SAMQ_CUDA_TRY(cudaGetLastError());
    return SAMQ_OK;
}

}  // namespace samq
