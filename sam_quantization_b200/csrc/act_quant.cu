// K1 — dynamic symmetric int8 quantization of activations (and weights) on B200.
//
// GPU restatement of the reference's absmax quantizers
// (RTN_quantization/per_tensor_channel_group.py:5-93) that produces the int8
// codes and the scale instead of the fake-quantized float tensor, optionally
// preceded by a SmoothQuant divisor (RTN_quantization/Smooth.py:39-40) and by
// the online Hadamard transforms of quarot/utils.py:253-289 /
// quarot/hadamard_utils.py:59-80.
//
// All kernels are bound by HBM bandwidth: a row of K fp16 values is read once
// with 16-byte loads, kept in registers (or, for the Hadamard path, in shared
// memory), and written once as K int8 codes plus one fp32 scale:
// 3K + 4 algorithmic bytes per row.
#include "common.cuh"
#include <type_traits>

namespace samq {

// ---------------------------------------------------------------------------
// 16-byte vector helpers
// ---------------------------------------------------------------------------
template <typename T> struct Vec16 { uint4 raw; };

template <typename T>
__device__ __forceinline__ void unpack(const uint4& raw, float (&f)[Elem<T>::kPerVec]);

template <> __device__ __forceinline__ void unpack<__half>(const uint4& raw, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
template <> __device__ __forceinline__ void unpack<__nv_bfloat16>(const uint4& raw, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
template <> __device__ __forceinline__ void unpack<float>(const uint4& raw, float (&f)[4]) {
    f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y);
    f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
}

template <typename T>
__device__ __forceinline__ uint4 pack(const float (&f)[Elem<T>::kPerVec]);

template <> __device__ __forceinline__ uint4 pack<__half>(const float (&f)[8]) {
    uint4 r; __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return r;
}
template <> __device__ __forceinline__ uint4 pack<__nv_bfloat16>(const float (&f)[8]) {
    uint4 r; __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return r;
}
template <> __device__ __forceinline__ uint4 pack<float>(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
}

// streaming (evict-first) 16-byte global load: every row is read exactly once
__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}

template <int N> struct PackedCodes;
template <> struct PackedCodes<8> { typedef uint2 type; };
template <> struct PackedCodes<4> { typedef uint32_t type; };

template <int N>
__device__ __forceinline__ typename PackedCodes<N>::type pack_codes(const float (&q)[N], float qmax);
template <> __device__ __forceinline__ uint2 pack_codes<8>(const float (&q)[8], float qmax) {
    uint32_t w[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t v = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) v |= code_byte(q[4 * h + i], qmax) << (8 * i);
        w[h] = v;
    }
    return make_uint2(w[0], w[1]);
}
template <> __device__ __forceinline__ uint32_t pack_codes<4>(const float (&q)[4], float qmax) {
    uint32_t v = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) v |= code_byte(q[i], qmax) << (8 * i);
    return v;
}

// ---------------------------------------------------------------------------
// What may precede the absmax in the row kernels (all optional):
//   row_map   gather: output row r reads source row row_map[r]; a negative entry is a row of
//             zeros (the zero padding of window_partition, quarot/model_utils.py:28-31)
//   SrcT      storage type of x when it differs from the tensor type T the arithmetic
//             emulates (bf16 attention output that the model casts to fp16 before proj)
//   LayerNorm y = T(gamma * (rstd * (x - mean)) + beta), fp32 statistics, the expression order
//             of torch's CUDA LayerNorm
//   divisor   SmoothQuant: y = T(y / d)
// ---------------------------------------------------------------------------
struct Prologue {
    const int32_t* row_map;
    const void* ln_gamma;
    const void* ln_beta;
    float ln_eps;
};

// ---------------------------------------------------------------------------
// Row kernel: a row lives in the registers of one warp (MULTI = false, up to 8 vectors of 16
// bytes per lane) or of `tpr` threads of a CTA (MULTI = true, 4 vectors per thread), so large
// rows keep occupancy.  Vector v of a row belongs to thread v % tpr: loads stay coalesced.
//   GRAN ROW    : scale from the row's absolute maximum
//   GRAN GROUP  : `lanes_per_group` adjacent lanes (a power of two <= 32) share a scale
//   GRAN TENSOR : the absolute maximum was reduced beforehand into *tensor_absmax
// ---------------------------------------------------------------------------
template <typename T, typename SrcT, int NV, bool MULTI, bool LN>
__global__ void __launch_bounds__(256, (LN && NV <= 5) ? 3 : 1)
quant_rows_kernel(const SrcT* __restrict__ x, int64_t M, int K, int64_t ldx, int tpr, Prologue pro,
                  const T* __restrict__ divisor, int gran, int lanes_per_group,
                  const float* __restrict__ tensor_absmax, float qmax,
                  int8_t* __restrict__ q_out, float* __restrict__ scale_out,
                  T* __restrict__ fq_out, T* __restrict__ tx_out)
{
    constexpr int E = Elem<T>::kPerVec;
    static_assert(sizeof(SrcT) == sizeof(T), "source and tensor types must have the same width");
    __shared__ float red[8];
    const int rows_per_cta = blockDim.x / tpr;
    const int rin = threadIdx.x / tpr;                 // row inside the CTA
    const int t = threadIdx.x - rin * tpr;             // thread inside the row
    const int64_t row = (int64_t)blockIdx.x * rows_per_cta + rin;
    const bool active = row < M;
    if (!MULTI && !active) return;
    const int nvec = K / E;

    int64_t src = row;
    if (pro.row_map != nullptr && active) src = pro.row_map[row];
    const bool live = active && src >= 0;
    const SrcT* xr = x + (live ? src : 0) * ldx;

    uint4 raw[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int v = i * tpr + t;
        raw[i] = (live && v < nvec) ? ld_stream(xr + (int64_t)v * E) : make_uint4(0, 0, 0, 0);
    }

    // ---- optional LayerNorm (single-warp rows only) -------------------------------------
    float mean = 0.f, rstd = 0.f;
    if constexpr (LN) {
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            float f[E];
            unpack<SrcT>(raw[i], f);
#pragma unroll
            for (int e = 0; e < E; ++e) sum += f[e];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        mean = sum / (float)K;
        float var = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int v = i * tpr + t;
            float f[E];
            unpack<SrcT>(raw[i], f);
            if (v < nvec) {
#pragma unroll
                for (int e = 0; e < E; ++e) { const float d = f[e] - mean; var += d * d; }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) var += __shfl_xor_sync(0xffffffffu, var, o);
        rstd = rsqrtf(var / (float)K + pro.ln_eps);
    }

    float vmax[NV];
    constexpr bool kPlainHalf = std::is_same<T, __half>::value && std::is_same<SrcT, __half>::value && !LN;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int v = i * tpr + t;
        if constexpr (kPlainHalf) {
            if (divisor == nullptr) {                  // |x| maximum on packed halves, no conversion
                const __half2* h = reinterpret_cast<const __half2*>(&raw[i]);
                const __half2 m2 = __hmax2(__hmax2(__habs2(h[0]), __habs2(h[1])), __hmax2(__habs2(h[2]), __habs2(h[3])));
                vmax[i] = fmaxf(__low2float(m2), __high2float(m2));
                continue;
            }
        }
        float f[E];
        unpack<SrcT>(raw[i], f);
        bool repack = !std::is_same<SrcT, T>::value;
        if (!std::is_same<SrcT, T>::value) RoundVec<T, E>::run(f);
        if constexpr (LN) {
            if (live && v < nvec) {
                float g[E], b[E];
                unpack<T>(*reinterpret_cast<const uint4*>(static_cast<const T*>(pro.ln_gamma) + (int64_t)v * E), g);
                unpack<T>(*reinterpret_cast<const uint4*>(static_cast<const T*>(pro.ln_beta) + (int64_t)v * E), b);
#pragma unroll
                for (int e = 0; e < E; ++e) f[e] = g[e] * (rstd * (f[e] - mean)) + b[e];
                RoundVec<T, E>::run(f);
                repack = true;
            }
        }
        if (divisor != nullptr && v < nvec) {
            float d[E];
            unpack<T>(*reinterpret_cast<const uint4*>(divisor + (int64_t)v * E), d);
#pragma unroll
            for (int e = 0; e < E; ++e) f[e] = __fdiv_rn(f[e], d[e]);
            RoundVec<T, E>::run(f);
            repack = true;
        }
        if (repack) raw[i] = pack<T>(f);
        float m = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) m = fmaxf(m, fabsf(f[e]));
        vmax[i] = m;
    }

    float row_scale = 0.f;
    if (gran == SAMQ_GRAN_ROW) {
        float m = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) m = fmaxf(m, vmax[i]);
        m = warp_max(m);
        if constexpr (MULTI) {
            if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
            __syncthreads();
            const int w0 = (rin * tpr) >> 5, nw = tpr >> 5;
            m = 0.f;
            for (int w = 0; w < nw; ++w) m = fmaxf(m, red[w0 + w]);
        }
        row_scale = scale_from_absmax<T>(m, qmax);
        if (active && t == 0 && scale_out != nullptr) scale_out[row] = row_scale;
    } else if (gran == SAMQ_GRAN_TENSOR) {
        row_scale = scale_from_absmax<T>(*tensor_absmax, qmax);
        if (row == 0 && t == 0 && scale_out != nullptr) scale_out[0] = row_scale;
    }
    if (MULTI && !active) return;

    const int groups_per_row = (gran == SAMQ_GRAN_GROUP) ? nvec / lanes_per_group : 0;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int v = i * tpr + t;
        float s = row_scale;
        if (gran == SAMQ_GRAN_GROUP) {
            float m = vmax[i];
            for (int o = lanes_per_group >> 1; o > 0; o >>= 1)
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            s = scale_from_absmax<T>(m, qmax);
            if (v < nvec && (t & (lanes_per_group - 1)) == 0 && scale_out != nullptr)
                scale_out[row * groups_per_row + v / lanes_per_group] = s;
        }
        if (v >= nvec) continue;
        float f[E], q[E];
        unpack<T>(raw[i], f);
        const Divider dv = make_divider(s);
#pragma unroll
        for (int e = 0; e < E; ++e) q[e] = div_exact(f[e], dv);
        if constexpr (std::is_same<T, __half>::value) {
            if (fq_out == nullptr) {
                // codes only: round the quotient to fp16, clamp, and let an fp16 addition of 1536
                // (ulp 1 in [1024, 2048)) do the round-half-even; the code is then the low byte of
                // the sum's bit pattern (0x6600 + q).  Two elements per instruction throughout.
                const __half2 hi = __float2half2_rn(qmax), lo = __float2half2_rn(-qmax), magic = __float2half2_rn(1536.0f);
                uint32_t hb[E / 2];
#pragma unroll
                for (int e = 0; e < E; e += 2) {
                    __half2 h = __floats2half2_rn(q[e], q[e + 1]);
                    h = __hadd2(__hmin2(__hmax2(h, lo), hi), magic);
                    hb[e / 2] = *reinterpret_cast<uint32_t*>(&h);
                }
                if (q_out != nullptr)
                    *reinterpret_cast<uint2*>(q_out + row * K + (int64_t)v * E) =
                        make_uint2(__byte_perm(hb[0], hb[1], 0x6420), __byte_perm(hb[2], hb[3], 0x6420));
                if (tx_out != nullptr)
                    *reinterpret_cast<uint4*>(tx_out + row * K + (int64_t)v * E) = raw[i];
                continue;
            }
        }
        RoundVec<T, E>::run(q);
#pragma unroll
        for (int e = 0; e < E; ++e) q[e] = rint_small(q[e], f[e]);
        if (q_out != nullptr)
            *reinterpret_cast<typename PackedCodes<E>::type*>(q_out + row * K + (int64_t)v * E) = pack_codes<E>(q, qmax);
        if (tx_out != nullptr)
            *reinterpret_cast<uint4*>(tx_out + row * K + (int64_t)v * E) = raw[i];
        if (fq_out != nullptr) {
#pragma unroll
            for (int e = 0; e < E; ++e) q[e] = q[e] * s;   // rounded to T by pack()
            *reinterpret_cast<uint4*>(fq_out + row * K + (int64_t)v * E) = pack<T>(q);
        }
    }
}

// ---------------------------------------------------------------------------
// Lean row kernel for the cases the encoder's fused block runs: fp16 arithmetic, one scale per
// row, codes only (no fake-quantized or transformed copy), K a multiple of 256 so that every
// lane owns exactly NV 16-byte vectors.  Same results as quant_rows_kernel, about a third of its
// instructions per element: the exact division and the LayerNorm run on packed pairs
// (fma.rn.f32x2), the absolute maximum and the rounding on packed halves, and gamma / beta sit
// in shared memory as fp32, converted once per CTA instead of once per row.
//   SRC_BF16 : x holds bf16 values that the model casts to fp16 first (attention output)
//   LN       : y = half(gamma * (rstd * (x - mean)) + beta), fp32 two-pass statistics
// A CTA of 8 warps walks `rows_per_cta` consecutive rows, one row per warp at a time.
// ---------------------------------------------------------------------------
template <bool CLAMP>
__device__ __forceinline__ uint2 codes_of_vector(const uint4& hv, float2 inv2, float2 neg_s2, __half2 lo, __half2 hi) {
    const __half2* h = reinterpret_cast<const __half2*>(&hv);
    const __half2 magic = __float2half2_rn(1536.0f);
    uint32_t hb[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        const float2 y0 = __fmul2_rn(f, inv2);
        const float2 e = __ffma2_rn(y0, neg_s2, f);
        const float2 y = __ffma2_rn(e, inv2, y0);                 // correctly rounded f / s
        __half2 q = __floats2half2_rn(y.x, y.y);                  // the fp16 quotient of the reference
        if (CLAMP) q = __hmin2(__hmax2(q, lo), hi);
        q = __hadd2(q, magic);                                    // ulp 1 in [1024, 2048): round-half-even
        hb[j] = *reinterpret_cast<uint32_t*>(&q);
    }
    return make_uint2(__byte_perm(hb[0], hb[1], 0x6420), __byte_perm(hb[2], hb[3], 0x6420));
}

template <bool SRC_BF16, bool LN, int NV>
__global__ void __launch_bounds__(256, (LN && NV <= 5) ? 4 : 1)
quant_rows_fast_kernel(const uint16_t* __restrict__ x, int64_t M, int K, int64_t ldx, int rows_per_cta,
                       const int32_t* __restrict__ row_map, const __half* __restrict__ gamma,
                       const __half* __restrict__ beta, float ln_eps, float qmax,
                       int8_t* __restrict__ q_out, float* __restrict__ scale_out)
{
    extern __shared__ float4 ln_smem[];            // LN: [2][nvec] gamma then [2][nvec] beta, as fp32 quads
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nvec = NV * 32;
    if constexpr (LN) {
        for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
            float g[8], b[8];
            unpack<__half>(*reinterpret_cast<const uint4*>(gamma + (int64_t)v * 8), g);
            unpack<__half>(*reinterpret_cast<const uint4*>(beta + (int64_t)v * 8), b);
            ln_smem[v] = make_float4(g[0], g[1], g[2], g[3]);
            ln_smem[nvec + v] = make_float4(g[4], g[5], g[6], g[7]);
            ln_smem[2 * nvec + v] = make_float4(b[0], b[1], b[2], b[3]);
            ln_smem[3 * nvec + v] = make_float4(b[4], b[5], b[6], b[7]);
        }
        __syncthreads();
    }
    const __half2 hi = __float2half2_rn(qmax), lo = __float2half2_rn(-qmax);
    const int64_t row0 = (int64_t)blockIdx.x * rows_per_cta;
    for (int r = warp; r < rows_per_cta; r += 8) {
        const int64_t row = row0 + r;
        if (row >= M) break;
        int64_t src = row;
        if (row_map != nullptr) src = row_map[row];
        const bool live = src >= 0;
        const uint16_t* xr = x + (live ? src : 0) * ldx;
        uint4 raw[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i)
            raw[i] = live ? ld_stream(xr + (int64_t)(i * 32 + lane) * 8) : make_uint4(0, 0, 0, 0);

        if constexpr (SRC_BF16) {
            // bf16 -> fp32 is a shift; fp32 -> fp16 rounds to nearest even as the cast does
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                uint32_t* w = reinterpret_cast<uint32_t*>(&raw[i]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const __half2 h = __floats2half2_rn(__uint_as_float(w[j] << 16), __uint_as_float(w[j] & 0xFFFF0000u));
                    w[j] = *reinterpret_cast<const uint32_t*>(&h);
                }
            }
        }
        if constexpr (LN) {
            if (live) {                                              // warp-uniform
                float2 d[NV][4];
                float2 acc = make_float2(0.f, 0.f);
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    const __half2* h = reinterpret_cast<const __half2*>(&raw[i]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) { d[i][j] = __half22float2(h[j]); acc = __fadd2_rn(acc, d[i][j]); }
                }
                float sum = acc.x + acc.y;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                const float mean = sum / (float)K;
                const float2 nmean = make_float2(-mean, -mean);
                acc = make_float2(0.f, 0.f);
#pragma unroll
                for (int i = 0; i < NV; ++i) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) { d[i][j] = __fadd2_rn(d[i][j], nmean); acc = __ffma2_rn(d[i][j], d[i][j], acc); }
                }
                float var = acc.x + acc.y;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) var += __shfl_xor_sync(0xffffffffu, var, o);
                const float rstd = rsqrtf(var / (float)K + ln_eps);
                const float2 rstd2 = make_float2(rstd, rstd);
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    const int v = i * 32 + lane;
                    const float4 g0 = ln_smem[v], g1 = ln_smem[nvec + v], b0 = ln_smem[2 * nvec + v], b1 = ln_smem[3 * nvec + v];
                    const float2 y0 = __ffma2_rn(make_float2(g0.x, g0.y), __fmul2_rn(rstd2, d[i][0]), make_float2(b0.x, b0.y));
                    const float2 y1 = __ffma2_rn(make_float2(g0.z, g0.w), __fmul2_rn(rstd2, d[i][1]), make_float2(b0.z, b0.w));
                    const float2 y2 = __ffma2_rn(make_float2(g1.x, g1.y), __fmul2_rn(rstd2, d[i][2]), make_float2(b1.x, b1.y));
                    const float2 y3 = __ffma2_rn(make_float2(g1.z, g1.w), __fmul2_rn(rstd2, d[i][3]), make_float2(b1.z, b1.w));
                    __half2* h = reinterpret_cast<__half2*>(&raw[i]);
                    h[0] = __floats2half2_rn(y0.x, y0.y); h[1] = __floats2half2_rn(y1.x, y1.y);
                    h[2] = __floats2half2_rn(y2.x, y2.y); h[3] = __floats2half2_rn(y3.x, y3.y);
                }
            }
        }

        __half2 m2 = __float2half2_rn(0.f);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const __half2* h = reinterpret_cast<const __half2*>(&raw[i]);
            m2 = __hmax2(m2, __hmax2(__hmax2(__habs2(h[0]), __habs2(h[1])), __hmax2(__habs2(h[2]), __habs2(h[3]))));
        }
        const float m = warp_max(fmaxf(__low2float(m2), __high2float(m2)));
        const float s = scale_from_absmax<__half>(m, qmax);
        if (lane == 0 && scale_out != nullptr) scale_out[row] = s;
        const float inv = __frcp_rn(s);
        const float2 inv2 = make_float2(inv, inv), neg_s2 = make_float2(-s, -s);
        int8_t* qr = q_out + row * K;
        // A normal fp16 scale is within 2^-11 of absmax / qmax, so no quotient rounds beyond qmax
        // and the clamp can go; a subnormal scale (absmax below ~8e-3) keeps it.
        if (s >= 6.103515625e-05f) {
#pragma unroll
            for (int i = 0; i < NV; ++i)
                *reinterpret_cast<uint2*>(qr + (int64_t)(i * 32 + lane) * 8) = codes_of_vector<false>(raw[i], inv2, neg_s2, lo, hi);
        } else {
#pragma unroll
            for (int i = 0; i < NV; ++i)
                *reinterpret_cast<uint2*>(qr + (int64_t)(i * 32 + lane) * 8) = codes_of_vector<true>(raw[i], inv2, neg_s2, lo, hi);
        }
    }
}

// ---------------------------------------------------------------------------
// Generic kernel: one warp per (row, group) unit, scalar accesses, two passes.
// Covers every shape the vector kernel does not (odd K, unaligned rows,
// very long rows, group sizes that are not 8 * 2^j).
// ---------------------------------------------------------------------------
template <typename T, typename SrcT>
__global__ void __launch_bounds__(256)
quant_rows_generic_kernel(const SrcT* __restrict__ x, int64_t M, int K, int64_t ldx, const int32_t* __restrict__ row_map,
                          const T* __restrict__ divisor, int gran, int group_size,
                          const float* __restrict__ tensor_absmax, float qmax,
                          int8_t* __restrict__ q_out, float* __restrict__ scale_out,
                          T* __restrict__ fq_out, T* __restrict__ tx_out)
{
    const int lane = threadIdx.x & 31;
    const int span = (gran == SAMQ_GRAN_GROUP) ? group_size : K;
    const int units_per_row = K / span;
    const int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= M * units_per_row) return;
    const int64_t row = unit / units_per_row;
    const int c0 = (int)(unit % units_per_row) * span;
    const int64_t src = row_map != nullptr ? (int64_t)row_map[row] : row;
    const SrcT* xr = x + (src >= 0 ? src : 0) * ldx;
    auto value = [&](int c) -> float {
        if (src < 0) return 0.f;
        float v = round_to<T>(Elem<SrcT>::up(xr[c]));
        if (divisor != nullptr) v = round_to<T>(__fdiv_rn(v, Elem<T>::up(divisor[c])));
        return v;
    };

    float s;
    if (gran == SAMQ_GRAN_TENSOR) {
        s = scale_from_absmax<T>(*tensor_absmax, qmax);
        if (unit == 0 && lane == 0 && scale_out != nullptr) scale_out[0] = s;
    } else {
        float m = 0.f;
        for (int c = c0 + lane; c < c0 + span; c += 32) m = fmaxf(m, fabsf(value(c)));
        m = warp_max(m);
        s = scale_from_absmax<T>(m, qmax);
        if (lane == 0 && scale_out != nullptr) scale_out[unit] = s;
    }
    const Divider dv = make_divider(s);
    for (int c = c0 + lane; c < c0 + span; c += 32) {
        const float v = value(c);
        const float q = quant_value<T>(v, dv);
        if (q_out != nullptr) q_out[row * K + c] = saturate_i8(q, qmax);
        if (tx_out != nullptr) tx_out[row * K + c] = Elem<T>::down(v);
        if (fq_out != nullptr) fq_out[row * K + c] = Elem<T>::down(q * s);
    }
}

// ---------------------------------------------------------------------------
// Per-tensor absolute maximum (first pass of per_tensor quantization).  The
// result lives in caller-provided scratch memory that the launcher zeroes.
// Non-negative floats order like their bit patterns, so atomicMax on the
// integer view is exact.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
absmax_kernel(const T* __restrict__ x, int64_t M, int K, int64_t ldx,
              const T* __restrict__ divisor, float* __restrict__ result)
{
    float m = 0.f;
    const int64_t total = M * (int64_t)K;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / K;
        const int c = (int)(i - r * K);
        float v = Elem<T>::up(x[r * ldx + c]);
        if (divisor != nullptr) v = round_to<T>(__fdiv_rn(v, Elem<T>::up(divisor[c])));
        m = fmaxf(m, fabsf(v));
    }
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<int*>(result), __float_as_int(m));
}

// ---------------------------------------------------------------------------
// Hadamard + quantization kernel: one CTA owns one row held in shared memory
// as fp32.  Butterflies run in registers, 4 index bits (16 values) per round,
// so a 4096-wide transform needs three passes over shared memory.
//
// The transform axis has length `axis` = had_k * 2^log2_pow and is embedded in
// the row as   index = (outer * axis + a) * inner + in,
//   FULL    : inner = 1,       outer = 1, axis = K
//   PARTIAL : inner = had_dim, outer = 1, axis = K / had_dim  (the head axis)
// Within the axis, a = k * 2^log2_pow + b: the 2^log2_pow part gets the
// butterflies (strides 1,2,4,... as matmul_hadU does), the had_k part is mixed
// by the explicit +-1 matrix.
// ---------------------------------------------------------------------------
__device__ __forceinline__ int padded(int i) { return i + (i >> 4); }

// in-register butterflies over the 4 low index bits of 16 values, strides 1, 2, 4, 8 in that order.
// Values j and j + 8 travel as one fp32 pair, so the first three stages are packed adds; a - c is
// formed as fma(c, -1, a), which rounds exactly as the subtraction does.
__device__ __forceinline__ void butterfly16(float (&v)[16]) {
    float2 p[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) p[i] = make_float2(v[i], v[i + 8]);
    const float2 neg1 = make_float2(-1.f, -1.f);
#pragma unroll
    for (int s = 1; s < 8; s <<= 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if ((i & s) == 0) {
                const float2 a = p[i], c = p[i | s];
                p[i] = __fadd2_rn(a, c);
                p[i | s] = __ffma2_rn(c, neg1, a);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) { v[i] = p[i].x + p[i].y; v[i + 8] = p[i].x - p[i].y; }
}

// The last arithmetic step of the transform: divide by sqrt(axis) (a true division), round once
// to T, and track the absolute maximum.
template <typename T>
__device__ __forceinline__ float finish_value(float v, const Divider& root, float& m) {
    v = round_to<T>(div_exact(v, root));
    m = fmaxf(m, fabsf(v));
    return v;
}
// the same for a pair (fp16: packed division, one conversion each way for both values)
template <typename T>
__device__ __forceinline__ float2 finish_pair(float2 v, const Divider& root, float& m) {
    if constexpr (std::is_same<T, __half>::value) {
        const float2 inv2 = make_float2(root.inv, root.inv), ns2 = make_float2(-root.s, -root.s);
        const float2 y0 = __fmul2_rn(v, inv2);
        const float2 e = __ffma2_rn(y0, ns2, v);
        const float2 y = __ffma2_rn(e, inv2, y0);
        const __half2 h = __floats2half2_rn(y.x, y.y);
        const __half2 a = __habs2(h);
        m = fmaxf(m, fmaxf(__low2float(a), __high2float(a)));
        return __half22float2(h);
    } else {
        return make_float2(finish_value<T>(v.x, root, m), finish_value<T>(v.y, root, m));
    }
}

// The HK x HK mix across chunks for two adjacent columns at a time: the inputs of both columns
// sit in registers as pairs, the +-1 entries come from shared memory (each stored twice, so one
// 16-byte load feeds two packed multiply-adds).  `ld` is the row pitch of the stored matrix,
// `halves` the number of independent HK-chunk blocks the mix is applied to (2 when an order-2HK
// factor is evaluated as [[A, A], [A, -A]]).  FINISH: also scale, round and track the maximum.
template <typename T, int HK, bool FINISH>
__device__ __forceinline__ void mix_columns(float* sm, const float4* hk4, int ld, int cols, int halves,
                                            int tid, int nthr, const Divider& root, float& m) {
    const int pairs = cols >> 1;
    for (int p = tid; p < pairs * halves; p += nthr) {
        const int half = p / pairs;
        const int c = (p - half * pairs) << 1;
        float* col = sm;
        const int k0 = half * HK;
        float2 in2[HK];
#pragma unroll
        for (int k = 0; k < HK; ++k) {                  // c is even: c and c + 1 share a 16-group, so their padded slots are adjacent
            const int a = padded((k0 + k) * cols + c);
            in2[k] = make_float2(col[a], col[a + 1]);
        }
#pragma unroll 1
        for (int k = 0; k < HK; ++k) {                   // not unrolled: the inputs alone fill the registers
            float2 acc = make_float2(0.f, 0.f);
#pragma unroll
            for (int k2 = 0; k2 < HK; k2 += 2) {
                const float4 h = hk4[(k * ld + k2) >> 1];
                acc = __ffma2_rn(make_float2(h.x, h.y), in2[k2], acc);
                acc = __ffma2_rn(make_float2(h.z, h.w), in2[k2 + 1], acc);
            }
            if (FINISH) acc = finish_pair<T>(acc, root, m);
            const int a = padded((k0 + k) * cols + c);
            col[a] = acc.x;
            col[a + 1] = acc.y;
        }
    }
}

// `vec` != 0: K % 16 == 0 and every pointer / row pitch allows 16-byte accesses; each thread then
// moves 16 consecutive elements at a time (two 16-byte loads of fp16, one 16-byte store of codes).
// HK: the explicit factor this instance is compiled for (1 = none, 12, 20, 40; 0 = any, read at
// run time).  An order-40 factor of the form [[A, A], [A, -A]] (checked in the kernel) runs as one
// butterfly across the two halves followed by the order-20 mix with A on each half.
template <typename T, typename SrcT, int HK>
__global__ void __launch_bounds__(512)
hadamard_quant_kernel(const SrcT* __restrict__ x, int64_t M, int K, int64_t ldx, const int32_t* __restrict__ row_map,
                      const T* __restrict__ divisor, const int8_t* __restrict__ signs,
                      int inner, int axis, int had_k, int log2_pow,
                      const float* __restrict__ hadk, float qmax,
                      int8_t* __restrict__ q_out, float* __restrict__ scale_out,
                      T* __restrict__ fq_out, T* __restrict__ tx_out, int vec)
{
    extern __shared__ float4 sm4[];        // padded(K) floats, then the had_k matrix, then 32 floats
    float* sm = reinterpret_cast<float*>(sm4);
    const int hk_off = (padded(K) + 1 + 3) & ~3;                      // 16-byte aligned
    float4* hk4 = reinterpret_cast<float4*>(sm + hk_off);             // entries stored twice: (h, h)
    float* hk = sm + hk_off;
    float* red = hk + 2 * had_k * had_k + 4;
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int64_t row = blockIdx.x;
    const int64_t src = row_map != nullptr ? (int64_t)row_map[row] : row;
    const SrcT* xr = x + (src >= 0 ? src : 0) * ldx;
    constexpr int E = Elem<T>::kPerVec;                               // elements per 16 bytes: 8 or 4
    const int chunks = K >> 4;
    const Divider root = make_divider(sqrtf((float)axis));
    float m = 0.f;                                                    // running |value| maximum of this thread
    bool finished = false;                                            // the scaling has been folded into a phase
    // the first four butterfly stages act on 16 consecutive elements: do them before the values
    // ever reach shared memory
    const bool first_in_regs = vec && inner == 1 && log2_pow >= 4;
    const bool only_round = first_in_regs && log2_pow == 4 && HK == 1;

    // (a) load (gathered row, or zeros for a padding row), SmoothQuant divisor, sign flip
    if (vec) {
        for (int g = tid; g < chunks; g += nthr) {
            const int c0 = g << 4;
            float v[16];
            if (src >= 0) {
#pragma unroll
                for (int i = 0; i < 16 / E; ++i) {
                    float f[E];
                    unpack<SrcT>(ld_stream(xr + c0 + i * E), f);
                    if (!std::is_same<SrcT, T>::value) RoundVec<T, E>::run(f);
#pragma unroll
                    for (int e = 0; e < E; ++e) v[i * E + e] = f[e];
                }
                if (divisor != nullptr) {
#pragma unroll
                    for (int i = 0; i < 16 / E; ++i) {
                        float d[E];
                        unpack<T>(*reinterpret_cast<const uint4*>(divisor + c0 + i * E), d);
#pragma unroll
                        for (int e = 0; e < E; ++e) v[i * E + e] = round_to<T>(__fdiv_rn(v[i * E + e], d[e]));
                    }
                }
                if (signs != nullptr) {
                    const uint4 sg = *reinterpret_cast<const uint4*>(signs + c0);
                    const uint32_t w[4] = {sg.x, sg.y, sg.z, sg.w};
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if ((w[j >> 2] >> (8 * (j & 3))) & 0x80u) v[j] = -v[j];
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = 0.f;
            }
            if (first_in_regs) butterfly16(v);
            if (only_round) {
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                    const float2 f = finish_pair<T>(make_float2(v[j], v[j + 1]), root, m);
                    v[j] = f.x; v[j + 1] = f.y;
                }
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) sm[c0 + g + j] = v[j];       // = padded(c0 + j)
        }
        finished = only_round;
    } else {
        for (int c = tid; c < K; c += nthr) {
            float v = src >= 0 ? round_to<T>(Elem<SrcT>::up(xr[c])) : 0.f;
            if (divisor != nullptr) v = round_to<T>(__fdiv_rn(v, Elem<T>::up(divisor[c])));
            if (signs != nullptr && signs[c] < 0) v = -v;
            sm[padded(c)] = v;
        }
    }
    bool blocked40 = false;
    if constexpr (HK != 1) {
        for (int i = tid; i < had_k * had_k; i += nthr) { const float h = hadk[i]; hk[2 * i] = h; hk[2 * i + 1] = h; }
        if constexpr (HK == 40) {
            // is the matrix [[A, A], [A, -A]] ?
            int ok = 1;
            for (int i = tid; i < 400; i += nthr) {
                const int k = i / 20, k2 = i - k * 20;
                const float a = hadk[k * 40 + k2];
                ok &= (hadk[k * 40 + k2 + 20] == a) & (hadk[(k + 20) * 40 + k2] == a) & (hadk[(k + 20) * 40 + k2 + 20] == -a);
            }
            blocked40 = __syncthreads_and(ok) != 0;
        }
    }
    // The second round (index bits 4..7) only mixes chunks written by threads of the same
    // half-warp when every thread owns exactly one chunk and one group: a warp barrier suffices.
    if (first_in_regs && chunks <= nthr && log2_pow >= 8) __syncwarp(); else __syncthreads();

    // (b) butterflies over the power-of-two part of the axis, 4 bits per round
    const int pow_len = 1 << log2_pow;
    for (int b = first_in_regs ? 4 : 0; b < log2_pow; b += 4) {
        const int r = min(4, log2_pow - b);
        const int R = 1 << r;
        const int groups = K >> r;
        const int rest_len = pow_len >> r;               // values of the axis index without the r bits
        const bool last = (HK == 1) && (b + 4 >= log2_pow);
        for (int g = tid; g < groups; g += nthr) {
            // g enumerates (k_chunk, rest, in) with `in` fastest
            int in = 0, t = g;
            if (inner != 1) { in = g % inner; t = g / inner; }
            const int rest = t & (rest_len - 1);
            const int kc = t / rest_len;                 // chunk of the had_k part (and outer)
            const int lo = rest & ((1 << b) - 1);
            const int hi = rest >> b;
            const int a0 = kc * pow_len + ((hi << (b + r)) | lo);
            const int base = a0 * inner + in;
            const int step = inner << b;
            // padded(base + j * step) is linear in j when the step is a multiple of 16
            const bool lin = (step & 15) == 0;
            const int pbase = padded(base), pstep = step + (step >> 4);
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) if (j < R) v[j] = sm[lin ? pbase + j * pstep : padded(base + j * step)];
            if (R == 16) {
                butterfly16(v);
            } else {
#pragma unroll
                for (int s = 1; s < 16; s <<= 1) {
                    if (s < R) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if ((j & s) == 0 && j < R) {
                                const float a = v[j], c = v[j | s];
                                v[j] = a + c;
                                v[j | s] = a - c;
                            }
                        }
                    }
                }
            }
            if (last) {
                if (R == 16) {
#pragma unroll
                    for (int j = 0; j < 16; j += 2) {
                        const float2 f = finish_pair<T>(make_float2(v[j], v[j + 1]), root, m);
                        v[j] = f.x; v[j + 1] = f.y;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) if (j < R) v[j] = finish_value<T>(v[j], root, m);
                }
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) if (j < R) sm[lin ? pbase + j * pstep : padded(base + j * step)] = v[j];
        }
        if (last) finished = true;
        else __syncthreads();                            // the closing barrier below follows the last round
    }

    // (c) explicit had_k x had_k mix across the chunks
    if constexpr (HK != 1) {
        const int cols = pow_len * inner;                // positions inside one chunk
        int done = 0;                                    // columns handled two at a time
        if constexpr (HK == 12 || HK == 20) {
            mix_columns<T, HK, true>(sm, hk4, HK, cols, 1, tid, nthr, root, m);
            done = cols & ~1;
        }
        if constexpr (HK == 40) {
            if (blocked40 && (cols & 1) == 0) {
                for (int i = tid; i < 20 * cols; i += nthr) {       // chunk k with chunk k + 20
                    const float a = sm[padded(i)], c = sm[padded(i + 20 * cols)];
                    sm[padded(i)] = a + c;
                    sm[padded(i + 20 * cols)] = a - c;
                }
                __syncthreads();
                mix_columns<T, 20, true>(sm, hk4, 40, cols, 2, tid, nthr, root, m);
                done = cols;
            }
        }
        // any other factor (and an odd last column): each thread owns whole columns
        for (int c = done + tid; c < cols; c += nthr) {
            float in_v[64];
            for (int k = 0; k < had_k; ++k) in_v[k] = sm[padded(k * cols + c)];
            for (int k = 0; k < had_k; ++k) {
                float acc = 0.f;
                for (int k2 = 0; k2 < had_k; ++k2) acc += hk[2 * (k * had_k + k2)] * in_v[k2];
                sm[padded(k * cols + c)] = finish_value<T>(acc, root, m);
            }
        }
        finished = true;
    }

    // (d) a transform of length one has no phase above to carry the scaling
    if (!finished) {
        __syncthreads();
        for (int c = tid; c < K; c += nthr) sm[padded(c)] = finish_value<T>(sm[padded(c)], root, m);
    }
    m = warp_max(m);
    if ((tid & 31) == 0) red[tid >> 5] = m;
    __syncthreads();                                     // values and per-warp maxima are in shared memory
    {
        float t = 0.f;
        for (int w = 0; w < ((nthr + 31) >> 5); ++w) t = fmaxf(t, red[w]);
        m = t;
    }
    const float s = scale_from_absmax<T>(m, qmax);
    if (tid == 0 && scale_out != nullptr) scale_out[row] = s;

    // (e) quantize and store
    const Divider dv = make_divider(s);
    if (vec) {
        for (int g = tid; g < chunks; g += nthr) {
            const int c0 = g << 4;
            float v16[16], q[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v16[j] = sm[c0 + g + j];
            if constexpr (std::is_same<T, __half>::value) {
                if (fq_out == nullptr && tx_out == nullptr && q_out != nullptr) {
                    // codes only: packed exact division, fp16 rounding of the quotient, clamp, and
                    // the round-half-even of an fp16 addition of 1536 (see quant_rows_fast_kernel)
                    const float2 inv2 = make_float2(dv.inv, dv.inv), ns2 = make_float2(-s, -s);
                    const __half2 hi2 = __float2half2_rn(qmax), lo2 = __float2half2_rn(-qmax), magic = __float2half2_rn(1536.0f);
                    uint32_t hb[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float2 f = make_float2(v16[2 * j], v16[2 * j + 1]);
                        const float2 y0 = __fmul2_rn(f, inv2);
                        const float2 e = __ffma2_rn(y0, ns2, f);
                        const float2 y = __ffma2_rn(e, inv2, y0);
                        __half2 h = __floats2half2_rn(y.x, y.y);
                        h = __hadd2(__hmin2(__hmax2(h, lo2), hi2), magic);
                        hb[j] = *reinterpret_cast<uint32_t*>(&h);
                    }
                    *reinterpret_cast<uint4*>(q_out + row * K + c0) =
                        make_uint4(__byte_perm(hb[0], hb[1], 0x6420), __byte_perm(hb[2], hb[3], 0x6420),
                                   __byte_perm(hb[4], hb[5], 0x6420), __byte_perm(hb[6], hb[7], 0x6420));
                    continue;
                }
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) q[j] = quant_value<T>(v16[j], dv);
            if (q_out != nullptr) {
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    w[i] = code_byte(q[4 * i], qmax) | (code_byte(q[4 * i + 1], qmax) << 8) |
                           (code_byte(q[4 * i + 2], qmax) << 16) | (code_byte(q[4 * i + 3], qmax) << 24);
                *reinterpret_cast<uint4*>(q_out + row * K + c0) = make_uint4(w[0], w[1], w[2], w[3]);
            }
#pragma unroll
            for (int i = 0; i < 16 / E; ++i) {
                float f[E];
                if (tx_out != nullptr) {
#pragma unroll
                    for (int e = 0; e < E; ++e) f[e] = v16[i * E + e];
                    *reinterpret_cast<uint4*>(tx_out + row * K + c0 + i * E) = pack<T>(f);
                }
                if (fq_out != nullptr) {
#pragma unroll
                    for (int e = 0; e < E; ++e) f[e] = q[i * E + e] * s;      // rounded to T by pack()
                    *reinterpret_cast<uint4*>(fq_out + row * K + c0 + i * E) = pack<T>(f);
                }
            }
        }
    } else {
        for (int c = tid; c < K; c += nthr) {
            const float v = sm[padded(c)];
            const float q = quant_value<T>(v, dv);
            if (q_out != nullptr) q_out[row * K + c] = saturate_i8(q, qmax);
            if (tx_out != nullptr) tx_out[row * K + c] = Elem<T>::down(v);
            if (fq_out != nullptr) fq_out[row * K + c] = Elem<T>::down(q * s);
        }
    }
}

// ---------------------------------------------------------------------------
// The 4096-point transform with 64 points per thread: 4096 = 64 x 64, so the twelve butterfly stages
// are two register passes (index bits 0..5, then 6..11, the reference's stage order) with ONE
// regrouping of the row through shared memory between them, instead of three passes and two
// regroupings at 16 points per thread.  A CTA is 64 threads (two warps) and walks rows in a loop:
//   load    the row arrives through cp.async, 16 bytes per thread and instruction, coalesced in global
//           memory and scattered to a padded layout (144-byte pitch per owner thread) so that every
//           thread then reads its own 64 consecutive values with conflict-free 16-byte loads; the
//           next row's copies are issued as soon as pass A has left the staging buffer, and travel
//           during the rest of the row (27 KB of shared memory and 121 registers: 8 CTAs per SM)
//   pass A  thread t owns elements 64 t + j
//   X       rows of 64 floats at a 68-float pitch, written with 16 x STS.128, column u read back
//   pass B  thread u owns elements 64 j + u, then the exact scaling by 1/64, one rounding to fp16,
//           the row maximum, the codes
//   codes   as bytes at 64 j + u, read back 16 bytes per thread in row order and stored coalesced
// Same values in the same order as every other kernel of the family: bit-identical results.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void butterfly64(float (&v)[64]) {
    float2 p[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) p[i] = make_float2(v[i], v[i + 32]);
    const float2 neg1 = make_float2(-1.f, -1.f);
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if ((i & s) == 0) {
                const float2 a = p[i], c = p[i | s];
                p[i] = __fadd2_rn(a, c);
                p[i | s] = __ffma2_rn(c, neg1, a);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) { v[i] = p[i].x + p[i].y; v[i + 32] = p[i].x - p[i].y; }
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                 ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}

// SMs of the current device (a grid of resident CTAs is sized from it)
inline int device_sm_count() {
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

template <typename SrcT>
__global__ void __launch_bounds__(64, 8)
hadamard_4096_r64_kernel(const SrcT* __restrict__ x, int64_t M, int64_t ldx, const int32_t* __restrict__ row_map,
                         const int8_t* __restrict__ signs, float qmax,
                         int8_t* __restrict__ q_out, float* __restrict__ scale_out)
{
    constexpr int K = 4096;
    constexpr int SPITCH = 144;                                 // bytes per owner thread in the staging buffer: 128 + 16
    constexpr int XPITCH = 68;                                  // floats per row of X
    __shared__ __align__(16) uint8_t stage[64 * SPITCH];
    __shared__ __align__(16) float xs[64 * XPITCH];             // X, then the byte codes
    __shared__ float red[2][2];
    const int t = threadIdx.x;
    auto source_row = [&](int64_t row) -> int64_t { return row_map != nullptr ? (int64_t)row_map[row] : row; };
    auto fetch = [&](int64_t src) {                             // one row into the staging buffer (nothing for a zero row)
        if (src >= 0) {
            const uint8_t* g = reinterpret_cast<const uint8_t*>(x + src * ldx);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int c = i * 64 + t;                       // 16-byte chunk of the row; owner c / 8, position c % 8
                cp_async16(&stage[(c >> 3) * SPITCH + (c & 7) * 16], g + 16 * c);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    int64_t row = blockIdx.x;
    int64_t src = row < M ? source_row(row) : -1;
    if (row < M) fetch(src);
    for (int it = 0; row < M; ++it, row += gridDim.x) {
        const int64_t next = row + gridDim.x;
        const int64_t next_src = next < M ? source_row(next) : -1;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                        // the row is in the staging buffer; xs is free
        float v[64];
        if (src >= 0) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                float f[8];
                unpack<SrcT>(*reinterpret_cast<const uint4*>(&stage[t * SPITCH + k * 16]), f);
                if (!std::is_same<SrcT, __half>::value) RoundVec<__half, 8>::run(f);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[k * 8 + e] = f[e];
            }
            if (signs != nullptr) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint4 sg = *reinterpret_cast<const uint4*>(signs + 64 * t + 16 * k);
                    const uint32_t w[4] = {sg.x, sg.y, sg.z, sg.w};
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if ((w[j >> 2] >> (8 * (j & 3))) & 0x80u) v[k * 16 + j] = -v[k * 16 + j];
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] = 0.f;
        }
        butterfly64(v);                                         // pass A: index bits 0..5
#pragma unroll
        for (int q = 0; q < 16; ++q)
            *reinterpret_cast<float4*>(xs + t * XPITCH + 4 * q) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        __syncthreads();                                        // X is complete, and nobody reads the staging buffer any more:
        if (next < M) fetch(next_src);                          // the next row travels while this one is transformed
#pragma unroll
        for (int j = 0; j < 64; ++j) v[j] = xs[j * XPITCH + t];
        butterfly64(v);                                         // pass B: bits 6..11; v[j] is element 64 j + t
        __half2 m2 = __float2half2_rn(0.f);
        const float2 root2 = make_float2(0.015625f, 0.015625f); // 1 / sqrt(4096), an exact scaling
#pragma unroll
        for (int i = 0; i < 64; i += 2) {                       // scale, round once to fp16, absolute maximum
            const float2 sv = __fmul2_rn(make_float2(v[i], v[i + 1]), root2);
            const __half2 h = __floats2half2_rn(sv.x, sv.y);
            m2 = __hmax2(m2, __habs2(h));
            const float2 f = __half22float2(h);
            v[i] = f.x; v[i + 1] = f.y;
        }
        float m = fmaxf(__low2float(m2), __high2float(m2));
        m = warp_max(m);
        if ((t & 31) == 0) red[it & 1][t >> 5] = m;
        __syncthreads();                                        // also: every thread is past its reads of X
        m = fmaxf(red[it & 1][0], red[it & 1][1]);
        const float sc = scale_from_absmax<__half>(m, qmax);
        if (t == 0 && scale_out != nullptr) scale_out[row] = sc;
        const float inv = __frcp_rn(sc);
        const float2 inv2 = make_float2(inv, inv), ns2 = make_float2(-sc, -sc);
        const __half2 hi2 = __float2half2_rn(qmax), lo2 = __float2half2_rn(-qmax), magic = __float2half2_rn(1536.0f);
        uint8_t* codes = reinterpret_cast<uint8_t*>(xs);
        // A normal fp16 scale is within 2^-11 of absmax / qmax, so no quotient rounds beyond qmax and the
        // clamp can go; a subnormal scale (absmax below ~8e-3) keeps it (as in quant_rows_fast_kernel).
        const bool clamp = !(sc >= 6.103515625e-05f);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float2 f = make_float2(v[2 * j], v[2 * j + 1]);
            const float2 y0 = __fmul2_rn(f, inv2);
            const float2 e = __ffma2_rn(y0, ns2, f);
            const float2 y = __ffma2_rn(e, inv2, y0);
            __half2 h = __floats2half2_rn(y.x, y.y);
            if (clamp) h = __hmin2(__hmax2(h, lo2), hi2);       // CTA-uniform
            h = __hadd2(h, magic);
            const uint32_t hb = *reinterpret_cast<uint32_t*>(&h);
            codes[64 * (2 * j) + t] = (uint8_t)hb;
            codes[64 * (2 * j + 1) + t] = (uint8_t)(hb >> 16);
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = i * 64 + t;                           // 16 consecutive codes of the row
            *reinterpret_cast<uint4*>(q_out + row * K + 16 * c) = *reinterpret_cast<const uint4*>(codes + 16 * c);
        }
        src = next_src;
        // the next iteration's first barrier orders these reads of the codes before X is written again
    }
}

// ---------------------------------------------------------------------------
// The 1024-point transform the same way: 1024 = 64 x 16.  A row belongs to 16 threads (half a warp), so
// nothing in the loop needs a CTA barrier; a CTA of 64 threads walks groups of four rows.
//   pass A  thread t of the row owns elements 64 t + j (bits 0..5), as in the 4096-point kernel
//   X       16 rows of 64 floats (68-float pitch), written with 16 x STS.128
//   pass B  thread u takes columns 4 u .. 4 u + 3 of all 16 rows with 16 x LDS.128: four independent
//           16-point butterflies (bits 6..9) on packed pairs, scaling by 1/32, rounding, row maximum
//           (shuffles inside the half-warp), codes; the four codes of a row of X are one 32-bit store
// LN: the LayerNorm of the source row in front (norm1 -> qkv, norm2 -> lin1 of a rotated ViT-L in one
// launch), fp32 two-pass statistics, y = half(gamma * (rstd * (x - mean)) + beta) as in
// quant_rows_fast_kernel, gamma / beta as fp32 quads in shared memory (quad q of thread t at q * 16 + t);
// a gathered zero row stays zero (the padding of window_partition comes after the norm).
// ---------------------------------------------------------------------------
template <typename SrcT, bool LN>
__global__ void __launch_bounds__(64, LN ? 6 : 8)
hadamard_1024_r64_kernel(const SrcT* __restrict__ x, int64_t M, int64_t ldx, const int32_t* __restrict__ row_map,
                         const int8_t* __restrict__ signs, const __half* __restrict__ gamma,
                         const __half* __restrict__ beta, float ln_eps, float qmax,
                         int8_t* __restrict__ q_out, float* __restrict__ scale_out)
{
    constexpr int K = 1024;
    constexpr int SPITCH = 144;                                 // bytes per owner thread in the staging buffer: 128 + 16
    constexpr int XPITCH = 68;                                  // floats per row of X
    __shared__ __align__(16) uint8_t stage_all[4 * 16 * SPITCH];
    __shared__ __align__(16) float xs_all[4 * 16 * XPITCH];     // X, then the byte codes
    __shared__ float4 ln_gb[LN ? 2 : 1][LN ? 256 : 1];
    const int r_in = threadIdx.x >> 4, u = threadIdx.x & 15;    // row inside the group, thread inside the row
    uint8_t* stage = stage_all + r_in * 16 * SPITCH;
    float* xs = xs_all + r_in * 16 * XPITCH;
    if constexpr (LN) {
        for (int o = threadIdx.x; o < 256; o += 64) {           // 16-byte loads of 8 halves: 128 of gamma, 128 of beta
            const int which = o >> 7, c = o & 127;              // columns 8 c .. 8 c + 7: owner c / 8, quads 2 (c % 8), + 1
            float f[8];
            unpack<__half>(*reinterpret_cast<const uint4*>((which ? beta : gamma) + 8 * c), f);
            ln_gb[which][((c & 7) * 2) * 16 + (c >> 3)] = make_float4(f[0], f[1], f[2], f[3]);
            ln_gb[which][((c & 7) * 2 + 1) * 16 + (c >> 3)] = make_float4(f[4], f[5], f[6], f[7]);
        }
        __syncthreads();
    }
    auto source_row = [&](int64_t row) -> int64_t {
        if (row >= M) return -1;
        return row_map != nullptr ? (int64_t)row_map[row] : row;
    };
    auto fetch = [&](int64_t src) {                             // this thread's share of its row (nothing for a zero row)
        if (src >= 0) {
            const uint8_t* g = reinterpret_cast<const uint8_t*>(x + src * ldx);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int c = i * 16 + u;                       // 16-byte chunk of the row; owner c / 8, position c % 8
                cp_async16(&stage[(c >> 3) * SPITCH + (c & 7) * 16], g + 16 * c);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int64_t groups = (M + 3) >> 2;
    int64_t grp = blockIdx.x;
    int64_t src = grp < groups ? source_row(4 * grp + r_in) : -1;
    if (grp < groups) fetch(src);
    for (; grp < groups; grp += gridDim.x) {
        const int64_t row = 4 * grp + r_in;
        const int64_t next = grp + gridDim.x;
        const int64_t next_src = next < groups ? source_row(4 * next + r_in) : -1;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();                                           // the row is in the staging buffer; its X is free
        float v[64];
        if (src >= 0) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                float f[8];
                unpack<SrcT>(*reinterpret_cast<const uint4*>(&stage[u * SPITCH + k * 16]), f);
                if (!std::is_same<SrcT, __half>::value) RoundVec<__half, 8>::run(f);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[k * 8 + e] = f[e];
            }
        } else {
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] = 0.f;
        }
        if constexpr (LN) {
            float2 acc = make_float2(0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 64; j += 2) acc = __fadd2_rn(acc, make_float2(v[j], v[j + 1]));
            float sum = acc.x + acc.y;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            const float mean = sum / (float)K;
            const float2 nmean = make_float2(-mean, -mean);
            acc = make_float2(0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 64; j += 2) {
                const float2 d = __fadd2_rn(make_float2(v[j], v[j + 1]), nmean);
                v[j] = d.x; v[j + 1] = d.y;
                acc = __ffma2_rn(d, d, acc);
            }
            float var = acc.x + acc.y;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) var += __shfl_xor_sync(0xffffffffu, var, o);
            const float rstd = rsqrtf(var / (float)K + ln_eps);
            const float2 rstd2 = make_float2(rstd, rstd);
            if (src >= 0) {
#pragma unroll
                for (int q = 0; q < 16; ++q) {
                    const float4 g = ln_gb[0][q * 16 + u], bb = ln_gb[LN ? 1 : 0][q * 16 + u];
                    const float2 y0 = __ffma2_rn(make_float2(g.x, g.y), __fmul2_rn(rstd2, make_float2(v[4 * q], v[4 * q + 1])), make_float2(bb.x, bb.y));
                    const float2 y1 = __ffma2_rn(make_float2(g.z, g.w), __fmul2_rn(rstd2, make_float2(v[4 * q + 2], v[4 * q + 3])), make_float2(bb.z, bb.w));
                    const float2 r0 = __half22float2(__floats2half2_rn(y0.x, y0.y));
                    const float2 r1 = __half22float2(__floats2half2_rn(y1.x, y1.y));
                    v[4 * q] = r0.x; v[4 * q + 1] = r0.y; v[4 * q + 2] = r1.x; v[4 * q + 3] = r1.y;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 64; ++j) v[j] = 0.f;
            }
        }
        if (src >= 0 && signs != nullptr) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint4 sg = *reinterpret_cast<const uint4*>(signs + 64 * u + 16 * k);
                const uint32_t w[4] = {sg.x, sg.y, sg.z, sg.w};
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if ((w[j >> 2] >> (8 * (j & 3))) & 0x80u) v[k * 16 + j] = -v[k * 16 + j];
            }
        }
        butterfly64(v);                                         // pass A: index bits 0..5
#pragma unroll
        for (int q = 0; q < 16; ++q)
            *reinterpret_cast<float4*>(xs + u * XPITCH + 4 * q) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        __syncwarp();                                           // X is complete, and nobody reads the staging buffer any more:
        if (next < groups) fetch(next_src);                     // the next row travels while this one is transformed
        float2 a[16], b[16];                                    // a[j] / b[j]: columns 4 u, 4 u + 1 / 4 u + 2, 4 u + 3 of row j of X
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float4 f = *reinterpret_cast<const float4*>(xs + j * XPITCH + 4 * u);
            a[j] = make_float2(f.x, f.y); b[j] = make_float2(f.z, f.w);
        }
        const float2 neg1 = make_float2(-1.f, -1.f);
#pragma unroll
        for (int s2 = 1; s2 < 16; s2 <<= 1) {                   // pass B: index bits 6..9
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                if ((j & s2) == 0) {
                    const float2 a0 = a[j], a1 = a[j | s2], b0 = b[j], b1 = b[j | s2];
                    a[j] = __fadd2_rn(a0, a1); a[j | s2] = __ffma2_rn(a1, neg1, a0);
                    b[j] = __fadd2_rn(b0, b1); b[j | s2] = __ffma2_rn(b1, neg1, b0);
                }
            }
        }
        __half2 m2 = __float2half2_rn(0.f);
        const float2 root2 = make_float2(0.03125f, 0.03125f);   // 1 / sqrt(1024), an exact scaling
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float2 sa = __fmul2_rn(a[j], root2), sb = __fmul2_rn(b[j], root2);
            const __half2 ha = __floats2half2_rn(sa.x, sa.y), hb = __floats2half2_rn(sb.x, sb.y);
            m2 = __hmax2(m2, __hmax2(__habs2(ha), __habs2(hb)));
            a[j] = __half22float2(ha); b[j] = __half22float2(hb);
        }
        float m = fmaxf(__low2float(m2), __high2float(m2));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const float sc = scale_from_absmax<__half>(m, qmax);
        if (u == 0 && row < M && scale_out != nullptr) scale_out[row] = sc;
        const float inv = __frcp_rn(sc);
        const float2 inv2 = make_float2(inv, inv), ns2 = make_float2(-sc, -sc);
        const __half2 hi2 = __float2half2_rn(qmax), lo2 = __float2half2_rn(-qmax), magic = __float2half2_rn(1536.0f);
        uint8_t* codes = reinterpret_cast<uint8_t*>(xs);
        const bool clamp = !(sc >= 6.103515625e-05f);           // only a subnormal fp16 scale lets a quotient round beyond qmax
        __syncwarp();                                           // every thread of the row is past its reads of X
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            uint32_t hw[2];
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
                const float2 f = h2 ? b[j] : a[j];
                const float2 y0 = __fmul2_rn(f, inv2);
                const float2 e = __ffma2_rn(y0, ns2, f);
                const float2 y = __ffma2_rn(e, inv2, y0);
                __half2 h = __floats2half2_rn(y.x, y.y);
                if (clamp) h = __hmin2(__hmax2(h, lo2), hi2);   // uniform over the row's half-warp
                h = __hadd2(h, magic);
                hw[h2] = *reinterpret_cast<uint32_t*>(&h);
            }
            *reinterpret_cast<uint32_t*>(codes + 64 * j + 4 * u) = __byte_perm(hw[0], hw[1], 0x6420);
        }
        __syncwarp();
        if (row < M) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int c = i * 16 + u;                       // 16 consecutive codes of the row
                *reinterpret_cast<uint4*>(q_out + row * K + 16 * c) = *reinterpret_cast<const uint4*>(codes + 16 * c);
            }
        }
        src = next_src;
        // the __syncwarp at the top of the next iteration orders these reads before X is written again
    }
}

// ---------------------------------------------------------------------------
// The transform across 16 heads on its own (`proj` input of the QuaRot configs with 16 heads):
// fp16 arithmetic, codes only, no shared memory.  A thread owns 8 consecutive positions of the
// head width for ALL 16 heads: sixteen 16-byte loads in flight, then for every position one
// 16-point butterfly over the heads in registers (stage order 1, 2, 4, 8 as everywhere), the exact
// scaling by 1 / sqrt(16), one rounding to fp16.  LPR lanes share a row (8 or 16, the next power of
// two at or above had_dim / 8), so the row maximum is a few shuffles.
// ---------------------------------------------------------------------------
template <typename SrcT, int LPR>
__global__ void __launch_bounds__(256)
hadamard_heads16_quant_kernel(const SrcT* __restrict__ x, int64_t M, int64_t ldx, const int32_t* __restrict__ row_map,
                              int had_dim, float qmax, int8_t* __restrict__ q_out, float* __restrict__ scale_out)
{
    constexpr int RPW = 32 / LPR;                              // rows per warp
    const int lane = threadIdx.x & 31;
    const int c = lane % LPR;                                  // 16-byte chunk of the head width
    const int64_t row = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * RPW + lane / LPR;
    const int K = 16 * had_dim;
    const bool active = row < M && c * 8 < had_dim;
    int64_t src = -1;
    if (active) src = row_map != nullptr ? (int64_t)row_map[row] : row;
    uint4 raw[16];                                             // [head] -> 8 fp16 values
#pragma unroll
    for (int h = 0; h < 16; ++h)
        raw[h] = src >= 0 ? ld_stream(x + src * ldx + h * had_dim + c * 8) : make_uint4(0, 0, 0, 0);
    if (!std::is_same<SrcT, __half>::value) {
#pragma unroll
        for (int h = 0; h < 16; ++h) {
            float f[8];
            unpack<SrcT>(raw[h], f);
            raw[h] = pack<__half>(f);                          // the cast to fp16 the model applies
        }
    }
    float m = 0.f;
#pragma unroll
    for (int pr = 0; pr < 4; ++pr) {                           // two positions at a time
        float va[16], vb[16];
#pragma unroll
        for (int h = 0; h < 16; ++h) {
            const float2 f = __half22float2(reinterpret_cast<const __half2*>(&raw[h])[pr]);
            va[h] = f.x; vb[h] = f.y;
        }
        butterfly16(va);
        butterfly16(vb);
#pragma unroll
        for (int h = 0; h < 16; ++h) {
            const __half2 hh = __floats2half2_rn(va[h] * 0.25f, vb[h] * 0.25f);
            const __half2 a = __habs2(hh);
            m = fmaxf(m, fmaxf(__low2float(a), __high2float(a)));
            reinterpret_cast<__half2*>(&raw[h])[pr] = hh;
        }
    }
#pragma unroll
    for (int o = LPR >> 1; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (!active) return;
    const float sc = scale_from_absmax<__half>(m, qmax);
    if (c == 0 && scale_out != nullptr) scale_out[row] = sc;
    const float inv = __frcp_rn(sc);
    const float2 inv2 = make_float2(inv, inv), ns2 = make_float2(-sc, -sc);
    const __half2 hi2 = __float2half2_rn(qmax), lo2 = __float2half2_rn(-qmax);
    int8_t* qr = q_out + row * K + c * 8;
#pragma unroll
    for (int h = 0; h < 16; ++h)
        *reinterpret_cast<uint2*>(qr + h * had_dim) = codes_of_vector<true>(raw[h], inv2, ns2, lo2, hi2);
}

// ---------------------------------------------------------------------------
// Host launchers
// ---------------------------------------------------------------------------
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T, typename SrcT>
static int launch_rows(const SrcT* x, int64_t M, int K, int64_t ldx, const Prologue& pro, const T* divisor,
                       int gran, int group_size, const float* tensor_absmax, float qmax,
                       int8_t* q, float* scale, T* fq, T* tx, cudaStream_t st)
{
    constexpr int E = Elem<T>::kPerVec;
    const bool ln = pro.ln_gamma != nullptr;
    bool vec_ok = (K % E == 0) && (ldx % E == 0) && aligned16(x) && aligned16(fq) && aligned16(tx) &&
                  aligned16(divisor) && aligned16(pro.ln_gamma) && aligned16(pro.ln_beta) &&
                  ((reinterpret_cast<uintptr_t>(q) & 7) == 0) && K <= 256 * 4 * E;
    int lanes_per_group = 32;
    if (gran == SAMQ_GRAN_GROUP) {
        lanes_per_group = group_size / E;
        const bool pow2 = lanes_per_group > 0 && (lanes_per_group & (lanes_per_group - 1)) == 0;
        vec_ok = vec_ok && (group_size % E == 0) && pow2 && lanes_per_group <= 32;
    }
    const int nvec = K / E;
    if (ln && !(vec_ok && nvec <= 320))
        return fail(SAMQ_ERR_UNSUPPORTED, "fused LayerNorm needs 16-byte aligned rows of at most %d elements (K=%d)", 320 * E, K);
    if constexpr (std::is_same<T, __half>::value) {
        // the lean kernel: fp16 arithmetic, per-row scale, codes only, whole vectors per lane
        const bool src_bf16 = std::is_same<SrcT, __nv_bfloat16>::value;
        if (vec_ok && gran == SAMQ_GRAN_ROW && divisor == nullptr && fq == nullptr && tx == nullptr && q != nullptr &&
            nvec % 32 == 0 && !(ln && src_bf16)) {
            const int nv = nvec / 32;
            const uint16_t* xs = reinterpret_cast<const uint16_t*>(x);
            const __half* g = static_cast<const __half*>(pro.ln_gamma);
            const __half* b = static_cast<const __half*>(pro.ln_beta);
            const int rows_per_cta = ln ? 32 : 8;
            const unsigned grid = (unsigned)((M + rows_per_cta - 1) / rows_per_cta);
            const size_t smem = ln ? (size_t)nvec * 64 : 0;
            bool launched = true;
#define SAMQ_FAST(BF, LN_, NVAL)                                                                            \
            quant_rows_fast_kernel<BF, LN_, NVAL><<<grid, 256, smem, st>>>(xs, M, K, ldx, rows_per_cta, pro.row_map, \
                                                                           g, b, pro.ln_eps, qmax, q, scale)
            if (ln) {
                switch (nv) {
                case 3: SAMQ_FAST(false, true, 3); break;
                case 4: SAMQ_FAST(false, true, 4); break;
                case 5: SAMQ_FAST(false, true, 5); break;
                default: launched = false;
                }
            } else if (src_bf16) {
                switch (nv) {
                case 3: SAMQ_FAST(true, false, 3); break;
                case 4: SAMQ_FAST(true, false, 4); break;
                case 5: SAMQ_FAST(true, false, 5); break;
                default: launched = false;
                }
            } else {
                switch (nv) {
                case 3: SAMQ_FAST(false, false, 3); break;
                case 4: SAMQ_FAST(false, false, 4); break;
                case 5: SAMQ_FAST(false, false, 5); break;
                case 12: SAMQ_FAST(false, false, 12); break;
                case 16: SAMQ_FAST(false, false, 16); break;
                case 20: SAMQ_FAST(false, false, 20); break;
                default: launched = false;
                }
            }
#undef SAMQ_FAST
            if (launched) {
                SAMQ_CUDA_TRY(cudaGetLastError());
                return SAMQ_OK;
            }
        }
    }
    if (vec_ok) {
#define SAMQ_LAUNCH(NVAL, MULTI_, LN_, TPR, GRID, BLOCK)                                               \
        quant_rows_kernel<T, SrcT, NVAL, MULTI_, LN_><<<GRID, BLOCK, 0, st>>>(x, M, K, ldx, TPR, pro,    \
            divisor, gran, lanes_per_group, tensor_absmax, qmax, q, scale, fq, tx)
        if (nvec <= 320) {
            const int nv = (nvec + 31) / 32;
            const unsigned grid = (unsigned)((M + 7) / 8);
            if (ln) {
                switch (nv) {
                case 1: SAMQ_LAUNCH(1, false, true, 32, grid, 256); break;
                case 2: SAMQ_LAUNCH(2, false, true, 32, grid, 256); break;
                case 3: SAMQ_LAUNCH(3, false, true, 32, grid, 256); break;
                case 4: SAMQ_LAUNCH(4, false, true, 32, grid, 256); break;
                case 5: SAMQ_LAUNCH(5, false, true, 32, grid, 256); break;
                case 6: SAMQ_LAUNCH(6, false, true, 32, grid, 256); break;
                case 7: case 8: SAMQ_LAUNCH(8, false, true, 32, grid, 256); break;
                default: SAMQ_LAUNCH(10, false, true, 32, grid, 256); break;
                }
            } else {
                switch (nv) {
                case 1: SAMQ_LAUNCH(1, false, false, 32, grid, 256); break;
                case 2: SAMQ_LAUNCH(2, false, false, 32, grid, 256); break;
                case 3: SAMQ_LAUNCH(3, false, false, 32, grid, 256); break;
                case 4: SAMQ_LAUNCH(4, false, false, 32, grid, 256); break;
                case 5: SAMQ_LAUNCH(5, false, false, 32, grid, 256); break;
                case 6: SAMQ_LAUNCH(6, false, false, 32, grid, 256); break;
                case 7: case 8: SAMQ_LAUNCH(8, false, false, 32, grid, 256); break;
                default: SAMQ_LAUNCH(10, false, false, 32, grid, 256); break;
                }
            }
        } else {
            int tpr = (((nvec + 3) / 4) + 31) / 32 * 32;             // threads per row at 4 vectors each
            const int rows_per_cta = 256 / tpr > 0 ? 256 / tpr : 1;
            const unsigned grid = (unsigned)((M + rows_per_cta - 1) / rows_per_cta);
            SAMQ_LAUNCH(4, true, false, tpr, grid, rows_per_cta * tpr);
        }
#undef SAMQ_LAUNCH
    } else {
        const int span = (gran == SAMQ_GRAN_GROUP) ? group_size : K;
        const int64_t units = M * (K / span);
        const int warps = 8;
        dim3 grid((unsigned)((units + warps - 1) / warps)), block(warps * 32);
        quant_rows_generic_kernel<T, SrcT><<<grid, block, 0, st>>>(x, M, K, ldx, pro.row_map, divisor, gran, group_size,
                                                                   tensor_absmax, qmax, q, scale, fq, tx);
    }
    SAMQ_CUDA_TRY(cudaGetLastError());
    return SAMQ_OK;
}

template <typename T, typename SrcT>
static int quant_typed(const SrcT* x, int64_t M, int K, int64_t ldx, const Prologue& pro, const T* divisor,
                       const samq_hadamard_spec* had, int gran, int group_size, float qmax,
                       int8_t* q, float* scale, T* fq, T* tx,
                       void* workspace, size_t workspace_bytes, cudaStream_t st)
{
    if (M == 0) return SAMQ_OK;
    if (had != nullptr && had->mode != SAMQ_HAD_NONE) {
        if (gran != SAMQ_GRAN_ROW)
            return fail(SAMQ_ERR_UNSUPPORTED, "an online Hadamard is only combined with per-token quantization");
        // LayerNorm + transform in one call exists for the kernel specialised for 1024 points (fp16, codes only)
        const bool ln_had = pro.ln_gamma != nullptr;
        int inner, axis;
        if (had->mode == SAMQ_HAD_FULL) { inner = 1; axis = K; }
        else if (had->mode == SAMQ_HAD_PARTIAL) {
            if (had->had_dim <= 0 || K % had->had_dim != 0)
                return fail(SAMQ_ERR_BAD_ARG, "had_dim %d does not divide K=%d", had->had_dim, K);
            inner = had->had_dim; axis = K / had->had_dim;
        } else return fail(SAMQ_ERR_BAD_ARG, "unknown hadamard mode %d", had->mode);
        const int hk = had->had_k;
        if (hk < 1 || hk > 64 || axis % hk != 0)
            return fail(SAMQ_ERR_UNSUPPORTED, "had_k=%d must be in [1,64] and divide the transform length %d", hk, axis);
        const int pw = axis / hk;
        if ((pw & (pw - 1)) != 0)
            return fail(SAMQ_ERR_UNSUPPORTED, "transform length %d is not had_k=%d times a power of two", axis, hk);
        if (hk > 1 && had->hadk == nullptr)
            return fail(SAMQ_ERR_BAD_ARG, "had_k=%d needs the hadk matrix", hk);
        int log2_pow = 0; while ((1 << log2_pow) < pw) ++log2_pow;
        const size_t smem = (size_t)(K + (K >> 4) + 8 + 2 * hk * hk + 4 + 32) * sizeof(float);
        if (smem > 200 * 1024) return fail(SAMQ_ERR_TOO_LARGE, "row of K=%d does not fit in shared memory", K);
        int threads = ((K / 16 + 31) / 32) * 32;
        threads = threads < 32 ? 32 : (threads > 512 ? 512 : threads);
        auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
        const int vec = (K % 16 == 0) && (ldx % Elem<T>::kPerVec == 0) && al16(x) && al16(divisor) && al16(had->signs) &&
                        al16(q) && al16(fq) && al16(tx);
#define SAMQ_HAD(HKV)                                                                                                  \
        do {                                                                                                           \
            if (smem > 48 * 1024)                                                                                      \
                SAMQ_CUDA_TRY(cudaFuncSetAttribute(hadamard_quant_kernel<T, SrcT, HKV>,                                \
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));           \
            hadamard_quant_kernel<T, SrcT, HKV><<<(unsigned)M, threads, smem, st>>>(x, M, K, ldx, pro.row_map, divisor, \
                had->signs, inner, axis, hk, log2_pow, had->hadk, qmax, q, scale, fq, tx, vec);                         \
        } while (0)
        if constexpr (std::is_same<T, __half>::value) {
            // the 1024- and 4096-point transforms with codes only have a kernel of their own
            if (had->mode == SAMQ_HAD_FULL && hk == 1 && (K == 4096 || K == 1024) && vec && divisor == nullptr && fq == nullptr &&
                tx == nullptr && q != nullptr &&
                (!ln_had || (K == 1024 && std::is_same<SrcT, __half>::value && al16(pro.ln_gamma) && al16(pro.ln_beta)))) {
                const __half* g = static_cast<const __half*>(pro.ln_gamma);
                const __half* b = static_cast<const __half*>(pro.ln_beta);
                if (K == 4096) {
                    const int64_t resident = (int64_t)device_sm_count() * 8;                 // 27 KB of shared memory, 121 registers per thread
                    hadamard_4096_r64_kernel<SrcT><<<(unsigned)(M < resident ? M : resident), 64, 0, st>>>(
                        x, M, ldx, pro.row_map, had->signs, qmax, q, scale);
                } else {
                    const int64_t groups = (M + 3) / 4;
                    const int64_t resident = (int64_t)device_sm_count() * (ln_had ? 6 : 8);
                    const unsigned grid = (unsigned)(groups < resident ? groups : resident);
                    if (ln_had) hadamard_1024_r64_kernel<SrcT, true><<<grid, 64, 0, st>>>(x, M, ldx, pro.row_map, had->signs, g, b, pro.ln_eps, qmax, q, scale);
                    else hadamard_1024_r64_kernel<SrcT, false><<<grid, 64, 0, st>>>(x, M, ldx, pro.row_map, had->signs, g, b, 0.f, qmax, q, scale);
                }
                SAMQ_CUDA_TRY(cudaGetLastError());
                return SAMQ_OK;
            }
        }
        if (ln_had)
            return fail(SAMQ_ERR_UNSUPPORTED, "LayerNorm and an online Hadamard are combined only for fp16 rows of 1024 elements with codes as the one output");
        if constexpr (std::is_same<T, __half>::value) {
            // so has the transform across 16 heads
            if (had->mode == SAMQ_HAD_PARTIAL && hk == 1 && axis == 16 && (inner & 7) == 0 && inner <= 128 && vec &&
                had->signs == nullptr && divisor == nullptr && fq == nullptr && tx == nullptr && q != nullptr) {
                if (inner <= 64) {
                    const unsigned grid = (unsigned)((M + 31) / 32);                 // 8 warps x 4 rows
                    hadamard_heads16_quant_kernel<SrcT, 8><<<grid, 256, 0, st>>>(x, M, ldx, pro.row_map, inner, qmax, q, scale);
                } else {
                    const unsigned grid = (unsigned)((M + 15) / 16);                 // 8 warps x 2 rows
                    hadamard_heads16_quant_kernel<SrcT, 16><<<grid, 256, 0, st>>>(x, M, ldx, pro.row_map, inner, qmax, q, scale);
                }
                SAMQ_CUDA_TRY(cudaGetLastError());
                return SAMQ_OK;
            }
        }
        if (hk == 1) SAMQ_HAD(1);
        else if (hk == 12) SAMQ_HAD(12);
        else if (hk == 20) SAMQ_HAD(20);
        else if (hk == 40) SAMQ_HAD(40);
        else SAMQ_HAD(0);
#undef SAMQ_HAD
        SAMQ_CUDA_TRY(cudaGetLastError());
        return SAMQ_OK;
    }
    const float* tensor_absmax = nullptr;
    if (gran == SAMQ_GRAN_TENSOR) {
        if (pro.row_map != nullptr || pro.ln_gamma != nullptr || !std::is_same<T, SrcT>::value)
            return fail(SAMQ_ERR_UNSUPPORTED, "per_tensor quantization takes no gather, LayerNorm or source-type prologue");
        if (workspace == nullptr || workspace_bytes < samq_quant_workspace_bytes(gran))
            return fail(SAMQ_ERR_WORKSPACE, "per_tensor quantization needs %zu bytes of workspace",
                        samq_quant_workspace_bytes(gran));
        SAMQ_CUDA_TRY(cudaMemsetAsync(workspace, 0, sizeof(float), st));
        const int64_t total = M * (int64_t)K;
        int blocks = (int)((total + 256 * 8 - 1) / (256 * 8));
        blocks = blocks < 1 ? 1 : (blocks > 148 * 8 ? 148 * 8 : blocks);
        absmax_kernel<T><<<blocks, 256, 0, st>>>(reinterpret_cast<const T*>(x), M, K, ldx, divisor, static_cast<float*>(workspace));
        SAMQ_CUDA_TRY(cudaGetLastError());
        tensor_absmax = static_cast<const float*>(workspace);
    } else if (gran == SAMQ_GRAN_GROUP) {
        if (group_size <= 0 || K % group_size != 0)
            return fail(SAMQ_ERR_BAD_ARG, "group_size %d must divide K=%d", group_size, K);
    } else if (gran != SAMQ_GRAN_ROW) {
        return fail(SAMQ_ERR_BAD_ARG, "unknown granularity %d", gran);
    }
    return launch_rows<T, SrcT>(x, M, K, ldx, pro, divisor, gran, group_size, tensor_absmax, qmax, q, scale, fq, tx, st);
}

int act_quant_dispatch(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx,
                       const samq_quant_prologue* prologue,
                       const void* divisor, const samq_hadamard_spec* had,
                       int gran, int group_size, int n_bits, int8_t* q, float* scale, void* fq, void* tx,
                       void* workspace, size_t workspace_bytes, void* stream)
{
    if (n_bits < 2 || n_bits > 8) return fail(SAMQ_ERR_UNSUPPORTED, "n_bits=%d: int8 codes hold 2..8 bits", n_bits);
    const float qmax = (float)((1 << (n_bits - 1)) - 1);
    if (M < 0 || K <= 0 || ldx < K) return fail(SAMQ_ERR_BAD_ARG, "bad shape M=%lld K=%lld ldx=%lld",
                                                (long long)M, (long long)K, (long long)ldx);
    if (M > 0 && x == nullptr) return fail(SAMQ_ERR_BAD_ARG, "x is null");
    if (K > (1 << 20)) return fail(SAMQ_ERR_TOO_LARGE, "K=%lld exceeds 2^20", (long long)K);
    if (M > 2147483647LL) return fail(SAMQ_ERR_TOO_LARGE, "M=%lld exceeds 2^31-1", (long long)M);
    Prologue pro = {nullptr, nullptr, nullptr, 0.f};
    int src_dtype = dtype;
    if (prologue != nullptr) {
        pro.row_map = prologue->row_map;
        pro.ln_gamma = prologue->ln_weight;
        pro.ln_beta = prologue->ln_bias;
        pro.ln_eps = prologue->ln_eps;
        if ((pro.ln_gamma == nullptr) != (pro.ln_beta == nullptr))
            return fail(SAMQ_ERR_BAD_ARG, "LayerNorm needs both weight and bias");
        if (prologue->src_dtype >= 0) src_dtype = prologue->src_dtype;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (src_dtype != dtype) {
        if (!(dtype == SAMQ_F16 && src_dtype == SAMQ_BF16))
            return fail(SAMQ_ERR_UNSUPPORTED, "the only mixed pair is bf16 storage read as an fp16 tensor");
        return quant_typed<__half, __nv_bfloat16>((const __nv_bfloat16*)x, M, (int)K, ldx, pro, (const __half*)divisor, had,
                                                  gran, group_size, qmax, q, scale, (__half*)fq, (__half*)tx,
                                                  workspace, workspace_bytes, st);
    }
    switch (dtype) {
    case SAMQ_F16:
        return quant_typed<__half, __half>((const __half*)x, M, (int)K, ldx, pro, (const __half*)divisor, had, gran, group_size,
                                           qmax, q, scale, (__half*)fq, (__half*)tx, workspace, workspace_bytes, st);
    case SAMQ_BF16:
        return quant_typed<__nv_bfloat16, __nv_bfloat16>((const __nv_bfloat16*)x, M, (int)K, ldx, pro, (const __nv_bfloat16*)divisor,
                                                         had, gran, group_size, qmax, q, scale, (__nv_bfloat16*)fq,
                                                         (__nv_bfloat16*)tx, workspace, workspace_bytes, st);
    case SAMQ_F32:
        return quant_typed<float, float>((const float*)x, M, (int)K, ldx, pro, (const float*)divisor, had, gran, group_size,
                                         qmax, q, scale, (float*)fq, (float*)tx, workspace, workspace_bytes, st);
    default:
        return fail(SAMQ_ERR_BAD_ARG, "unknown dtype %d", dtype);
    }
}

// ---------------------------------------------------------------------------
// Per-tensor quantization for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc on the path that runs a
// layer: a plugin loaded into someone else's serving process that was handed
// a fixed arena at start-up, or code running where the allocator is frozen
// (inside a region that forbids allocator traffic).  The per-tensor quantizer
// is the one kernel here that needs scratch beyond its inputs and outputs
// (the running absolute maximum), so this variant keeps that scratch in a
// fixed array that is part of the loaded library image instead of in a
// caller-provided workspace.
//
// Layout of the array: slots [0, kStaticPartials) hold one partial maximum
// per block of 64 rows; slot kStaticPartials holds the reduced maximum.  Every
// GPU that loads the library reserves the 16.4 KB until the process exits.
// ---------------------------------------------------------------------------
constexpr int kStaticRowsPerBlock = 64;
constexpr int kStaticPartials = 4096;                       // => at most 262144 rows per call
constexpr int64_t kStaticMaxRows = (int64_t)kStaticRowsPerBlock * kStaticPartials;

static __device__ __align__(256) float g_static_scratch[kStaticPartials + 64];

// one block reduces |x| over its 64 rows and overwrites its own slot
template <typename T>
__global__ void __launch_bounds__(256)
static_partial_absmax_kernel(const T* __restrict__ x, int64_t M, int K, int64_t ldx, float* __restrict__ partials)
{
    __shared__ float red[8];
    const int64_t r0 = (int64_t)blockIdx.x * kStaticRowsPerBlock;
    const int64_t r1 = (r0 + kStaticRowsPerBlock < M) ? r0 + kStaticRowsPerBlock : M;
    float m = 0.f;
    for (int64_t r = r0 + (threadIdx.x >> 5); r < r1; r += 8)
        for (int c = threadIdx.x & 31; c < K; c += 32)
            m = fmaxf(m, fabsf(Elem<T>::up(x[r * ldx + c])));
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
        t = warp_max(t);
        if (threadIdx.x == 0) partials[blockIdx.x] = t;
    }
}

// a single block folds the partials of this call into the final slot
__global__ void __launch_bounds__(256)
static_reduce_partials_kernel(const float* __restrict__ partials, int n, float* __restrict__ result)
{
    __shared__ float red[8];
    float m = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, partials[i]);
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
        t = warp_max(t);
        if (threadIdx.x == 0) *result = t;
    }
}

// Device address of g_static_scratch for the current device.  In host code the array's
// name is only a handle; the address a kernel can use comes from cudaGetSymbolAddress,
// asked once per device with that device current.
static int static_scratch_address(float** out)
{
    constexpr int kMaxDevices = 64;
    static float* cached[kMaxDevices] = {nullptr};
    int dev = 0;
    SAMQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(SAMQ_ERR_UNSUPPORTED, "device index %d beyond %d", dev, kMaxDevices);
    float* p = __atomic_load_n(&cached[dev], __ATOMIC_ACQUIRE);
    if (p == nullptr) {
        void* addr = nullptr;
        SAMQ_CUDA_TRY(cudaGetSymbolAddress(&addr, g_static_scratch));
        p = static_cast<float*>(addr);
        __atomic_store_n(&cached[dev], p, __ATOMIC_RELEASE);
    }
    *out = p;
    return SAMQ_OK;
}

template <typename T>
static int per_tensor_static_typed(const T* x, int64_t M, int K, int64_t ldx, float qmax,
                                   int8_t* q, float* scale, T* fq, cudaStream_t st)
{
    float* scratch = nullptr;
    int rc = static_scratch_address(&scratch);
    if (rc != SAMQ_OK) return rc;
    const int blocks = (int)((M + kStaticRowsPerBlock - 1) / kStaticRowsPerBlock);
    static_partial_absmax_kernel<T><<<blocks, 256, 0, st>>>(x, M, K, ldx, scratch);
    SAMQ_CUDA_TRY(cudaGetLastError());
    static_reduce_partials_kernel<<<1, 256, 0, st>>>(scratch, blocks, scratch + kStaticPartials);
    SAMQ_CUDA_TRY(cudaGetLastError());
    const Prologue none = {nullptr, nullptr, nullptr, 0.f};
    return launch_rows<T, T>(x, M, K, ldx, none, nullptr, SAMQ_GRAN_TENSOR, 0, scratch + kStaticPartials, qmax,
                             q, scale, fq, nullptr, st);
}

int act_quant_per_tensor_static_dispatch(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx, int n_bits,
                                         int8_t* q, float* scale, void* fq, void* stream)
{
    if (M < 0 || K <= 0 || ldx < K) return fail(SAMQ_ERR_BAD_ARG, "bad shape M=%lld K=%lld ldx=%lld",
                                                (long long)M, (long long)K, (long long)ldx);
    if (M > kStaticMaxRows)
        return fail(SAMQ_ERR_TOO_LARGE, "M=%lld rows exceed the %lld rows the built-in scratch array covers; "
                    "use samq_act_quant_i8 with a caller workspace", (long long)M, (long long)kStaticMaxRows);
    if (K > (1 << 20)) return fail(SAMQ_ERR_TOO_LARGE, "K=%lld exceeds 2^20", (long long)K);
    if (n_bits < 2 || n_bits > 8) return fail(SAMQ_ERR_UNSUPPORTED, "n_bits=%d: int8 codes hold 2..8 bits", n_bits);
    if (M == 0) return SAMQ_OK;
    if (x == nullptr) return fail(SAMQ_ERR_BAD_ARG, "x is null");
    const float qmax = (float)((1 << (n_bits - 1)) - 1);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (dtype) {
    case SAMQ_F16:  return per_tensor_static_typed<__half>((const __half*)x, M, (int)K, ldx, qmax, q, scale, (__half*)fq, st);
    case SAMQ_BF16: return per_tensor_static_typed<__nv_bfloat16>((const __nv_bfloat16*)x, M, (int)K, ldx, qmax, q, scale, (__nv_bfloat16*)fq, st);
    case SAMQ_F32:  return per_tensor_static_typed<float>((const float*)x, M, (int)K, ldx, qmax, q, scale, (float*)fq, st);
    default:        return fail(SAMQ_ERR_BAD_ARG, "unknown dtype %d", dtype);
    }
}


}  // namespace samq
