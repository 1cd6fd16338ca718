// Shared device/host helpers for the samq kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/samq.h"

namespace samq {

// ---- thread-local error text -------------------------------------------------
char* error_buffer();              // 512 bytes, thread-local (defined in abi.cu)
int fail(int code, const char* fmt, ...);

#define SAMQ_CUDA_TRY(expr)                                                        \
    do {                                                                           \
        cudaError_t _e = (expr);                                                   \
        if (_e != cudaSuccess)                                                     \
            return ::samq::fail(SAMQ_ERR_CUDA, "%s failed: %s", #expr,             \
                                cudaGetErrorString(_e));                           \
    } while (0)

// ---- element-type traits: widen to fp32 and round back exactly once --------
template <typename T> struct Elem;
template <> struct Elem<__half> {
    static __device__ __forceinline__ float up(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half down(float v) { return __float2half_rn(v); }
    static constexpr int kPerVec = 8;   // elements in a 16-byte vector
};
template <> struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float up(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 down(float v) { return __float2bfloat16_rn(v); }
    static constexpr int kPerVec = 8;
};
template <> struct Elem<float> {
    static __device__ __forceinline__ float up(float v) { return v; }
    static __device__ __forceinline__ float down(float v) { return v; }
    static constexpr int kPerVec = 4;
};

// round v to T and widen again: the value a tensor of dtype T would hold
template <typename T>
__device__ __forceinline__ float round_to(float v) { return Elem<T>::up(Elem<T>::down(v)); }

// The reference clamps the absolute maximum with `clamp_(min=1e-5)` in the
// tensor dtype and divides by q_max = 2^(n_bits-1)-1 in that dtype
// (RTN_quantization/per_tensor_channel_group.py:57-59).
template <typename T>
__device__ __forceinline__ float scale_from_absmax(float absmax, float qmax) {
    const float floor_t = round_to<T>(1e-5f);
    float a = fmaxf(absmax, floor_t);
    return round_to<T>(__fdiv_rn(a, qmax));
}

// Division by a scale that is shared by many elements.  x / s is formed as a multiply by the
// correctly rounded reciprocal followed by one residual correction,
//     y0 = x * inv;  e = fma(-y0, s, x);  y = fma(e, inv, y0),
// which yields the correctly rounded IEEE quotient (the classic two-FMA correction of a
// faithful estimate) while keeping the special-function unit out of the per-element path.
struct Divider { float s, inv; };
__device__ __forceinline__ Divider make_divider(float s) { Divider d; d.s = s; d.inv = __frcp_rn(s); return d; }
__device__ __forceinline__ float div_exact(float x, const Divider& d) {
    const float y0 = x * d.inv;
    const float e = fmaf(-y0, d.s, x);
    return fmaf(e, d.inv, y0);
}

// round-half-even to an integer for |v| < 2^22 by adding and subtracting 1.5 * 2^23
constexpr float kRoundMagic = 12582912.0f;
// The sign is taken from `sign_src` (the dividend: the scale is positive), so that -0.4 and
// -0.0 round to -0.0 as the reference's div_().round_() does.
__device__ __forceinline__ float rint_small(float v, float sign_src) {
    const float r = (v + kRoundMagic) - kRoundMagic;
    return __int_as_float(__float_as_int(r) | (__float_as_int(sign_src) & 0x80000000));
}

// q = round_half_even( T(x / s) ) as a float holding an integer value
// (`t.div_(scales).round_()`, per_tensor_channel_group.py:60).
template <typename T>
__device__ __forceinline__ float quant_value(float x, const Divider& d) {
    return rint_small(round_to<T>(div_exact(x, d)), x);
}

// two's-complement byte of an integer-valued float clamped to [-qmax, qmax]
__device__ __forceinline__ uint32_t code_byte(float q, float qmax) {
    q = fminf(fmaxf(q, -qmax), qmax);
    return (uint32_t)__float_as_int(q + kRoundMagic) & 0xFFu;
}
__device__ __forceinline__ int8_t saturate_i8(float q, float qmax) { return (int8_t)code_byte(q, qmax); }

// round every element of a vector to T (RNE) and widen again, two elements per conversion
template <typename T, int E> struct RoundVec;
template <int E> struct RoundVec<__half, E> {
    static __device__ __forceinline__ void run(float (&f)[E]) {
#pragma unroll
        for (int i = 0; i < E; i += 2) { float2 t = __half22float2(__floats2half2_rn(f[i], f[i + 1])); f[i] = t.x; f[i + 1] = t.y; }
    }
};
template <int E> struct RoundVec<__nv_bfloat16, E> {
    static __device__ __forceinline__ void run(float (&f)[E]) {
#pragma unroll
        for (int i = 0; i < E; i += 2) { float2 t = __bfloat1622float2(__floats2bfloat162_rn(f[i], f[i + 1])); f[i] = t.x; f[i + 1] = t.y; }
    }
};
template <int E> struct RoundVec<float, E> {
    static __device__ __forceinline__ void run(float (&)[E]) {}
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

}  // namespace samq
