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

// q = round_half_even( T(x / s) ) as a float holding an integer value
// (`t.div_(scales).round_()`, per_tensor_channel_group.py:60).
template <typename T>
__device__ __forceinline__ float quant_value(float x, float s) {
    return rintf(round_to<T>(__fdiv_rn(x, s)));
}

__device__ __forceinline__ int8_t saturate_i8(float q, float qmax) {
    q = fminf(fmaxf(q, -qmax), qmax);
    return (int8_t)(int)q;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

}  // namespace samq
