// Pieces shared by the int8 GEMM kernels: epilogue math, output-type traits and the host-side
// tensor-map builders.
#pragma once

#include "common.cuh"
#include "tcgen05.cuh"
#include <string.h>
#include <type_traits>

namespace samq {
namespace gemm {

constexpr int BK = 128;            // bytes (= int8 elements) of K per stage: one 128-byte swizzle row

// Exact (erf) GELU, x * Phi(x), with one exp2, no division and no branch:
//   0.5 * erfc(u / sqrt 2) = 2^Q(u),  u = min(|x|, 6.08),  Q a degree-6 polynomial fitted on [0, 6.08]
//   (beyond that the tail is below 1e-9), and  gelu(x) = max(x, 0) - |x| * 2^Q(u).
// Absolute error < 3e-7, relative < 2e-5 — two orders below fp16 resolution — in 10 instructions,
// which matters because the epilogue of a K = 1280 tile has only ~20 issue slots per output.
__device__ __forceinline__ float gelu_erf(float x) {
    const float u = fminf(fabsf(x), 6.08f);
    float q = 3.586083039e-05f;
    q = fmaf(q, u, -7.942179800e-04f);
    q = fmaf(q, u, 8.166280575e-03f);
    q = fmaf(q, u, -5.355186760e-02f);
    q = fmaf(q, u, -4.586586654e-01f);
    q = fmaf(q, u, -1.151242375e+00f);
    q = fmaf(q, u, -9.999881387e-01f);
    float h;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(h) : "f"(q));
    return fmaf(-fabsf(x), h, fmaxf(x, 0.f));
}

// The same function on two values at once: the polynomial and the final multiply-add run as
// packed fp32x2 FMAs (same roundings as the scalar form, so the results are identical).
__device__ __forceinline__ float2 gelu_erf2(float2 x) {
    const float2 u = make_float2(fminf(fabsf(x.x), 6.08f), fminf(fabsf(x.y), 6.08f));
    float2 q = make_float2(3.586083039e-05f, 3.586083039e-05f);
    q = __ffma2_rn(q, u, make_float2(-7.942179800e-04f, -7.942179800e-04f));
    q = __ffma2_rn(q, u, make_float2(8.166280575e-03f, 8.166280575e-03f));
    q = __ffma2_rn(q, u, make_float2(-5.355186760e-02f, -5.355186760e-02f));
    q = __ffma2_rn(q, u, make_float2(-4.586586654e-01f, -4.586586654e-01f));
    q = __ffma2_rn(q, u, make_float2(-1.151242375e+00f, -1.151242375e+00f));
    q = __ffma2_rn(q, u, make_float2(-9.999881387e-01f, -9.999881387e-01f));
    float2 h;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(h.x) : "f"(q.x));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(h.y) : "f"(q.y));
    return __ffma2_rn(make_float2(-fabsf(x.x), -fabsf(x.y)), h, make_float2(fmaxf(x.x, 0.f), fmaxf(x.y, 0.f)));
}

// y[j] = float(acc[j]) * a_s * w[j] + b[j] for 32 accumulator columns, two columns per instruction
// (the multiply and the fused multiply-add round exactly as their scalar forms do)
__device__ __forceinline__ void dequant32(const uint32_t (&r)[32], float a_s, const float* __restrict__ ws,
                                          const float* __restrict__ bs, float (&y)[32]) {
    const float2 a2 = make_float2(a_s, a_s);
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
        const float4 w4 = *reinterpret_cast<const float4*>(ws + j);
        const float4 b4 = *reinterpret_cast<const float4*>(bs + j);
        const float2 lo = __ffma2_rn(__fmul2_rn(make_float2(__int2float_rn((int)r[j + 0]), __int2float_rn((int)r[j + 1])), a2),
                                     make_float2(w4.x, w4.y), make_float2(b4.x, b4.y));
        const float2 hi = __ffma2_rn(__fmul2_rn(make_float2(__int2float_rn((int)r[j + 2]), __int2float_rn((int)r[j + 3])), a2),
                                     make_float2(w4.z, w4.w), make_float2(b4.z, b4.w));
        y[j + 0] = lo.x; y[j + 1] = lo.y; y[j + 2] = hi.x; y[j + 3] = hi.y;
    }
}

__device__ __forceinline__ void gelu32(float (&y)[32]) {
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
        const float2 g = gelu_erf2(make_float2(y[j], y[j + 1]));
        y[j] = g.x; y[j + 1] = g.y;
    }
}

template <typename OutT> struct OutOps;
template <> struct OutOps<__half> {
    static __device__ __forceinline__ float up(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half down(float v) { return __float2half_rn(v); }
    // 32 values -> four 16-byte vectors, two values per conversion
    static __device__ __forceinline__ void pack32(const float (&y)[32], uint4 (&packed)[4]) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const __half2 h = __floats2half2_rn(y[8 * j + 2 * e], y[8 * j + 2 * e + 1]);
                w[e] = *reinterpret_cast<const uint32_t*>(&h);
            }
            packed[j] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
};
template <> struct OutOps<__nv_bfloat16> {
    static __device__ __forceinline__ float up(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 down(float v) { return __float2bfloat16_rn(v); }
    static __device__ __forceinline__ void pack32(const float (&y)[32], uint4 (&packed)[4]) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(y[8 * j + 2 * e], y[8 * j + 2 * e + 1]);
                w[e] = *reinterpret_cast<const uint32_t*>(&h);
            }
            packed[j] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
};
template <> struct OutOps<float> {
    static __device__ __forceinline__ float up(float v) { return v; }
    static __device__ __forceinline__ float down(float v) { return v; }
    static __device__ __forceinline__ void pack32(const float (&y)[32], uint4 (&packed)[8]) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
            packed[j] = make_uint4(__float_as_uint(y[4 * j]), __float_as_uint(y[4 * j + 1]), __float_as_uint(y[4 * j + 2]), __float_as_uint(y[4 * j + 3]));
    }
};

// ---- host side -----------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(ptr);
    }();
    return fn;
}

// [rows, K] int8 row-major with row stride ld bytes; box = box_rows x 128 bytes, 128-byte swizzle, zero fill.
inline int make_operand_map(CUtensorMap* map, const int8_t* base, int64_t rows, int64_t K, int64_t ld, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return fail(SAMQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SAMQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return SAMQ_OK;
}

inline int sm_count() {
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

// [M, N] output with row stride ldo elements of esize bytes; box = 32 rows x 64 bytes, 64-byte swizzle.
inline int make_out_map(CUtensorMap* map, void* base, int64_t M, int64_t N, int64_t ldo, int esize) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return fail(SAMQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
    cuuint64_t strides[1] = {(cuuint64_t)(ldo * esize)};
    cuuint32_t box[2] = {(cuuint32_t)(64 / esize), 32u};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, esize == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, base, dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                    CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SAMQ_ERR_CUDA, "cuTensorMapEncodeTiled (output) failed with CUresult %d", (int)r);
    return SAMQ_OK;
}


}  // namespace gemm
}  // namespace samq
