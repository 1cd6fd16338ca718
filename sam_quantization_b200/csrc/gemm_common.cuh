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

template <typename OutT> struct OutOps;
template <> struct OutOps<__half> {
    static __device__ __forceinline__ float up(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half down(float v) { return __float2half_rn(v); }
};
template <> struct OutOps<__nv_bfloat16> {
    static __device__ __forceinline__ float up(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 down(float v) { return __float2bfloat16_rn(v); }
};
template <> struct OutOps<float> {
    static __device__ __forceinline__ float up(float v) { return v; }
    static __device__ __forceinline__ float down(float v) { return v; }
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
