// The packed int4 path of the reference's native extension
// (quant/qgemm/kernels/quant.cu:11-97, bindings.cpp:7-91, gemm.cu:6-45):
//
//   sym_quant   : q = clamp(round_half_even(half(x / scale[row])), -8, 7), two codes per byte,
//                 element 2j in the low nibble of byte j (cutlass::int4b_t storage order)
//   matmul      : C[m,n] = sum_k A[m,k] * B[n,k], int32, from the packed operands
//   sym_dequant : y = (scale_row[m] * scale_col[n]) * half(C[m,n]), every product rounded to fp16
//
// Blackwell's tcgen05 tensor cores have no 4-bit integer kind (kind::i8 is the narrowest integer
// operand), so the packed form is a storage format here: it halves what a weight occupies in a
// checkpoint and in HBM, and the codes are widened to int8 on the way into the GEMM.  Widening
// inside the GEMM's shared-memory pipeline was not built: expanding both operands on chip would
// add more shared-memory traffic (write 48 KB + read 24 KB per stage) than the int8 operands the
// tensor core reads (48 KB per stage) and the pipeline is already within 25 % of that bandwidth.
#include "common.cuh"

namespace samq {

namespace {

__device__ __forceinline__ int quant4(__half x, __half s) {
    const int q = __half2int_rn(__hdiv(x, s));
    return q < -8 ? -8 : (q > 7 ? 7 : q);
}

// one thread: 8 source elements (16 bytes) -> 4 packed bytes
__global__ void __launch_bounds__(256)
sym_quant_i4_kernel(const __half* __restrict__ x, const __half* __restrict__ scale, int64_t rows, int64_t cols, int64_t ldx,
                    int64_t cols_dst, uint8_t* __restrict__ q, int vec_ok)
{
    const int64_t words_per_row = (cols_dst + 3) / 4;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * words_per_row) return;
    const int64_t row = idx / words_per_row, w = idx - row * words_per_row;
    const __half s = scale[row];
    const __half* xr = x + row * ldx + w * 8;
    uint8_t* qr = q + row * cols_dst + w * 4;
    const int64_t left = cols - w * 8;
    if (vec_ok && left >= 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(xr);
        const __half* h = reinterpret_cast<const __half*>(&raw);
        uint32_t packed = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) packed |= (uint32_t)(quant4(h[i], s) & 0xF) << (4 * i);
        *reinterpret_cast<uint32_t*>(qr) = packed;
    } else {
        for (int b = 0; b < 4 && w * 4 + b < cols_dst; ++b) {
            uint32_t byte = 0;
            for (int i = 0; i < 2; ++i)
                if (2 * b + i < left) byte |= (uint32_t)(quant4(xr[2 * b + i], s) & 0xF) << (4 * i);
            qr[b] = (uint8_t)byte;
        }
    }
}

// one thread: 4 packed bytes -> 8 int8 codes (sign-extended)
__global__ void __launch_bounds__(256)
unpack_i4_kernel(const uint8_t* __restrict__ q, int64_t rows, int64_t cols, int64_t ldq, int8_t* __restrict__ out, int64_t ldo, int vec_ok)
{
    const int64_t cols_src = (cols + 1) / 2;
    const int64_t words_per_row = (cols_src + 3) / 4;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * words_per_row) return;
    const int64_t row = idx / words_per_row, w = idx - row * words_per_row;
    const uint8_t* qr = q + row * ldq + w * 4;
    int8_t* o = out + row * ldo + w * 8;
    const int64_t left = cols - w * 8;
    if (vec_ok && left >= 8) {
        const uint32_t p = *reinterpret_cast<const uint32_t*>(qr);
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            lo |= (uint32_t)(uint8_t)(((int32_t)(p << (28 - 4 * i))) >> 28) << (8 * i);
            hi |= (uint32_t)(uint8_t)(((int32_t)(p << (12 - 4 * i))) >> 28) << (8 * i);
        }
        *reinterpret_cast<uint2*>(o) = make_uint2(lo, hi);
    } else {
        for (int i = 0; i < 8 && i < left; ++i) {
            const uint32_t byte = qr[i >> 1];
            o[i] = (int8_t)(((int32_t)(byte << (28 - 4 * (i & 1)))) >> 28);
        }
    }
}

// one thread: 8 int8 codes (each in [-8, 7]) -> 4 packed bytes
__global__ void __launch_bounds__(256)
pack_i4_kernel(const int8_t* __restrict__ codes, int64_t rows, int64_t cols, int64_t ldc, uint8_t* __restrict__ q, int64_t ldq)
{
    const int64_t cols_dst = (cols + 1) / 2;
    const int64_t words_per_row = (cols_dst + 3) / 4;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * words_per_row) return;
    const int64_t row = idx / words_per_row, w = idx - row * words_per_row;
    const int8_t* c = codes + row * ldc + w * 8;
    const int64_t left = cols - w * 8;
    for (int b = 0; b < 4 && w * 4 + b < cols_dst; ++b) {
        uint32_t byte = 0;
        for (int i = 0; i < 2; ++i)
            if (2 * b + i < left) byte |= ((uint32_t)c[2 * b + i] & 0xFu) << (4 * i);
        q[row * ldq + w * 4 + b] = (uint8_t)byte;
    }
}

__global__ void __launch_bounds__(256)
sym_dequant_i32_kernel(const int32_t* __restrict__ q, const __half* __restrict__ scale_row, const __half* __restrict__ scale_col,
                       int64_t rows, int64_t cols, __half* __restrict__ out)
{
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * cols) return;
    const int64_t row = idx / cols, col = idx - row * cols;
    out[idx] = __hmul(__hmul(scale_row[row], scale_col[col]), __int2half_rn(q[idx]));
}

unsigned blocks_for(int64_t n) { return (unsigned)((n + 255) / 256); }

}  // namespace

int sym_quant_i4_dispatch(const void* x, const void* scale, int64_t rows, int64_t cols, int64_t ldx, uint8_t* q, void* stream)
{
    if (rows < 0 || cols <= 0 || ldx < cols) return fail(SAMQ_ERR_BAD_ARG, "bad shape rows=%lld cols=%lld ldx=%lld", (long long)rows, (long long)cols, (long long)ldx);
    if (rows == 0) return SAMQ_OK;
    if (x == nullptr || scale == nullptr || q == nullptr) return fail(SAMQ_ERR_BAD_ARG, "null pointer");
    const int64_t cols_dst = (cols + 1) / 2;
    const int vec_ok = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && (ldx % 8 == 0) && ((reinterpret_cast<uintptr_t>(q) & 3) == 0) && (cols_dst % 4 == 0);
    const int64_t n = rows * ((cols_dst + 3) / 4);
    sym_quant_i4_kernel<<<blocks_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(x), static_cast<const __half*>(scale), rows, cols, ldx, cols_dst, q, vec_ok);
    SAMQ_CUDA_TRY(cudaGetLastError());
    return SAMQ_OK;
}

int unpack_i4_dispatch(const uint8_t* q, int64_t rows, int64_t cols, int64_t ldq, int8_t* out, int64_t ldo, void* stream)
{
    if (rows < 0 || cols <= 0 || ldq < (cols + 1) / 2 || ldo < cols) return fail(SAMQ_ERR_BAD_ARG, "bad shape rows=%lld cols=%lld", (long long)rows, (long long)cols);
    if (rows == 0) return SAMQ_OK;
    if (q == nullptr || out == nullptr) return fail(SAMQ_ERR_BAD_ARG, "null pointer");
    const int vec_ok = ((reinterpret_cast<uintptr_t>(q) & 3) == 0) && (ldq % 4 == 0) && ((reinterpret_cast<uintptr_t>(out) & 7) == 0) && (ldo % 8 == 0);
    const int64_t n = rows * (((cols + 1) / 2 + 3) / 4);
    unpack_i4_kernel<<<blocks_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(q, rows, cols, ldq, out, ldo, vec_ok);
    SAMQ_CUDA_TRY(cudaGetLastError());
    return SAMQ_OK;
}

int pack_i4_dispatch(const int8_t* codes, int64_t rows, int64_t cols, int64_t ldc, uint8_t* q, int64_t ldq, void* stream)
{
    if (rows < 0 || cols <= 0 || ldc < cols || ldq < (cols + 1) / 2) return fail(SAMQ_ERR_BAD_ARG, "bad shape rows=%lld cols=%lld", (long long)rows, (long long)cols);
    if (rows == 0) return SAMQ_OK;
    if (codes == nullptr || q == nullptr) return fail(SAMQ_ERR_BAD_ARG, "null pointer");
    const int64_t n = rows * (((cols + 1) / 2 + 3) / 4);
    pack_i4_kernel<<<blocks_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(codes, rows, cols, ldc, q, ldq);
    SAMQ_CUDA_TRY(cudaGetLastError());
    return SAMQ_OK;
}

int sym_dequant_i32_dispatch(const int32_t* q, const void* scale_row, const void* scale_col, int64_t rows, int64_t cols, void* out, void* stream)
{
    if (rows < 0 || cols < 0) return fail(SAMQ_ERR_BAD_ARG, "bad shape rows=%lld cols=%lld", (long long)rows, (long long)cols);
    if (rows == 0 || cols == 0) return SAMQ_OK;
    if (q == nullptr || scale_row == nullptr || scale_col == nullptr || out == nullptr) return fail(SAMQ_ERR_BAD_ARG, "null pointer");
    sym_dequant_i32_kernel<<<blocks_for(rows * cols), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        q, static_cast<const __half*>(scale_row), static_cast<const __half*>(scale_col), rows, cols, static_cast<__half*>(out));
    SAMQ_CUDA_TRY(cudaGetLastError());
    return SAMQ_OK;
}

}  // namespace samq
