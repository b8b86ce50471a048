// Per-row, per-128-column dynamic FP8 e4m3 quantisation (bandwidth kernel).
// Rounding sequence of the reference's torch oracle (aiter/ops/quant.py:64-94):
//   amax -> scale = amax / 448 (IEEE division; 0 -> 1) -> code = RNE_e4m3(x / scale) (IEEE division)
// so the codes and scales are bit-identical to it.  The reference's HIP kernel multiplies by
// reciprocals instead (csrc/kernels/quant_kernels.cu:121,159-160), which is not.
//
// 16 lanes own one 128-element group (8 bf16 = one 16-byte load each), two groups per warp.

#include <algorithm>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "quant_device.cuh"

namespace b200 {
namespace {

constexpr int kQuantThreads = 256;
constexpr int kGroupsPerBlock = kQuantThreads / 16;

// num_rows (optional, device): only the first *num_rows * rows_factor rows are quantised. transposed: the scale of
// group (row, col-group) goes to scales[col-group * rows_used + row] instead of scales[row * groups_per_row + col-group]
// (the layout the reference's 1-stage path reads, csrc/kernels/quant_kernels.cu:143-146; rows_used = the dynamic
// row count when num_rows is given, as there).
template <bool F16>
__global__ void __launch_bounds__(kQuantThreads) quant_1x128_kernel(
    const uint4* __restrict__ x, uint2* __restrict__ q, float* __restrict__ scales, int64_t groups, int groups_per_row,
    const int* __restrict__ num_rows, int rows_factor, int transposed) {
    const int64_t g = (int64_t)blockIdx.x * kGroupsPerBlock + (threadIdx.x >> 4);
    const int sub = threadIdx.x & 15;
    int64_t rows_used = groups / groups_per_row;
    if (num_rows) rows_used = min(rows_used, (int64_t)*num_rows * rows_factor);
    const bool live = g < rows_used * groups_per_row;
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (live) raw = __ldg(x + g * 16 + sub);
    uint2 codes;
    const float scale = quant_group16<F16>(raw, codes);
    if (live) {
        q[g * 16 + sub] = codes;
        if (sub == 0) {
            const int64_t row = g / groups_per_row, cg = g - row * groups_per_row;
            scales[transposed ? cg * rows_used + row : g] = scale;
        }
    }
}

// Per-row dynamic FP8 quantisation over the whole row (QuantType.per_Token): one CTA per row, the row is
// kept in shared memory between the amax pass and the conversion pass. Same rounding sequence as above
// (aiter/ops/quant.py:64-94 over the last dimension). Rows >= *row_limit (if given) are skipped.
template <bool F16>
__global__ void __launch_bounds__(256) quant_per_token_kernel(const uint4* __restrict__ x, uint2* __restrict__ q,
                                                              float* __restrict__ scales, int cols8,
                                                              const int* __restrict__ row_limit, int rows_factor) {
    extern __shared__ uint4 row_s[];
    __shared__ float red[8];
    const int64_t row = blockIdx.x;
    if (row_limit && row >= (int64_t)*row_limit * rows_factor) return;
    float amax = 0.f;
    for (int i = threadIdx.x; i < cols8; i += blockDim.x) {
        const uint4 raw = __ldg(x + row * cols8 + i);
        row_s[i] = raw;
        float v[8];
        unpack8<F16>(raw, v);
#pragma unroll
        for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(v[k]));
    }
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) amax = fmaxf(amax, red[k]);
    float scale = __fdiv_rn(amax, 448.0f);
    if (scale == 0.f) scale = 1.f;
    for (int i = threadIdx.x; i < cols8; i += blockDim.x) {
        const uint4 raw = row_s[i];
        float v[8];
        unpack8<F16>(raw, v);
        uint32_t w[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(v[4 * k], scale), __fdiv_rn(v[4 * k + 1], scale)),
                                                         __NV_SATFINITE, __NV_E4M3);
            const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(v[4 * k + 2], scale), __fdiv_rn(v[4 * k + 3], scale)),
                                                         __NV_SATFINITE, __NV_E4M3);
            w[k] = lo | (hi << 16);
        }
        q[row * cols8 + i] = make_uint2(w[0], w[1]);
    }
    if (threadIdx.x == 0) scales[row] = scale;
}

// Per-tensor dynamic FP8 quantisation (QuantType.per_Tensor; torch twin per_tensor_quant, aiter/ops/quant.py:318-328:
// scale = max|x| / 448 and codes = RNE_e4m3(x / scale), both IEEE divisions, no zero guard). Two passes:
// the maximum over the rows below *row_limit goes to amax[0] (non-negative floats order like their bit patterns,
// so an integer atomicMax does it), then every row is converted with the one scale, which is also written to
// scale[0] and, if asked, once per row to row_scales (the GEMM kernels take one activation scale per row).
template <bool F16>
__global__ void __launch_bounds__(256) amax_kernel(const uint4* __restrict__ x, int64_t rows, int cols8,
                                                   const int* __restrict__ row_limit, unsigned int* __restrict__ amax) {
    const int64_t limit = row_limit ? min((int64_t)*row_limit, rows) : rows;
    const int64_t n = limit * cols8;
    float m = 0.f;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const uint4 raw = __ldg(x + i);
        float v[8];
        unpack8<F16>(raw, v);
#pragma unroll
        for (int k = 0; k < 8; ++k) m = fmaxf(m, fabsf(v[k]));
    }
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    if ((threadIdx.x & 31) == 0 && m > 0.f) atomicMax(amax, __float_as_uint(m));
}

template <bool F16>
__global__ void __launch_bounds__(256) quant_per_tensor_kernel(const uint4* __restrict__ x, uint2* __restrict__ q,
                                                               float* __restrict__ scale_out, float* __restrict__ row_scales,
                                                               int64_t rows, int cols8, const int* __restrict__ row_limit,
                                                               const unsigned int* __restrict__ amax) {
    const int64_t limit = row_limit ? min((int64_t)*row_limit, rows) : rows;
    const float scale = __fdiv_rn(__uint_as_float(*amax), 448.0f);
    if (blockIdx.x == 0 && threadIdx.x == 0) scale_out[0] = scale;
    const int64_t n = limit * cols8;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const uint4 raw = __ldg(x + i);
        float v[8];
        unpack8<F16>(raw, v);
        uint32_t w[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(v[4 * k], scale), __fdiv_rn(v[4 * k + 1], scale)),
                                                         __NV_SATFINITE, __NV_E4M3);
            const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(v[4 * k + 2], scale), __fdiv_rn(v[4 * k + 3], scale)),
                                                         __NV_SATFINITE, __NV_E4M3);
            w[k] = lo | (hi << 16);
        }
        q[i] = make_uint2(w[0], w[1]);
    }
    if (row_scales)
        for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += (int64_t)gridDim.x * blockDim.x)
            row_scales[r] = scale;
}

}  // namespace

// input dtype of the three quantisers: bf16 or fp16 (the reference takes either, aiter/fused_moe.py:752-756)
static bool input_is_f16(const aiter_tensor_t* input) {
    B200_CHECK(input != nullptr, "input must not be NULL");
    B200_CHECK(input->dtype_ == AITER_DTYPE_bf16 || input->dtype_ == AITER_DTYPE_fp16,
               "input must be bf16 or fp16, got dtype code ", input->dtype_);
    return input->dtype_ == AITER_DTYPE_fp16;
}

void launch_quant_per_tensor(aiter_tensor_t* out, const aiter_tensor_t* input, aiter_tensor_t* scale, aiter_tensor_t* amax,
                             aiter_tensor_t* row_scales, const aiter_tensor_t* row_limit, cudaStream_t stream) {
    const bool f16 = input_is_f16(input);
    check_tensor(input, "input", -1, 2);
    check_tensor(out, "out", AITER_DTYPE_fp8, 2);
    check_tensor(scale, "scale", AITER_DTYPE_fp32, -1);
    check_tensor(amax, "amax", AITER_DTYPE_fp32, -1);
    const int64_t rows = input->shape[0], cols = input->shape[1];
    B200_CHECK(cols % 8 == 0 && cols >= 8, "row length must be a multiple of 8, got ", cols);
    B200_CHECK(out->shape[0] == rows && out->shape[1] == cols, "out must have the shape of input");
    B200_CHECK(scale->numel_ >= 1 && amax->numel_ >= 1, "scale and amax need one element each");
    B200_CHECK(((uintptr_t)input->ptr & 15) == 0 && ((uintptr_t)out->ptr & 7) == 0, "input must be 16-byte and out 8-byte aligned");
    if (row_scales) {
        check_tensor(row_scales, "row_scales", AITER_DTYPE_fp32, -1);
        B200_CHECK((int64_t)row_scales->numel_ >= rows, "row_scales needs one element per row");
    }
    if (row_limit) check_tensor(row_limit, "row_limit", AITER_DTYPE_i32, -1);
    B200_CUDA(cudaMemsetAsync(amax->ptr, 0, sizeof(float), stream));
    if (rows == 0) return;
    const int64_t n = rows * (cols / 8);
    const int grid = (int)std::min<int64_t>((n + 255) / 256, (int64_t)sm_count(input->device_id) * 8);
    const int* lim = row_limit ? (const int*)row_limit->ptr : nullptr;
    if (f16) {
        amax_kernel<true><<<grid, 256, 0, stream>>>((const uint4*)input->ptr, rows, (int)(cols / 8), lim, (unsigned int*)amax->ptr);
        quant_per_tensor_kernel<true><<<grid, 256, 0, stream>>>((const uint4*)input->ptr, (uint2*)out->ptr, (float*)scale->ptr,
                                                                row_scales ? (float*)row_scales->ptr : nullptr, rows,
                                                                (int)(cols / 8), lim, (const unsigned int*)amax->ptr);
    } else {
        amax_kernel<false><<<grid, 256, 0, stream>>>((const uint4*)input->ptr, rows, (int)(cols / 8), lim, (unsigned int*)amax->ptr);
        quant_per_tensor_kernel<false><<<grid, 256, 0, stream>>>((const uint4*)input->ptr, (uint2*)out->ptr, (float*)scale->ptr,
                                                                 row_scales ? (float*)row_scales->ptr : nullptr, rows,
                                                                 (int)(cols / 8), lim, (const unsigned int*)amax->ptr);
    }
    B200_CUDA(cudaGetLastError());
}

void launch_quant_per_token(aiter_tensor_t* out, const aiter_tensor_t* input, aiter_tensor_t* scales,
                            const aiter_tensor_t* row_limit, int rows_factor, cudaStream_t stream) {
    const bool f16 = input_is_f16(input);
    check_tensor(input, "input", -1, 2);
    check_tensor(out, "out", AITER_DTYPE_fp8, 2);
    check_tensor(scales, "scales", AITER_DTYPE_fp32, -1);
    const int64_t rows = input->shape[0], cols = input->shape[1];
    B200_CHECK(cols % 8 == 0 && cols >= 8, "row length must be a multiple of 8, got ", cols);
    B200_CHECK(cols * 2 <= 200 * 1024, "row too long for the shared-memory row cache: ", cols);
    B200_CHECK(out->shape[0] == rows && out->shape[1] == cols, "out must have the shape of input");
    B200_CHECK((int64_t)scales->numel_ >= rows, "scales needs one element per row");
    B200_CHECK(((uintptr_t)input->ptr & 15) == 0 && ((uintptr_t)out->ptr & 7) == 0, "input must be 16-byte and out 8-byte aligned");
    B200_CHECK(rows_factor >= 1, "num_rows_factor must be >= 1, got ", rows_factor);
    if (row_limit) check_tensor(row_limit, "num_rows", AITER_DTYPE_i32, -1);
    if (rows == 0) return;
    const size_t smem = (size_t)cols * 2;
    static bool attr_set[64] = {false};
    const int dev = input->device_id;
    if (dev >= 64 || !attr_set[dev]) {
        B200_CUDA(cudaFuncSetAttribute(quant_per_token_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        B200_CUDA(cudaFuncSetAttribute(quant_per_token_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        if (dev < 64) attr_set[dev] = true;
    }
    const int* lim = row_limit ? (const int*)row_limit->ptr : nullptr;
    if (f16)
        quant_per_token_kernel<true><<<(unsigned)rows, 256, smem, stream>>>((const uint4*)input->ptr, (uint2*)out->ptr,
                                                                             (float*)scales->ptr, (int)(cols / 8), lim, rows_factor);
    else
        quant_per_token_kernel<false><<<(unsigned)rows, 256, smem, stream>>>((const uint4*)input->ptr, (uint2*)out->ptr,
                                                                              (float*)scales->ptr, (int)(cols / 8), lim, rows_factor);
    B200_CUDA(cudaGetLastError());
}

void launch_quant_1x128(aiter_tensor_t* out, const aiter_tensor_t* input, aiter_tensor_t* scales,
                        const aiter_tensor_t* num_rows, int rows_factor, int transpose_scale, cudaStream_t stream) {
    const bool f16 = input_is_f16(input);
    check_tensor(input, "input", -1, -1);
    check_tensor(out, "out", AITER_DTYPE_fp8, -1);
    check_tensor(scales, "scales", AITER_DTYPE_fp32, -1);
    B200_CHECK(input->ndim >= 1, "input must have at least one dimension");
    const int64_t cols = input->shape[input->ndim - 1];
    B200_CHECK(cols % 128 == 0, "last dimension must be a multiple of 128, got ", cols);
    B200_CHECK(out->numel_ == input->numel_, "out must have as many elements as input");
    const int64_t groups = (int64_t)input->numel_ / 128;
    B200_CHECK((int64_t)scales->numel_ >= groups, "scales needs ", groups, " elements, has ",
               scales->numel_);
    B200_CHECK(((uintptr_t)input->ptr & 15) == 0 && ((uintptr_t)out->ptr & 7) == 0,
               "input must be 16-byte and out 8-byte aligned");
    B200_CHECK(rows_factor >= 1, "num_rows_factor must be >= 1, got ", rows_factor);
    if (num_rows) check_tensor(num_rows, "num_rows", AITER_DTYPE_i32, -1);
    if (groups == 0) return;
    const int64_t blocks = (groups + kGroupsPerBlock - 1) / kGroupsPerBlock;
    B200_CHECK(blocks < ((int64_t)1 << 31), "input too large");
    const int* lim = num_rows ? (const int*)num_rows->ptr : nullptr;
    if (f16)
        quant_1x128_kernel<true><<<(unsigned)blocks, kQuantThreads, 0, stream>>>(
            (const uint4*)input->ptr, (uint2*)out->ptr, (float*)scales->ptr, groups, (int)(cols / 128), lim, rows_factor,
            transpose_scale);
    else
        quant_1x128_kernel<false><<<(unsigned)blocks, kQuantThreads, 0, stream>>>(
            (const uint4*)input->ptr, (uint2*)out->ptr, (float*)scales->ptr, groups, (int)(cols / 128), lim, rows_factor,
            transpose_scale);
    B200_CUDA(cudaGetLastError());
}

}  // namespace b200
