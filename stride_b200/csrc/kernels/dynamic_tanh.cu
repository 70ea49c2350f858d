// Dynamic Tanh norm fused with the residual sum, and the scaled residual sum on its own.
//
// The norm computes no statistic: y = tanh(alpha * x) * w + b per element, with a scalar alpha. For row r
// (source row s = rows ? rows[r] : r):
//   x = residual[s] + scale * delta[s]     (float32; delta may be absent)
//   residual[s] = x                        (only when rows == nullptr)
//   out[r] = tanh(alpha * x) * w + b       (float32, one rounding at the end)
// `scale` is the multiplier an architecture puts on every sum into its stream (1 where it has none).
#include "common.cuh"

namespace stride {

template <typename T>
__global__ void add_dyt_kernel(float* __restrict__ residual, const T* __restrict__ delta, float scale,
                               const float* __restrict__ weight, const float* __restrict__ bias, float alpha,
                               T* __restrict__ out, const int32_t* __restrict__ rows, int hidden) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const size_t s = rows ? static_cast<size_t>(rows[r]) : static_cast<size_t>(r);
    float* res = residual + s * hidden;
    const T* del = delta ? delta + s * hidden : nullptr;
    T* dst = out + static_cast<size_t>(r) * hidden;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < hidden; i += gridDim.y * blockDim.x) {
        float x = res[i];
        if (del) {
            x = __fmaf_rn(scale, to_f32(del[i]), x);
            if (!rows) res[i] = x;
        }
        dst[i] = from_f32<T>(__fmaf_rn(tanhf(alpha * x), weight[i], bias[i]));
    }
}

template <typename T>
__global__ void add_scaled_kernel(float* __restrict__ residual, const T* __restrict__ delta, float scale, size_t n) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x)
        residual[i] = __fmaf_rn(scale, to_f32(delta[i]), residual[i]);
}

}  // namespace stride

using namespace stride;

extern "C" {

int stride_add_dyt(float* residual, const void* delta, float scale, const float* weight, const float* bias, float alpha,
                   void* out, const int32_t* rows, int num_rows, int hidden, int dtype, cudaStream_t stream) {
    if (num_rows < 0 || hidden <= 0) return STRIDE_BAD_ARGUMENT;
    if (num_rows == 0) return 0;
    const int threads = 256;
    const int per_row = hidden >= 4096 ? 4 : (hidden >= 1024 ? 2 : 1);
    const dim3 grid(num_rows, per_row);
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(add_dyt_kernel<float>, grid, dim3(threads), 0, stream, residual, static_cast<const float*>(delta), scale, weight,
                       bias, alpha, static_cast<float*>(out), rows, hidden);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(add_dyt_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, residual,
                       static_cast<const __nv_bfloat16*>(delta), scale, weight, bias, alpha, static_cast<__nv_bfloat16*>(out), rows, hidden);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

int stride_add_scaled(float* residual, const void* delta, float scale, long long n, int dtype, cudaStream_t stream) {
    if (n < 0) return STRIDE_BAD_ARGUMENT;
    if (n == 0) return 0;
    const unsigned blocks = static_cast<unsigned>(n / 256 >= 4096 ? 4096 : (n + 255) / 256);
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(add_scaled_kernel<float>, dim3(blocks), dim3(256), 0, stream, residual, static_cast<const float*>(delta), scale,
                       static_cast<size_t>(n));
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(add_scaled_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, residual,
                       static_cast<const __nv_bfloat16*>(delta), scale, static_cast<size_t>(n));
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

}  // extern "C"
