// Per-layer token input: a slice of a second embedding, gated by the residual stream, added to the stream.
//
// For token t with id v and stream row x (float32 [hidden]):
//   e = table[v, offset : offset + dim]
//   g = gelu_tanh(W_gate x) * e                    W_gate [dim, hidden]
//   y = W_proj g                                   W_proj [hidden, dim]
//   x <- x + scale * y / sqrt(mean(y^2) + eps) * norm_w
// Two forms. As products: the stream rounded to the compute type (cast_rows), W_gate as a matrix product, side_gate
// (gelu * e), W_proj as a matrix product, side_norm_add (unit RMS, weight, scaled sum into the float32 stream); the
// matrices are then read once a step. And token_side, all of it in one kernel in float32 on the stream row itself,
// one CTA per token, which reads the matrices once per token: the statement of the rule that the other form is
// tested against, and the form for sizes where products do not pay. Padded tokens are left alone.
#include "common.cuh"

namespace stride {

__device__ __forceinline__ float gelu_tanh(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void __launch_bounds__(256)
token_side_kernel(float* __restrict__ residual, const int32_t* __restrict__ ids, const int32_t* __restrict__ seq_of_token,
                  const T* __restrict__ table, int table_width, int offset, int vocab, const T* __restrict__ w_gate,
                  const T* __restrict__ w_proj, const float* __restrict__ norm_w, int hidden, int dim, float eps, float scale) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    float* xs = smem;                 // hidden: the row, later y
    float* g = smem + hidden;         // dim
    float* scratch = g + dim;         // 32
    const int t = blockIdx.x;
    if (seq_of_token && seq_of_token[t] < 0) return;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    float* row = residual + static_cast<size_t>(t) * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) xs[i] = row[i];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const T* e = table + static_cast<size_t>(id) * table_width + offset;
    for (int d = warp; d < dim; d += nwarps) {
        const T* w = w_gate + static_cast<size_t>(d) * hidden;
        float acc = 0.f;
        for (int i = lane; i < hidden; i += 32) acc = fmaf(xs[i], to_f32(w[i]), acc);
        acc = warp_sum(acc);
        if (lane == 0) g[d] = gelu_tanh(acc) * to_f32(e[d]);
    }
    __syncthreads();
    float sq = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const T* w = w_proj + static_cast<size_t>(c) * dim;
        float y = 0.f;
        for (int d = 0; d < dim; ++d) y = fmaf(to_f32(w[d]), g[d], y);
        xs[c] = y;                    // each thread rewrites only the columns it reads back below
        sq = fmaf(y, y, sq);
    }
    const float total = block_sum(sq, scratch);
    const float inv = rsqrtf(total / static_cast<float>(hidden) + eps);
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) row[c] = __fmaf_rn(scale, xs[c] * inv * norm_w[c], row[c]);
}

template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ src, T* __restrict__ dst, size_t n) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x)
        dst[i] = from_f32<T>(src[i]);
}

template <typename T>
__global__ void side_gate_kernel(const T* __restrict__ pre, const int32_t* __restrict__ ids, const int32_t* __restrict__ seq_of_token,
                                 const T* __restrict__ table, int table_width, int offset, int vocab, T* __restrict__ out, int dim) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const bool live = !seq_of_token || seq_of_token[t] >= 0;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const T* e = table + static_cast<size_t>(id) * table_width + offset;
    for (int d = threadIdx.x; d < dim; d += blockDim.x)
        out[static_cast<size_t>(t) * dim + d] = from_f32<T>(live ? gelu_tanh(to_f32(pre[static_cast<size_t>(t) * dim + d])) * to_f32(e[d]) : 0.f);
}

template <typename T>
__global__ void __launch_bounds__(256)
side_norm_add_kernel(float* __restrict__ residual, const T* __restrict__ y, const int32_t* __restrict__ seq_of_token,
                     const float* __restrict__ norm_w, int hidden, float eps, float scale) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    if (seq_of_token && seq_of_token[t] < 0) return;
    const T* row = y + static_cast<size_t>(t) * hidden;
    float sq = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = to_f32(row[c]);
        sq = fmaf(v, v, sq);
    }
    const float inv = rsqrtf(block_sum(sq, scratch) / static_cast<float>(hidden) + eps);
    float* res = residual + static_cast<size_t>(t) * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) res[c] = __fmaf_rn(scale, to_f32(row[c]) * inv * norm_w[c], res[c]);
}

}  // namespace stride

using namespace stride;

extern "C" int stride_cast_rows(const float* src, void* dst, long long n, int dtype, cudaStream_t stream) {
    if (n < 0) return STRIDE_BAD_ARGUMENT;
    if (n == 0) return 0;
    const unsigned blocks = static_cast<unsigned>(n / 256 >= 8192 ? 8192 : (n + 255) / 256);
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(cast_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, src, static_cast<float*>(dst), static_cast<size_t>(n));
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(cast_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, src, static_cast<__nv_bfloat16*>(dst), static_cast<size_t>(n));
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

extern "C" int stride_side_gate(const void* pre, const int32_t* ids, const int32_t* seq_of_token, const void* table, int table_width,
                                int offset, int vocab, void* out, int tokens, int dim, int dtype, cudaStream_t stream) {
    if (tokens < 0 || dim <= 0 || offset < 0 || offset + dim > table_width || vocab <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    const int threads = dim >= 256 ? 256 : (dim + 31) / 32 * 32;
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(side_gate_kernel<float>, dim3(tokens), dim3(threads), 0, stream, static_cast<const float*>(pre), ids, seq_of_token,
                       static_cast<const float*>(table), table_width, offset, vocab, static_cast<float*>(out), dim);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(side_gate_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream, static_cast<const __nv_bfloat16*>(pre), ids,
                       seq_of_token, static_cast<const __nv_bfloat16*>(table), table_width, offset, vocab, static_cast<__nv_bfloat16*>(out), dim);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

extern "C" int stride_side_norm_add(float* residual, const void* y, const int32_t* seq_of_token, const float* norm_w, int tokens, int hidden,
                                    float eps, float scale, int dtype, cudaStream_t stream) {
    if (tokens < 0 || hidden <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(side_norm_add_kernel<float>, dim3(tokens), dim3(256), 0, stream, residual, static_cast<const float*>(y), seq_of_token,
                       norm_w, hidden, eps, scale);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(side_norm_add_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, residual, static_cast<const __nv_bfloat16*>(y),
                       seq_of_token, norm_w, hidden, eps, scale);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

extern "C" int stride_token_side(float* residual, const int32_t* ids, const int32_t* seq_of_token, const void* table, int table_width,
                                 int offset, int vocab, const void* w_gate, const void* w_proj, const float* norm_w, int tokens,
                                 int hidden, int dim, float eps, float scale, int dtype, cudaStream_t stream) {
    if (tokens < 0 || hidden <= 0 || dim <= 0 || offset < 0 || offset + dim > table_width || vocab <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    const size_t smem = static_cast<size_t>(hidden + dim + 32) * sizeof(float);
    if (smem > 48 * 1024) return STRIDE_UNSUPPORTED;
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(token_side_kernel<float>, dim3(tokens), dim3(256), smem, stream, residual, ids, seq_of_token,
                       static_cast<const float*>(table), table_width, offset, vocab, static_cast<const float*>(w_gate),
                       static_cast<const float*>(w_proj), norm_w, hidden, dim, eps, scale);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(token_side_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), smem, stream, residual, ids, seq_of_token,
                       static_cast<const __nv_bfloat16*>(table), table_width, offset, vocab, static_cast<const __nv_bfloat16*>(w_gate),
                       static_cast<const __nv_bfloat16*>(w_proj), norm_w, hidden, dim, eps, scale);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}
