// Recurrent block with a real-gated linear recurrent unit (the recurrent layer of Griffin: De et al., "Griffin:
// Mixing Gated Linear Recurrences with Local Attention for Efficient Language Models").
//
// Per token, from the two projections of the layer's input (y~ and x~, both [width], in one matrix `xy`):
//   x  = x~ + bias_x ;  u = conv_b + sum_j conv[c, j] * x(t - (taps - 1) + j)         causal, per channel
//   r  = sigmoid(Wa[b] u_b + ba) ; i = sigmoid(Wi[b] u_b + bi)                        per block b of width / blocks channels
//   a  = exp(-decay * r * softplus(lam)) ;  S_t = a S_(t-1) + sqrt(1 - a^2) * i * u   S in float32, zero at the start
//   out = S_t * gelu_tanh(y~ + bias_y)
// Everything after the projections is float32. Per request the state slot holds taps rows of [width] float32: rows
// 0 .. taps-2 are the last taps-1 inputs x (oldest first; zero before the sequence starts, which is what a fresh slot
// holds), row taps-1 is S. Three kernels, run in this order on any mix of portions and single tokens:
//   rglru_conv    u for every token (reads the tail of the state, writes nothing to it)
//   rglru_gates   the block-diagonal products, with a - 1 and the gated input in the epilogue. a - 1 = expm1(log a) is
//                 what is handed on: for a channel that forgets slowly a is 1 - 1e-4 or closer, where float32 has
//                 steps of 6e-8, and the error of a rounded (and, with a biased exponential, shifted) a grows with
//                 every token of a long sequence
//   rglru_scan    the recurrence over each request's tokens, the output, and the new state (S and the tail)
#include "common.cuh"

namespace stride {

constexpr int kMaxTaps = 16;

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

template <typename T>
__global__ void __launch_bounds__(256)
rglru_conv_kernel(const T* __restrict__ xy, int ld, int x_off, const float* __restrict__ bias_x, const T* __restrict__ conv_w,
                  const float* __restrict__ conv_b, const float* __restrict__ state, const int32_t* __restrict__ seq_of_token,
                  const int32_t* __restrict__ q_start, const int32_t* __restrict__ state_slot, float* __restrict__ u, int width,
                  int taps) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int seq = seq_of_token[t];
    if (seq < 0) {
        u[static_cast<size_t>(t) * width + c] = 0.f;
        return;
    }
    const int start = q_start[seq];
    const int local = t - start;
    const float* tail = state + static_cast<size_t>(state_slot[seq]) * taps * width;
    float acc = conv_b[c];
    for (int j = 0; j < taps; ++j) {
        const int src = local - (taps - 1) + j;
        const float v = src >= 0 ? to_f32(xy[static_cast<size_t>(start + src) * ld + x_off + c]) + bias_x[c]
                                 : tail[static_cast<size_t>(taps - 1 + src) * width + c];
        acc = fmaf(to_f32(conv_w[static_cast<size_t>(c) * taps + j]), v, acc);
    }
    u[static_cast<size_t>(t) * width + c] = acc;
}

// wa_t / wi_t: the gate matrices transposed per block, [blocks, in, out], so that threads of neighbouring output
// channels read neighbouring addresses. One CTA: GT tokens x 32 output channels of one block, the sum over the block's
// inputs cut into four slices (one a warp) that are added in the order of the slices: many small CTAs, so that a step of
// a few tokens still spreads the weights' read over the device.
constexpr int GT = 8, GC = 32, GS = 4;

template <typename T>
__global__ void __launch_bounds__(GC * GS)
rglru_gates_kernel(const float* __restrict__ u, const T* __restrict__ wa_t, const T* __restrict__ wi_t, const float* __restrict__ ba,
                   const float* __restrict__ bi, const float* __restrict__ lam, float decay, float* __restrict__ a_out,
                   float* __restrict__ gx_out, int tokens, int width, int bw) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float us[];                   // [GT][bw], then the slices' sums [GS][2][GT][GC]
    float* part = us + GT * bw;
    const int b = blockIdx.y;
    const int t0 = blockIdx.z * GT;
    const int lane = threadIdx.x & (GC - 1), slice = threadIdx.x / GC;
    const int oc = blockIdx.x * GC + lane;          // output channel inside the block
    for (int i = threadIdx.x; i < GT * bw; i += GC * GS) {
        const int tt = i / bw, k = i % bw;
        us[i] = t0 + tt < tokens ? u[static_cast<size_t>(t0 + tt) * width + b * bw + k] : 0.f;
    }
    __syncthreads();
    float accr[GT], acci[GT];
#pragma unroll
    for (int tt = 0; tt < GT; ++tt) accr[tt] = acci[tt] = 0.f;
    const int per = (bw + GS - 1) / GS;
    const int k_lo = slice * per, k_hi = min(bw, k_lo + per);
    if (oc < bw) {
        const T* wa = wa_t + static_cast<size_t>(b) * bw * bw + oc;
        const T* wi = wi_t + static_cast<size_t>(b) * bw * bw + oc;
#pragma unroll 4
        for (int k = k_lo; k < k_hi; ++k) {
            const float wr = to_f32(wa[static_cast<size_t>(k) * bw]), wg = to_f32(wi[static_cast<size_t>(k) * bw]);
#pragma unroll
            for (int tt = 0; tt < GT; ++tt) {
                const float x = us[tt * bw + k];
                accr[tt] = fmaf(wr, x, accr[tt]);
                acci[tt] = fmaf(wg, x, acci[tt]);
            }
        }
    }
#pragma unroll
    for (int tt = 0; tt < GT; ++tt) {
        part[((slice * 2 + 0) * GT + tt) * GC + lane] = accr[tt];
        part[((slice * 2 + 1) * GT + tt) * GC + lane] = acci[tt];
    }
    __syncthreads();
    if (oc >= bw) return;
    const int c = b * bw + oc;
    const float rate = decay * softplus_f(lam[c]);
    const float br = ba[c], bg = bi[c];
    // warp `slice` finishes the tokens slice, slice + GS, ...
    for (int tt = slice; tt < GT; tt += GS) {
        if (t0 + tt >= tokens) break;
        float sr = 0.f, sg = 0.f;
#pragma unroll
        for (int s2 = 0; s2 < GS; ++s2) {
            sr += part[((s2 * 2 + 0) * GT + tt) * GC + lane];
            sg += part[((s2 * 2 + 1) * GT + tt) * GC + lane];
        }
        const float r = sigmoid_f(sr + br), g = sigmoid_f(sg + bg);
        const float log_a = -rate * r;
        const size_t at = static_cast<size_t>(t0 + tt) * width + c;
        a_out[at] = expm1f(log_a);      // a - 1: a itself, rounded to float32, would lose the rate of a slowly decaying channel
        gx_out[at] = sqrtf(-expm1f(2.f * log_a)) * g * us[tt * bw + oc];
    }
}

// The same products for a long step: GT tokens x 128 output channels of one block a CTA, each thread one channel and
// the whole sum over the block's inputs; the tokens' inputs lie [input][token] in shared memory, so that a thread takes
// the eight tokens of an input with two 16-byte loads for sixteen multiply-adds.
template <typename T>
__global__ void __launch_bounds__(128)
rglru_gates_wide_kernel(const float* __restrict__ u, const T* __restrict__ wa_t, const T* __restrict__ wi_t, const float* __restrict__ ba,
                        const float* __restrict__ bi, const float* __restrict__ lam, float decay, float* __restrict__ a_out,
                        float* __restrict__ gx_out, int tokens, int width, int bw) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float us[];         // [bw][GT]
    const int b = blockIdx.y;
    const int t0 = blockIdx.z * GT;
    const int oc = blockIdx.x * 128 + threadIdx.x;
    for (int i = threadIdx.x; i < GT * bw; i += 128) {
        const int tt = i / bw, k = i % bw;
        us[k * GT + tt] = t0 + tt < tokens ? u[static_cast<size_t>(t0 + tt) * width + b * bw + k] : 0.f;
    }
    __syncthreads();
    if (oc >= bw) return;
    float accr[GT], acci[GT];
#pragma unroll
    for (int tt = 0; tt < GT; ++tt) accr[tt] = acci[tt] = 0.f;
    const T* wa = wa_t + static_cast<size_t>(b) * bw * bw + oc;
    const T* wi = wi_t + static_cast<size_t>(b) * bw * bw + oc;
#pragma unroll 4
    for (int k = 0; k < bw; ++k) {
        const float wr = to_f32(wa[static_cast<size_t>(k) * bw]), wg = to_f32(wi[static_cast<size_t>(k) * bw]);
        const float4 x0 = *reinterpret_cast<const float4*>(us + k * GT), x1 = *reinterpret_cast<const float4*>(us + k * GT + 4);
        const float x[GT] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
        for (int tt = 0; tt < GT; ++tt) {
            accr[tt] = fmaf(wr, x[tt], accr[tt]);
            acci[tt] = fmaf(wg, x[tt], acci[tt]);
        }
    }
    const int c = b * bw + oc;
    const float rate = decay * softplus_f(lam[c]);
    const float br = ba[c], bg = bi[c];
#pragma unroll
    for (int tt = 0; tt < GT; ++tt) {
        if (t0 + tt >= tokens) break;
        const float r = sigmoid_f(accr[tt] + br), g = sigmoid_f(acci[tt] + bg);
        const float log_a = -rate * r;
        const size_t at = static_cast<size_t>(t0 + tt) * width + c;
        a_out[at] = expm1f(log_a);
        gx_out[at] = sqrtf(-expm1f(2.f * log_a)) * g * us[oc * GT + tt];
    }
}

template <typename T>
__global__ void __launch_bounds__(64)
rglru_scan_kernel(const float* __restrict__ a /* a - 1 */, const float* __restrict__ gx, const T* __restrict__ xy, int ld, int x_off, int y_off,
                  const float* __restrict__ bias_x, const float* __restrict__ bias_y, float* __restrict__ state,
                  const int32_t* __restrict__ q_start, const int32_t* __restrict__ q_len, const int32_t* __restrict__ state_slot,
                  T* __restrict__ out, int width, int taps) {
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.y;
    const int n = q_len[seq];
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (n <= 0 || c >= width) return;
    const int start = q_start[seq];
    float* rows = state + static_cast<size_t>(state_slot[seq]) * taps * width;
    float s = rows[static_cast<size_t>(taps - 1) * width + c];
    const float by = bias_y[c];
    // Nothing the loop loads depends on s: eight tokens' values are fetched into registers before the chain of s runs
    // over them, so their latencies overlap. The order of the arithmetic is the token order either way.
    constexpr int AHEAD = 8;
    int i = 0;
    for (; i + AHEAD <= n; i += AHEAD) {
        float am1[AHEAD], g[AHEAD], yp[AHEAD];
#pragma unroll
        for (int j = 0; j < AHEAD; ++j) {
            const size_t at = static_cast<size_t>(start + i + j) * width + c;
            am1[j] = a[at];
            g[j] = gx[at];
            yp[j] = to_f32(xy[static_cast<size_t>(start + i + j) * ld + y_off + c]);
        }
#pragma unroll
        for (int j = 0; j < AHEAD; ++j) {
            s = fmaf(am1[j], s, s) + g[j];      // a S + gx with a - 1 stored
            out[static_cast<size_t>(start + i + j) * width + c] = from_f32<T>(s * gelu_tanh_f(yp[j] + by));
        }
    }
    for (; i < n; ++i) {
        const size_t at = static_cast<size_t>(start + i) * width + c;
        s = fmaf(a[at], s, s) + gx[at];
        const float y = gelu_tanh_f(to_f32(xy[static_cast<size_t>(start + i) * ld + y_off + c]) + by);
        out[at] = from_f32<T>(s * y);
    }
    rows[static_cast<size_t>(taps - 1) * width + c] = s;
    // the last taps-1 inputs, oldest first: from this step's tokens where it has them, else from the old tail
    float tail[kMaxTaps];
    const float bx = bias_x[c];
    for (int r = 0; r < taps - 1; ++r) {
        const int src = n - (taps - 1) + r;
        tail[r] = src >= 0 ? to_f32(xy[static_cast<size_t>(start + src) * ld + x_off + c]) + bx
                           : rows[static_cast<size_t>(taps - 1 + src) * width + c];
    }
    for (int r = 0; r < taps - 1; ++r) rows[static_cast<size_t>(r) * width + c] = tail[r];
}

// ---- the recurrence of a long portion in three passes, parallel over pieces of SEG tokens (bfloat16 mode; the 32-bit
// path keeps the one chain in token order above). With S_t = a_t S_(t-1) + g_t a piece maps the state at its start to
// the state at its end as S -> P S + B, P the product of its a and B its own scan from zero:
//   rglru_piece_kernel   P and B of every piece                      (parallel over pieces and channels)
//   rglru_carry_kernel   the state at the start of every piece        (per request and channel, one step a piece),
//                        the request's new state and convolution tail
//   rglru_apply_kernel   the scan of every piece from its start state, times the gelu branch
constexpr int SEG = 64;

__global__ void __launch_bounds__(64)
rglru_piece_kernel(const float* __restrict__ a, const float* __restrict__ gx, const int32_t* __restrict__ q_start,
                   const int32_t* __restrict__ q_len, float* __restrict__ piece /* [tokens / SEG + seqs][2][width] by first row */,
                   int width) {
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.y, j = blockIdx.z;
    const int n = q_len[seq];
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (j * SEG >= n || c >= width) return;
    const int first = q_start[seq] + j * SEG, count = min(SEG, n - j * SEG);
    float p = 1.f, b = 0.f;
#pragma unroll 8
    for (int i = 0; i < count; ++i) {
        const size_t at = static_cast<size_t>(first + i) * width + c;
        const float am1 = a[at];
        b = fmaf(am1, b, b) + gx[at];
        p = fmaf(am1, p, p);
    }
    // a piece is named by the row of its first token: pieces of different requests never share one
    float* dst = piece + static_cast<size_t>(first / SEG + seq) * 2 * width;
    dst[c] = p;
    dst[width + c] = b;
}

template <typename T>
__global__ void __launch_bounds__(64)
rglru_carry_kernel(float* __restrict__ piece, const T* __restrict__ xy, int ld, int x_off, const float* __restrict__ bias_x,
                   float* __restrict__ state, const int32_t* __restrict__ q_start, const int32_t* __restrict__ q_len,
                   const int32_t* __restrict__ state_slot, int width, int taps) {
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.y;
    const int n = q_len[seq];
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (n <= 0 || c >= width) return;
    const int start = q_start[seq];
    float* rows = state + static_cast<size_t>(state_slot[seq]) * taps * width;
    float s = rows[static_cast<size_t>(taps - 1) * width + c];
    for (int j = 0; j * SEG < n; ++j) {
        float* pb = piece + static_cast<size_t>((start + j * SEG) / SEG + seq) * 2 * width;
        const float p = pb[c], b = pb[width + c];
        pb[c] = s;                          // the piece's start state takes the place of its P
        s = fmaf(p, s, b);
    }
    rows[static_cast<size_t>(taps - 1) * width + c] = s;
    float tail[kMaxTaps];
    const float bx = bias_x[c];
    for (int r = 0; r < taps - 1; ++r) {
        const int src = n - (taps - 1) + r;
        tail[r] = src >= 0 ? to_f32(xy[static_cast<size_t>(start + src) * ld + x_off + c]) + bx
                           : rows[static_cast<size_t>(taps - 1 + src) * width + c];
    }
    for (int r = 0; r < taps - 1; ++r) rows[static_cast<size_t>(r) * width + c] = tail[r];
}

template <typename T>
__global__ void __launch_bounds__(64)
rglru_apply_kernel(const float* __restrict__ a, const float* __restrict__ gx, const float* __restrict__ piece, const T* __restrict__ xy,
                   int ld, int y_off, const float* __restrict__ bias_y, const int32_t* __restrict__ q_start,
                   const int32_t* __restrict__ q_len, T* __restrict__ out, int width) {
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.y, j = blockIdx.z;
    const int n = q_len[seq];
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (j * SEG >= n || c >= width) return;
    const int first = q_start[seq] + j * SEG, count = min(SEG, n - j * SEG);
    float s = piece[static_cast<size_t>(first / SEG + seq) * 2 * width + c];
    const float by = bias_y[c];
#pragma unroll 8
    for (int i = 0; i < count; ++i) {
        const size_t at = static_cast<size_t>(first + i) * width + c;
        s = fmaf(a[at], s, s) + gx[at];
        out[at] = from_f32<T>(s * gelu_tanh_f(to_f32(xy[static_cast<size_t>(first + i) * ld + y_off + c]) + by));
    }
}

}  // namespace stride

using namespace stride;

extern "C" {

int stride_rglru_conv(const void* xy, int ld, int x_off, const float* bias_x, const void* conv_w, const float* conv_b, const float* state,
                      const int32_t* seq_of_token, const int32_t* q_start, const int32_t* state_slot, float* u, int tokens, int width,
                      int taps, int dtype, cudaStream_t stream) {
    if (tokens < 0 || width <= 0 || taps <= 0 || ld <= 0 || x_off < 0) return STRIDE_BAD_ARGUMENT;
    if (taps > kMaxTaps) return STRIDE_UNSUPPORTED;
    if (tokens == 0) return 0;
    const dim3 grid(tokens, (width + 255) / 256);
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(rglru_conv_kernel<float>, grid, dim3(256), 0, stream, static_cast<const float*>(xy), ld, x_off, bias_x,
                       static_cast<const float*>(conv_w), conv_b, state, seq_of_token, q_start, state_slot, u, width, taps);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(rglru_conv_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(xy), ld, x_off,
                       bias_x, static_cast<const __nv_bfloat16*>(conv_w), conv_b, state, seq_of_token, q_start, state_slot, u, width, taps);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

int stride_rglru_gates(const float* u, const void* wa_t, const void* wi_t, const float* ba, const float* bi, const float* lam, float decay,
                       float* a_out, float* gx_out, int tokens, int width, int blocks, int dtype, cudaStream_t stream) {
    if (tokens < 0 || width <= 0 || blocks <= 0 || width % blocks) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    const int bw = width / blocks;
    const size_t smem = (static_cast<size_t>(GT) * bw + GS * 2 * GT * GC) * sizeof(float);
    if (smem > 200 * 1024) return STRIDE_UNSUPPORTED;
    if (smem > 48 * 1024) {     // blocks of more than 1,280 channels: ask for the shared memory beyond the default limit
        const int want = static_cast<int>(smem);
        if (cudaFuncSetAttribute(rglru_gates_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, want) != cudaSuccess ||
            cudaFuncSetAttribute(rglru_gates_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, want) != cudaSuccess ||
            cudaFuncSetAttribute(rglru_gates_wide_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, want) != cudaSuccess)
            return STRIDE_UNSUPPORTED;
    }
    const dim3 grid((bw + GC - 1) / GC, blocks, (tokens + GT - 1) / GT);
    if (grid.z > 65535 || grid.y > 65535) return STRIDE_UNSUPPORTED;
    if (tokens > 64 && dtype == STRIDE_DTYPE_BF16) {
        // Long steps in bfloat16 mode: one thread sums all of a block's inputs. (The 32-bit path keeps one form for
        // every step, so that a token's sums have the same order however the step was cut.)
        const dim3 wide((bw + 127) / 128, blocks, (tokens + GT - 1) / GT);
        stride::launch(rglru_gates_wide_kernel<__nv_bfloat16>, wide, dim3(128), static_cast<size_t>(GT) * bw * sizeof(float), stream, u,
                       static_cast<const __nv_bfloat16*>(wa_t), static_cast<const __nv_bfloat16*>(wi_t), ba, bi, lam, decay, a_out, gx_out,
                       tokens, width, bw);
        return STRIDE_LAUNCH_STATUS();
    }
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(rglru_gates_kernel<float>, grid, dim3(GC * GS), smem, stream, u, static_cast<const float*>(wa_t),
                       static_cast<const float*>(wi_t), ba, bi, lam, decay, a_out, gx_out, tokens, width, bw);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(rglru_gates_kernel<__nv_bfloat16>, grid, dim3(GC * GS), smem, stream, u, static_cast<const __nv_bfloat16*>(wa_t),
                       static_cast<const __nv_bfloat16*>(wi_t), ba, bi, lam, decay, a_out, gx_out, tokens, width, bw);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

int stride_rglru_scan(const float* a, const float* gx, const void* xy, int ld, int x_off, int y_off, const float* bias_x,
                      const float* bias_y, float* state, const int32_t* q_start, const int32_t* q_len, const int32_t* state_slot, void* out,
                      int num_seqs, int width, int taps, int dtype, cudaStream_t stream) {
    if (num_seqs < 0 || width <= 0 || taps <= 0 || num_seqs > 65535) return STRIDE_BAD_ARGUMENT;
    if (taps > kMaxTaps) return STRIDE_UNSUPPORTED;
    if (num_seqs == 0) return 0;
    const dim3 grid((width + 63) / 64, num_seqs);
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(rglru_scan_kernel<float>, grid, dim3(64), 0, stream, a, gx, static_cast<const float*>(xy), ld, x_off, y_off, bias_x,
                       bias_y, state, q_start, q_len, state_slot, static_cast<float*>(out), width, taps);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(rglru_scan_kernel<__nv_bfloat16>, grid, dim3(64), 0, stream, a, gx, static_cast<const __nv_bfloat16*>(xy), ld, x_off,
                       y_off, bias_x, bias_y, state, q_start, q_len, state_slot, static_cast<__nv_bfloat16*>(out), width, taps);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

// The same as stride_rglru_scan in three passes over pieces of 64 tokens (bfloat16 activations). `piece`: float32 scratch of
// (tokens / 64 + num_seqs + 1) * 2 * width. max_q_len: the most tokens a request brings (sizes the grid).
int stride_rglru_scan_pieces(const float* a, const float* gx, const void* xy, int ld, int x_off, int y_off, const float* bias_x,
                             const float* bias_y, float* state, const int32_t* q_start, const int32_t* q_len, const int32_t* state_slot,
                             void* out, float* piece, int num_seqs, int max_q_len, int width, int taps, int dtype, cudaStream_t stream) {
    if (num_seqs < 0 || width <= 0 || taps <= 0 || num_seqs > 65535 || max_q_len <= 0 || !piece) return STRIDE_BAD_ARGUMENT;
    if (taps > kMaxTaps || dtype != STRIDE_DTYPE_BF16) return STRIDE_UNSUPPORTED;
    if (num_seqs == 0) return 0;
    const int pieces = (max_q_len + SEG - 1) / SEG;
    if (pieces > 65535) return STRIDE_UNSUPPORTED;
    const dim3 wide((width + 63) / 64, num_seqs, pieces), narrow((width + 63) / 64, num_seqs);
    const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(xy);
    stride::launch(rglru_piece_kernel, wide, dim3(64), 0, stream, a, gx, q_start, q_len, piece, width);
    stride::launch(rglru_carry_kernel<__nv_bfloat16>, narrow, dim3(64), 0, stream, piece, x, ld, x_off, bias_x, state, q_start, q_len,
                   state_slot, width, taps);
    stride::launch(rglru_apply_kernel<__nv_bfloat16>, wide, dim3(64), 0, stream, a, gx, static_cast<const float*>(piece), x, ld, y_off,
                   bias_y, q_start, q_len, static_cast<__nv_bfloat16*>(out), width);
    return STRIDE_LAUNCH_STATUS();
}

}  // extern "C"
