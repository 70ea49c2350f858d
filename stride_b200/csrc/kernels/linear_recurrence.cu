// Mixers that keep a matrix per head as their memory: S [D, DV] in float32, updated once a token by a rank-one term and
// read with a query. Two rules:
//
//   gated delta rule     S <- diag(g_t) S ;  u = beta_t (v_t - S^T k_t) ;  S <- S + k_t u^T ;  o_t = S^T q_t
//                        (Yang, Kautz, Hatamizadeh, "Gated Delta Networks: Improving Mamba2 with Delta Rule"; here the
//                        decay g_t is a vector over the D key channels)
//   decayed memory with a bonus (the time mixing of RWKV-6: Peng et al., "Eagle and Finch: RWKV with Matrix-Valued
//                        States and Dynamic Recurrence")
//                        o_t = (S + diag(b) k_t v_t^T)^T r_t ;  S <- diag(w_t) S + k_t v_t^T
//
// Both are independent over the DV columns of S, and along a column the only coupling is one sum over D per read. The
// scan kernel gives a column to four neighbouring lanes: lane l of the four holds rows l, l + 4, l + 8, ... in
// registers (R rows, so D <= 4 R; rows beyond D carry zeros), sums its part and the four add up by two shuffles, always
// in the same order. A CTA of 128 threads owns 32 columns of one head of one request and walks the request's tokens of
// the step in order, 16 tokens' inputs staged in shared memory at a time. The order of every sum depends on the token
// only, so a token's output is bitwise the same in a whole prompt, in portions or decoded alone. State per request lives
// in one float32 row of the mixer's state tensor: S [heads, D, DV], then whatever the mixer needs of the past inputs.
//
// Kernels around the scans:
//   delta_prepare   per token: causal convolution (taps from the state's tail at a portion's start) and SiLU of the q, k
//                   and v projections, unit length for q and k per head (q also times D^-1/2), beta = sigmoid, and the
//                   decay exp(-exp(A_log) softplus(a + dt_bias)); everything float32
//   shift_mix       per token: the lerps between a token's input and the previous token's (the state's at a portion's
//                   start), one per consumer; the portion's last input goes into the state
//   head_norm_gate  o / rms(o) * weight * gate per head, into the compute type for the output projection
// The scans end by writing S back and, for the delta rule, by moving the convolution's tail in the state forward.
#include "common.cuh"

namespace stride {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

__device__ __forceinline__ float load_any(const void* p, size_t i, int is_bf16) {
    return is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]) : static_cast<const float*>(p)[i];
}

// ------------------------------------------------------------------------------------------------ delta_prepare
// proj [tokens, ld] (compute type): columns [0, GD) q, [GD, 2GD) k, [2GD, 2GD + HV) v, then H columns of beta's
// projection. conv_w [C, taps] float32 for the C = 2GD + HV channels in the same order. low [tokens, ld_low] float32:
// columns [0, HD) the decay's projection. tail: the state's rows [taps - 1, C] at `tail_off` floats into a slot's row.
// Outputs float32: qk [tokens, 2GD] (q then k, unit length), v [tokens, HV], beta [tokens, H], decay [tokens, HD].
// What is handed on of a decay g is g - 1 = expm1(log g), and the scans compute S + (g - 1) S: for a channel that forgets
// slowly g is within 1e-4 of 1, where float32 has steps of 6e-8 and a rounded g costs a little with every token.
// One warp a head: warps 0..2G-1 the q and k heads, then H warps for the v heads, which also do beta and the decay.
constexpr int kPrepWarps = 8;
constexpr int kMaxPerLane = 8;      // head sizes up to 256

template <typename T>
__global__ void __launch_bounds__(kPrepWarps * 32)
delta_prepare_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ conv_w, const float* __restrict__ low, int ld_low,
                     const float* __restrict__ a_log, const float* __restrict__ dt_bias, const float* __restrict__ state,
                     long long state_stride, long long tail_off, const int32_t* __restrict__ seq_of_token,
                     const int32_t* __restrict__ q_start, const int32_t* __restrict__ state_slot, float* __restrict__ qk,
                     float* __restrict__ v_out, float* __restrict__ beta, float* __restrict__ decay, int G, int H, int D, int DV,
                     int taps, float unit_eps) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * kPrepWarps + warp;
    if (head >= 2 * G + H) return;
    const int GD = G * D, HV = H * DV, C = 2 * GD + HV;
    const bool is_v = head >= 2 * G;
    const int n = is_v ? DV : D;
    const int c0 = is_v ? 2 * GD + (head - 2 * G) * DV : head * D;       // first channel of this head
    const int seq = seq_of_token[t];
    float* dst = is_v ? v_out + static_cast<size_t>(t) * HV + (head - 2 * G) * DV : qk + static_cast<size_t>(t) * 2 * GD + head * D;
    if (seq < 0) {          // a padded row of a fixed-size batch
        for (int e = lane; e < n; e += 32) dst[e] = 0.f;
        if (is_v) {
            const int h = head - 2 * G;
            for (int e = lane; e < D; e += 32) decay[static_cast<size_t>(t) * H * D + h * D + e] = 0.f;
            if (lane == 0) beta[static_cast<size_t>(t) * H + h] = 0.f;
        }
        return;
    }
    const int start = q_start[seq];
    const int local = t - start;
    const float* tail = state + static_cast<size_t>(state_slot[seq]) * state_stride + tail_off;
    float y[kMaxPerLane];
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < kMaxPerLane; ++r) {
        const int e = lane + 32 * r;
        y[r] = 0.f;
        if (e < n) {
            const int c = c0 + e;
            float acc = 0.f;
            for (int j = 0; j < taps; ++j) {
                const int src = local - (taps - 1) + j;
                const float x = src >= 0 ? to_f32(proj[static_cast<size_t>(start + src) * ld + c])
                                         : tail[static_cast<size_t>(taps - 1 + src) * C + c];
                acc = fmaf(conv_w[static_cast<size_t>(c) * taps + j], x, acc);
            }
            y[r] = silu_f(acc);
            ss = fmaf(y[r], y[r], ss);
        }
    }
    float mult = 1.f;
    if (!is_v) {
        ss = warp_sum(ss);
        mult = 1.f / sqrtf(ss + unit_eps);
        if (head < G) mult *= 1.f / sqrtf(static_cast<float>(D));
    }
#pragma unroll
    for (int r = 0; r < kMaxPerLane; ++r) {
        const int e = lane + 32 * r;
        if (e < n) dst[e] = y[r] * mult;
    }
    if (is_v) {
        const int h = head - 2 * G;
        const float rate = expf(a_log[h]);
        for (int e = lane; e < D; e += 32) {
            const float a = low[static_cast<size_t>(t) * ld_low + h * D + e] + dt_bias[h * D + e];
            decay[static_cast<size_t>(t) * H * D + h * D + e] = expm1f(-rate * softplus_f(a));
        }
        if (lane == 0) beta[static_cast<size_t>(t) * H + h] = sigmoid_f(to_f32(proj[static_cast<size_t>(t) * ld + C + h]));
    }
}

// ---------------------------------------------------------------------------------------------------- shift_mix
// x [tokens, width] (compute type); mu [mixes, width] float32; out [mixes, tokens, width] (compute type):
// out[s, t] = x[t] + (prev - x[t]) * mu[s], prev = x[t - 1] inside a portion and the state's vector at its start. The CTA
// of a portion's first token then stores the portion's last input as the new state (it alone touches the state).
template <typename T>
__global__ void __launch_bounds__(256)
shift_mix_kernel(const T* __restrict__ x, const float* __restrict__ mu, float* __restrict__ state, long long state_stride,
                 long long prev_off, const int32_t* __restrict__ seq_of_token, const int32_t* __restrict__ q_start,
                 const int32_t* __restrict__ q_len, const int32_t* __restrict__ state_slot, T* __restrict__ out, int tokens, int width,
                 int mixes) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int seq = seq_of_token[t];
    if (seq < 0) {
        for (int c = threadIdx.x; c < width; c += blockDim.x)
            for (int s = 0; s < mixes; ++s) out[(static_cast<size_t>(s) * tokens + t) * width + c] = from_f32<T>(0.f);
        return;
    }
    const int start = q_start[seq];
    const bool first = t == start;
    float* prev_state = state + static_cast<size_t>(state_slot[seq]) * state_stride + prev_off;
    const T* last = x + static_cast<size_t>(start + q_len[seq] - 1) * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float cur = to_f32(x[static_cast<size_t>(t) * width + c]);
        const float prev = first ? prev_state[c] : to_f32(x[static_cast<size_t>(t - 1) * width + c]);
        const float d = prev - cur;
        for (int s = 0; s < mixes; ++s)
            out[(static_cast<size_t>(s) * tokens + t) * width + c] = from_f32<T>(fmaf(d, mu[static_cast<size_t>(s) * width + c], cur));
        if (first) prev_state[c] = to_f32(last[c]);
    }
}

// ------------------------------------------------------------------------------------------------ head_norm_gate
// o [tokens, H, DV] float32 -> out [tokens, H * DV] (compute type): o / sqrt(mean(o^2) + eps) * weight * gate.
// weight [.. ] float32 read at h * w_head_stride + j (0: one weight for all heads). gate_kind 0: sigmoid of float32
// gate[t * ld_gate + h * DV + j]; 1: silu of a compute-type gate at the same place. One warp a (token, head).
template <typename T>
__global__ void __launch_bounds__(256)
head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ weight, int w_head_stride, const void* __restrict__ gate,
                      int ld_gate, int gate_kind, T* __restrict__ out, int tokens, int H, int DV, float eps) {
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long pair = static_cast<long long>(blockIdx.x) * 8 + warp;
    if (pair >= static_cast<long long>(tokens) * H) return;
    const int t = static_cast<int>(pair / H), h = static_cast<int>(pair % H);
    const float* row = o + (static_cast<size_t>(t) * H + h) * DV;
    float ss = 0.f;
    for (int j = lane; j < DV; j += 32) ss = fmaf(row[j], row[j], ss);
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / static_cast<float>(DV) + eps);
    for (int j = lane; j < DV; j += 32) {
        const size_t at = static_cast<size_t>(t) * ld_gate + h * DV + j;
        const float g = gate_kind == 0 ? sigmoid_f(static_cast<const float*>(gate)[at]) : silu_f(to_f32(static_cast<const T*>(gate)[at]));
        out[(static_cast<size_t>(t) * H + h) * DV + j] = from_f32<T>(row[j] * inv * weight[h * w_head_stride + j] * g);
    }
}

// --------------------------------------------------------------------------------------------------------- scans
constexpr int kLanes = 4;           // lanes that share a column's rows
constexpr int kCols = 32;           // columns a CTA
constexpr int kChunk = 16;          // tokens staged at a time

__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    return v;
}

struct ScanArgs {
    const void* a;          // queries (delta) / receptance (memory with bonus): [tokens, lda], head h at column (h / group) * D
    const void* k;          // keys, the same layout
    const float* w;         // [tokens, H * D]: the decay minus one (delta), or its double logarithm before w0 (bonus rule)
    const void* v;          // values [tokens, ldv], head h at column h * DV
    const float* beta;      // [tokens, H] (delta) or null
    const float* w0;        // [H * D] added to w before exp(-exp(.)) (bonus rule) or null
    const float* bonus;     // [H * D] (bonus rule) or null
    float* o;               // [tokens, H * DV] float32
    float* state;           // [slots, state_stride]; S of head h at h * D * DV
    long long state_stride;
    const int32_t* q_start;
    const int32_t* q_len;
    const int32_t* state_slot;
    int lda, ldv, H, group, D, DV, in_bf16;
    // the convolution's tail (delta rule; taps 0: none): the last taps - 1 rows of proj's first C columns
    const void* proj;
    int ld_proj, C, taps, proj_bf16;
    long long tail_off;
};

template <int R, int RULE>      // RULE 0: gated delta rule, 1: decayed memory with a bonus
__global__ void __launch_bounds__(kCols * kLanes)
scan_kernel(const ScanArgs p) {
    pdl_trigger();
    pdl_wait();
    constexpr int DP = R * kLanes;
    __shared__ float s_a[kChunk][DP], s_k[kChunk][DP], s_w[kChunk][DP], s_v[kChunk][kCols], s_beta[kChunk], s_bonus[DP];
    const int seq = blockIdx.z, h = blockIdx.y;
    const int len = p.q_len[seq];
    if (len <= 0) return;
    const int start = p.q_start[seq];
    const int il = threadIdx.x & (kLanes - 1), jc = threadIdx.x >> 2;
    const int j = blockIdx.x * kCols + jc;
    const int D = p.D, DV = p.DV, H = p.H;
    const int hk = h / p.group;
    float* S_g = p.state + static_cast<size_t>(p.state_slot[seq]) * p.state_stride + static_cast<size_t>(h) * D * DV;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = il + kLanes * r;
        S[r] = (i < D && j < DV) ? S_g[static_cast<size_t>(i) * DV + j] : 0.f;
    }
    if (RULE == 1)
        for (int i = threadIdx.x; i < DP; i += blockDim.x) s_bonus[i] = i < D ? p.bonus[h * D + i] : 0.f;

    for (int c0 = 0; c0 < len; c0 += kChunk) {
        const int nt = min(kChunk, len - c0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * DP; idx += blockDim.x) {
            const int tt = idx / DP, i = idx - tt * DP;
            const size_t row = static_cast<size_t>(start + c0 + tt);
            float a = 0.f, k = 0.f, w = 0.f;
            if (i < D) {
                a = load_any(p.a, row * p.lda + hk * D + i, p.in_bf16);
                k = load_any(p.k, row * p.lda + hk * D + i, p.in_bf16);
                w = p.w[row * H * D + h * D + i];
                if (RULE == 1) w = expm1f(-expf(w + p.w0[h * D + i]));
            }
            s_a[tt][i] = a;
            s_k[tt][i] = k;
            s_w[tt][i] = w;
        }
        for (int idx = threadIdx.x; idx < nt * kCols; idx += blockDim.x) {
            const int tt = idx / kCols, c = idx - tt * kCols;
            const int col = blockIdx.x * kCols + c;
            s_v[tt][c] = col < DV ? load_any(p.v, static_cast<size_t>(start + c0 + tt) * p.ldv + h * DV + col, p.in_bf16) : 0.f;
        }
        if (RULE == 0 && threadIdx.x < nt) s_beta[threadIdx.x] = p.beta[static_cast<size_t>(start + c0 + threadIdx.x) * H + h];
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float vj = s_v[tt][jc];
            float out;
            if (RULE == 0) {
                // four partial sums each (R is a multiple of 4): a single chain of R dependent additions would set the pace
                float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int i = il + kLanes * r;
                    S[r] = fmaf(S[r], s_w[tt][i], S[r]);
                    d[r & 3] = fmaf(S[r], s_k[tt][i], d[r & 3]);
                }
                const float dot = quad_sum((d[0] + d[1]) + (d[2] + d[3]));
                const float u = s_beta[tt] * (vj - dot);
                float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int i = il + kLanes * r;
                    S[r] = fmaf(s_k[tt][i], u, S[r]);
                    a[r & 3] = fmaf(S[r], s_a[tt][i], a[r & 3]);
                }
                out = quad_sum((a[0] + a[1]) + (a[2] + a[3]));
            } else {
                float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int i = il + kLanes * r;
                    const float kv = s_k[tt][i] * vj;
                    a[r & 3] = fmaf(s_a[tt][i], fmaf(s_bonus[i], kv, S[r]), a[r & 3]);
                    S[r] = fmaf(s_w[tt][i], S[r], S[r]) + kv;
                }
                out = quad_sum((a[0] + a[1]) + (a[2] + a[3]));
            }
            if (il == 0 && j < DV) p.o[(static_cast<size_t>(start + c0 + tt) * H + h) * DV + j] = out;
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = il + kLanes * r;
        if (i < D && j < DV) S_g[static_cast<size_t>(i) * DV + j] = S[r];
    }
    // The convolution's tail: row m of the new tail is the input of local token len - (taps - 1) + m, which lies in
    // this step or, for a short step, further up in the old tail. Channels are shared out over the CTAs of the request;
    // a channel's rows move in ascending order, so a row is read before it is overwritten.
    if (p.taps > 1) {
        const int keep = p.taps - 1;
        float* tail = p.state + static_cast<size_t>(p.state_slot[seq]) * p.state_stride + p.tail_off;
        const int cta = blockIdx.y * gridDim.x + blockIdx.x, ctas = gridDim.x * gridDim.y;
        for (int c = cta * blockDim.x + threadIdx.x; c < p.C; c += ctas * blockDim.x)
            for (int m = 0; m < keep; ++m) {
                const int src = len - keep + m;
                tail[static_cast<size_t>(m) * p.C + c] = src >= 0 ? load_any(p.proj, static_cast<size_t>(start + src) * p.ld_proj + c, p.proj_bf16)
                                                                 : tail[static_cast<size_t>(m + len) * p.C + c];
            }
    }
}

template <int RULE>
int launch_scan(const ScanArgs& p, int num_seqs, cudaStream_t stream) {
    const dim3 grid((p.DV + kCols - 1) / kCols, p.H, num_seqs), block(kCols * kLanes);
    const int rows = (p.D + kLanes - 1) / kLanes;
    if (rows <= 4) stride::launch(scan_kernel<4, RULE>, grid, block, 0, stream, p);
    else if (rows <= 8) stride::launch(scan_kernel<8, RULE>, grid, block, 0, stream, p);
    else if (rows <= 12) stride::launch(scan_kernel<12, RULE>, grid, block, 0, stream, p);
    else if (rows <= 16) stride::launch(scan_kernel<16, RULE>, grid, block, 0, stream, p);
    else if (rows <= 24) stride::launch(scan_kernel<24, RULE>, grid, block, 0, stream, p);
    else if (rows <= 32) stride::launch(scan_kernel<32, RULE>, grid, block, 0, stream, p);
    else return STRIDE_UNSUPPORTED;
    return STRIDE_LAUNCH_STATUS();
}

}  // namespace stride

using namespace stride;

extern "C" {

int stride_delta_prepare(const void* proj, int ld, const float* conv_w, const float* low, int ld_low, const float* a_log,
                         const float* dt_bias, const float* state, long long state_stride, long long tail_off,
                         const int32_t* seq_of_token, const int32_t* q_start, const int32_t* state_slot, float* qk, float* v_out,
                         float* beta, float* decay, int tokens, int G, int H, int D, int DV, int taps, float unit_eps, int dtype,
                         cudaStream_t stream) {
    if (tokens < 0 || G <= 0 || H <= 0 || D <= 0 || DV <= 0 || taps <= 0 || H % G) return STRIDE_BAD_ARGUMENT;
    if (D > 32 * kMaxPerLane || DV > 32 * kMaxPerLane) return STRIDE_UNSUPPORTED;
    if (tokens == 0) return 0;
    const dim3 grid(tokens, (2 * G + H + kPrepWarps - 1) / kPrepWarps), block(kPrepWarps * 32);
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(delta_prepare_kernel<float>, grid, block, 0, stream, static_cast<const float*>(proj), ld, conv_w, low, ld_low, a_log,
                       dt_bias, state, state_stride, tail_off, seq_of_token, q_start, state_slot, qk, v_out, beta, decay, G, H, D, DV, taps,
                       unit_eps);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(delta_prepare_kernel<__nv_bfloat16>, grid, block, 0, stream, static_cast<const __nv_bfloat16*>(proj), ld, conv_w, low,
                       ld_low, a_log, dt_bias, state, state_stride, tail_off, seq_of_token, q_start, state_slot, qk, v_out, beta, decay, G, H,
                       D, DV, taps, unit_eps);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

// The gated delta rule over the step's requests. qk, v, beta, decay: what delta_prepare wrote. proj: the projections
// whose last taps - 1 rows become the convolution's new tail.
int stride_delta_scan(const float* qk, const float* v, const float* beta, const float* decay, float* o, float* state,
                      long long state_stride, long long tail_off, const void* proj, int ld_proj, const int32_t* q_start,
                      const int32_t* q_len, const int32_t* state_slot, int num_seqs, int G, int H, int D, int DV, int taps, int dtype,
                      cudaStream_t stream) {
    if (num_seqs < 0 || G <= 0 || H <= 0 || D <= 0 || DV <= 0 || taps <= 0 || H % G) return STRIDE_BAD_ARGUMENT;
    if (dtype != STRIDE_DTYPE_F32 && dtype != STRIDE_DTYPE_BF16) return STRIDE_BAD_ARGUMENT;
    if (num_seqs == 0) return 0;
    ScanArgs p = {};
    p.a = qk;
    p.k = qk + static_cast<size_t>(G) * D;
    p.lda = 2 * G * D;
    p.w = decay;
    p.v = v;
    p.ldv = H * DV;
    p.beta = beta;
    p.o = o;
    p.state = state;
    p.state_stride = state_stride;
    p.q_start = q_start;
    p.q_len = q_len;
    p.state_slot = state_slot;
    p.H = H;
    p.group = H / G;
    p.D = D;
    p.DV = DV;
    p.in_bf16 = 0;
    p.proj = proj;
    p.ld_proj = ld_proj;
    p.C = 2 * G * D + H * DV;
    p.taps = taps;
    p.tail_off = tail_off;
    p.proj_bf16 = dtype == STRIDE_DTYPE_BF16 ? 1 : 0;      // the tail is read in the projections' type, the rest is float32
    return launch_scan<0>(p, num_seqs, stream);
}

// Decayed memory with a bonus. r, k, v [tokens, H * D] in the compute type (one head size for keys and values);
// wlog [tokens, H * D] float32: the decay is exp(-exp(wlog + w0)).
int stride_bonus_scan(const void* r, const void* k, const void* v, const float* wlog, const float* w0, const float* bonus, float* o,
                      float* state, long long state_stride, const int32_t* q_start, const int32_t* q_len, const int32_t* state_slot,
                      int num_seqs, int H, int D, int dtype, cudaStream_t stream) {
    if (num_seqs < 0 || H <= 0 || D <= 0) return STRIDE_BAD_ARGUMENT;
    if (dtype != STRIDE_DTYPE_F32 && dtype != STRIDE_DTYPE_BF16) return STRIDE_BAD_ARGUMENT;
    if (num_seqs == 0) return 0;
    ScanArgs p = {};
    p.a = r;
    p.k = k;
    p.lda = H * D;
    p.w = wlog;
    p.w0 = w0;
    p.bonus = bonus;
    p.v = v;
    p.ldv = H * D;
    p.o = o;
    p.state = state;
    p.state_stride = state_stride;
    p.q_start = q_start;
    p.q_len = q_len;
    p.state_slot = state_slot;
    p.H = H;
    p.group = 1;
    p.D = D;
    p.DV = D;
    p.in_bf16 = dtype == STRIDE_DTYPE_BF16 ? 1 : 0;
    p.taps = 0;
    return launch_scan<1>(p, num_seqs, stream);
}

int stride_shift_mix(const void* x, const float* mu, float* state, long long state_stride, long long prev_off,
                     const int32_t* seq_of_token, const int32_t* q_start, const int32_t* q_len, const int32_t* state_slot, void* out,
                     int tokens, int width, int mixes, int dtype, cudaStream_t stream) {
    if (tokens < 0 || width <= 0 || mixes <= 0) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(shift_mix_kernel<float>, dim3(tokens), dim3(256), 0, stream, static_cast<const float*>(x), mu, state, state_stride,
                       prev_off, seq_of_token, q_start, q_len, state_slot, static_cast<float*>(out), tokens, width, mixes);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(shift_mix_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(x), mu, state,
                       state_stride, prev_off, seq_of_token, q_start, q_len, state_slot, static_cast<__nv_bfloat16*>(out), tokens, width,
                       mixes);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

int stride_head_norm_gate(const float* o, const float* weight, int w_head_stride, const void* gate, int ld_gate, int gate_kind, void* out,
                          int tokens, int H, int DV, float eps, int dtype, cudaStream_t stream) {
    if (tokens < 0 || H <= 0 || DV <= 0 || gate_kind < 0 || gate_kind > 1) return STRIDE_BAD_ARGUMENT;
    if (tokens == 0) return 0;
    const long long pairs = static_cast<long long>(tokens) * H;
    const dim3 grid(static_cast<unsigned>((pairs + 7) / 8)), block(256);
    if (dtype == STRIDE_DTYPE_F32)
        stride::launch(head_norm_gate_kernel<float>, grid, block, 0, stream, o, weight, w_head_stride, gate, ld_gate, gate_kind,
                       static_cast<float*>(out), tokens, H, DV, eps);
    else if (dtype == STRIDE_DTYPE_BF16)
        stride::launch(head_norm_gate_kernel<__nv_bfloat16>, grid, block, 0, stream, o, weight, w_head_stride, gate, ld_gate, gate_kind,
                       static_cast<__nv_bfloat16*>(out), tokens, H, DV, eps);
    else
        return STRIDE_BAD_ARGUMENT;
    return STRIDE_LAUNCH_STATUS();
}

}  // extern "C"
