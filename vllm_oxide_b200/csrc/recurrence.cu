// Linear recurrences over a matrix state per request and head: the state S [K key channels,
// V value channels] is float32, lives in the request's state slot and is carried from token to
// token, across steps:
//     mode 0 (delta rule with decay):  S_t = diag(w_t) S_(t-1) - b_t (u_t^T S_(t-1)) + k_t v_t^T
//     mode 1 (fixed decay per head):   S_t = d_h S_(t-1) + k_t v_t^T
//     mode 2 (gated delta rule):       S' = diag(w_t) S_(t-1);  S_t = S' + k_t (b_t (v_t - S'^T k_t))^T
//     mode 3 (state space):            S_t = b_t S_(t-1) + k_t (u_t v_t)^T     (b_t a decay, u_t a step size: one number
//                                      per token and head each; heads may share r and k in groups, as in mode 2)
//     o_t = S_t^T r_t
// w_t, b_t, u_t are float32 vectors per token, head and key channel, prepared by vob_delta_prep (or
// by anything else that writes them); d_h is one number per head; in mode 2 b_t is one number per token
// and head (the writing strength) and several heads may share one r and k (`rk_div` heads each).
//
// Every value column of S evolves on its own, so the work is cut by columns: a block owns VT
// columns of one head of one request, KS threads share a column (thread q of them holds key
// channels q * KPT .. q * KPT + KPT - 1 in registers) and the two dot products over key channels are finished
// by shuffles among those KS lanes, in a fixed order. The block walks the request's rows of this
// step in order, a few tokens at a time staged in shared memory. A step of one token is the same
// kernel: read the state, one update, write it back (bound by the state's bytes). The arithmetic
// of a token never depends on how the tokens were cut into steps or what else is in the batch.
//
// Beside the scan: vob_delta_prep (unit key, removal rate, decay from its low-rank projection),
// vob_gated_delta_prep (short causal convolutions with silu, unit q and k, writing strength, decay from
// softplus) with vob_conv_state_update (the convolutions' last inputs, kept per request),
// vob_rotate_scale (rotary positions on the first `rot` features of every head, times a scale,
// to float32) and vob_recurrence_post (per-head RMS norm of o, an optional weight, a gate).
#include "common.cuh"
VOB_PDL_SWITCH(recurrence)

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// An element as its raw bits, and back: a value fetched ahead stays untouched in its register until it is
// used (a conversion right behind the load would make the warp wait for the load there and then).
__device__ __forceinline__ unsigned raw_ld(const float* p) { return __float_as_uint(*p); }
__device__ __forceinline__ unsigned raw_ld(const __nv_bfloat16* p) { return *reinterpret_cast<const unsigned short*>(p); }
template <typename T> __device__ __forceinline__ float raw_to_float(unsigned x);
template <> __device__ __forceinline__ float raw_to_float<float>(unsigned x) { return __uint_as_float(x); }
template <> __device__ __forceinline__ float raw_to_float<__nv_bfloat16>(unsigned x) { return __uint_as_float(x << 16); }

// ---------------------------------------------------------------------------------------------
// Delta-rule preparation, per token t, head h and key channel c (ch = h * K + c):
//   u = k / sqrt(sum_c k^2 + 1e-6)                      (the key at unit length, per head)
//   a = sigmoid(a_in + a_bias)                          (removal rate)       b = a * u
//   w = exp(-exp(-1/2) * sigmoid(w0 + sum_j w2[ch, j] * tanh(low[j])))       (decay, in (0.545, 1))
// k, a_in and low (the rank-R projection) are columns of one projection output `proj` [T, ld].
// Launch: one block of 128 threads per (8 tokens, head). All arithmetic float32.
// ---------------------------------------------------------------------------------------------
#define VOB_PREP_TOKENS 8
template <typename T, typename TW>
__global__ void __launch_bounds__(128)
delta_prep_kernel(const T* __restrict__ proj, long ld, int k_off, int a_off, int low_off, int R, const TW* __restrict__ w2t,
                  const float* __restrict__ w0, const float* __restrict__ a_bias, int T_rows, int H, int K, float* __restrict__ w_out,
                  float* __restrict__ b_out, float* __restrict__ u_out) {
    pdl_launch_dependents();
    pdl_wait(41);
    extern __shared__ float th[];          // tanh of the low-rank projection, [VOB_PREP_TOKENS][R]
    __shared__ float red[VOB_PREP_TOKENS][4];
    const int t0 = blockIdx.x * VOB_PREP_TOKENS, h = blockIdx.y, tid = threadIdx.x;
    const int nt = min(VOB_PREP_TOKENS, T_rows - t0);
    for (int e = tid; e < nt * R; e += blockDim.x) {
        const int tt = e / R, j = e - tt * R;
        th[e] = tanhf(ld_f(proj + (size_t)(t0 + tt) * ld + low_off + j));
    }
    for (int tt = 0; tt < nt; ++tt) {
        const T* row = proj + (size_t)(t0 + tt) * ld;
        float ss = 0.f;
        for (int c = tid; c < K; c += blockDim.x) {
            const float kv = ld_f(row + k_off + h * K + c);
            ss = fmaf(kv, kv, ss);
        }
        ss = warp_sum(ss);
        if ((tid & 31) == 0) red[tt][tid >> 5] = ss;
    }
    __syncthreads();
    const int HK = H * K;
    for (int c = tid; c < K; c += blockDim.x) {
        const int ch = h * K + c;
        float low[VOB_PREP_TOKENS];
#pragma unroll
        for (int tt = 0; tt < VOB_PREP_TOKENS; ++tt) low[tt] = w0[ch];
        // w2t is [R, H * K]: neighbouring threads read neighbouring channels; every element serves all the block's tokens
        for (int j = 0; j < R; ++j) {
            const float wv = ld_f(w2t + (size_t)j * HK + ch);
#pragma unroll
            for (int tt = 0; tt < VOB_PREP_TOKENS; ++tt) low[tt] = fmaf(wv, th[tt * R + j], low[tt]);
        }
        const float ab = a_bias[ch];
#pragma unroll
        for (int tt = 0; tt < VOB_PREP_TOKENS; ++tt) {
            if (tt < nt) {
                const T* row = proj + (size_t)(t0 + tt) * ld;
                const float inv = 1.0f / sqrtf((red[tt][0] + red[tt][1]) + (red[tt][2] + red[tt][3]) + 1e-6f);
                const float u = ld_f(row + k_off + ch) * inv;
                const float a = sigmoidf_(ld_f(row + a_off + ch) + ab);
                const size_t o = (size_t)(t0 + tt) * HK + ch;
                w_out[o] = expf(-0.6065306597126334f * sigmoidf_(low[tt]));
                b_out[o] = a * u;
                u_out[o] = u;
            }
        }
    }
}

// w2t: the second decay projection transposed, [R, H * K].
VOB_EXPORT int vob_delta_prep(const void* proj, int code, long ld, int k_off, int a_off, int low_off, int R, const void* w2t,
                              int w2_code, const float* w0, const float* a_bias, int T, int H, int K, float* w_out, float* b_out,
                              float* u_out, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || K <= 0 || R <= 0 || H > 65535 || (size_t)R * 4 * VOB_PREP_TOKENS > 40 * 1024) return VOB_ERR_BAD_ARG;
    if (code != w2_code) return VOB_ERR_BAD_ARG;
    const int blocks = (T + VOB_PREP_TOKENS - 1) / VOB_PREP_TOKENS;
    VOB_DISPATCH_ELEM(code, return vob_launch(delta_prep_kernel<ElemT, ElemT>, dim3(blocks, H), dim3(128), (size_t)R * 4 * VOB_PREP_TOKENS,
                                              stream, (const ElemT*)proj, ld, k_off, a_off, low_off, R, (const ElemT*)w2t, w0, a_bias, T, H, K,
                                              w_out, b_out, u_out));
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Gated-delta preparation, per token. The columns x_off .. x_off + C - 1 of `proj` [T, ld] hold the q, k and v
// projections side by side (G heads of K, G heads of K, H heads of V; C = 2 G K + H V). Each channel c passes
// a causal convolution over the request's tokens and silu:
//   y_t[c] = sum_i cw[c][taps - 1 - i] * x_(t - i)[c],  i = 0 .. taps - 1;   x before the step's first row comes from
//   the request's convolution state [slots, taps - 1, C] (the last taps - 1 inputs, oldest first; zeros at the start)
// then, all float32:
//   q = silu(y_q) / sqrt(sum_head(.^2) + 1e-6) * K^-1/2,   k = silu(y_k) / sqrt(sum_head(.^2) + 1e-6)
//   v = silu(y_v) (in the activations' type)
//   strength[h] = sigmoid(proj[b_off + h])
//   decay[h, c] = exp(-exp(a_log[h]) * softplus(low[a_off + h K + c] + dt_bias[h K + c]))
//   or, with one decay per head (`decay_per_head`): decay[h, c] = exp(-exp(a_log[h]) * softplus(low[a_off + h] + dt_bias[h]))
//   for every c (the scan reads a decay per key channel either way)
// `low` [T, ld_low] is the output of the second, low-rank projections. Rows with a negative position
// (padding) are skipped. Launch: grid (tokens, ceil(jobs / 4)), blocks of 128 threads; a warp takes one
// head (or one head's decays, or the strengths) of one token. K up to 512.
// ---------------------------------------------------------------------------------------------
// NI: key channels a lane holds of a q or k head, 32 * NI >= K.
template <typename T, int NI>
__global__ void __launch_bounds__(128)
gated_delta_prep_kernel(const T* __restrict__ proj, long ld, int x_off, int b_off, const T* __restrict__ low, long ld_low, int a_off,
                        const float* __restrict__ cw, int taps, const float* __restrict__ cstate, const float* __restrict__ a_log,
                        const float* __restrict__ dt_bias, const int* __restrict__ positions, const int* __restrict__ row_seq,
                        const int* __restrict__ seq_starts, const int* __restrict__ state_slots, int H, int G, int K, int V,
                        float* __restrict__ q_out, float* __restrict__ k_out, T* __restrict__ v_out, float* __restrict__ decay,
                        float* __restrict__ strength, int decay_per_head) {
    pdl_launch_dependents();
    pdl_wait(45);
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (positions[t] < 0) return;
    const int s = row_seq[t];
    const int j = t - seq_starts[s];                 // the row's place among the request's rows of this step
    const int C = 2 * G * K + H * V;
    const float* st = cstate + (size_t)state_slots[s] * (taps - 1) * C;
    auto conv_silu = [&](int c) -> float {
        float y = 0.f;
        for (int i = taps - 1; i >= 0; --i) {        // oldest input first
            const int jj = j - i;
            const float x = jj >= 0 ? ld_f(proj + (size_t)(t - i) * ld + x_off + c) : st[(size_t)(taps - 1 + jj) * C + c];
            y = fmaf(cw[(size_t)c * taps + (taps - 1 - i)], x, y);
        }
        return y / (1.0f + expf(-y));
    };
    const int jobs = 2 * G + 2 * H + 1;
    {
        const int job = blockIdx.y * 4 + warp;
        if (job >= jobs) return;
        if (job < 2 * G) {                           // a q or k head: convolution, silu, unit length
            const bool is_q = job < G;
            const int head = is_q ? job : job - G;
            const int c0 = job * K;                  // q heads then k heads lie side by side
            float x[NI];
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                const int f = lane + 32 * i;
                x[i] = f < K ? conv_silu(c0 + f) : 0.f;
                ss = fmaf(x[i], x[i], ss);
            }
            float mul = 1.0f / sqrtf(warp_sum(ss) + 1e-6f);
            if (is_q) mul *= 1.0f / sqrtf((float)K);
            float* dst = (is_q ? q_out : k_out) + (size_t)t * G * K + (size_t)head * K;
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                const int f = lane + 32 * i;
                if (f < K) dst[f] = x[i] * mul;
            }
        } else if (job < 2 * G + H) {                // a v head: convolution, silu
            const int head = job - 2 * G;
            for (int f = lane; f < V; f += 32)
                st_f(v_out + (size_t)t * H * V + (size_t)head * V + f, conv_silu(2 * G * K + head * V + f));
        } else if (job < 2 * G + 2 * H) {            // a head's decays
            const int head = job - 2 * G - H;
            const float rate = expf(a_log[head]);
            if (decay_per_head) {
                const float z = ld_f(low + (size_t)t * ld_low + a_off + head) + dt_bias[head];
                const float sp = z > 20.f ? z : log1pf(expf(z));
                const float d = expf(-rate * sp);
                for (int f = lane; f < K; f += 32) decay[(size_t)t * H * K + head * K + f] = d;
            } else {
                for (int f = lane; f < K; f += 32) {
                    const int ch = head * K + f;
                    const float z = ld_f(low + (size_t)t * ld_low + a_off + ch) + dt_bias[ch];
                    const float sp = z > 20.f ? z : log1pf(expf(z));
                    decay[(size_t)t * H * K + ch] = expf(-rate * sp);
                }
            }
        } else {                                     // writing strengths
            for (int h = lane; h < H; h += 32)
                strength[(size_t)t * H + h] = sigmoidf_(ld_f(proj + (size_t)t * ld + b_off + h));
        }
    }
}

VOB_EXPORT int vob_gated_delta_prep(const void* proj, int code, long ld, int x_off, int b_off, const void* low, long ld_low, int a_off,
                                    const float* cw, int taps, const float* cstate, const float* a_log, const float* dt_bias,
                                    const int* positions, const int* row_seq, const int* seq_starts, const int* state_slots, int T,
                                    int H, int G, int K, int V, float* q_out, float* k_out, void* v_out, float* decay,
                                    float* strength, int decay_per_head, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || G <= 0 || K <= 0 || V <= 0 || taps < 1 || H % G != 0) return VOB_ERR_BAD_ARG;
    if (K > 512) return VOB_ERR_UNSUPPORTED;
    if ((2 * G + 2 * H + 1 + 3) / 4 > 65535) return VOB_ERR_UNSUPPORTED;
#define VOB_GDPREP(NI_)                                                                                                              \
    VOB_DISPATCH_ELEM(code, return vob_launch(gated_delta_prep_kernel<ElemT, NI_>, dim3(T, (2 * G + 2 * H + 1 + 3) / 4), dim3(128), 0,       \
                                              stream, (const ElemT*)proj, ld, x_off, b_off, (const ElemT*)low, ld_low, a_off, cw, taps,     \
                                              cstate, a_log, dt_bias, positions, row_seq, seq_starts, state_slots, H, G, K, V, q_out, k_out, \
                                              (ElemT*)v_out, decay, strength, decay_per_head))
    if (K <= 32) VOB_GDPREP(1);
    else if (K <= 64) VOB_GDPREP(2);
    else if (K <= 128) VOB_GDPREP(4);
    else if (K <= 256) VOB_GDPREP(8);
    else VOB_GDPREP(16);
#undef VOB_GDPREP
    return 0;
}

// ---------------------------------------------------------------------------------------------
// The convolution state after a step: per request the last taps - 1 inputs of every channel, oldest
// first. A request that brought n rows keeps its own last entries where n < taps - 1:
//   new[m] = x_(n - (taps - 1) + m) if that row is of this step, else old[m + n],   m = 0 .. taps - 2
// (in place, m ascending: old[m + n] lies behind what has been written). Runs behind the kernel
// that read the old state. Launch: grid (requests, ceil(C / 128)). The scan in mode 2 can do the same
// on its way (`conv_x` given): its blocks of a request share the channels out among themselves.
// ---------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void conv_state_shift(const T* __restrict__ x, long ld, int C, int taps, float* __restrict__ st, int r0, int n,
                                                 int c) {
    for (int m = 0; m < taps - 1; ++m) {
        const int tau = n - (taps - 1) + m;
        st[(size_t)m * C + c] = tau >= 0 ? ld_f(x + (size_t)(r0 + tau) * ld + c) : st[(size_t)(m + n) * C + c];
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
conv_state_update_kernel(const T* __restrict__ proj, long ld, int x_off, int C, int taps, float* __restrict__ cstate,
                         const int* __restrict__ seq_starts, const int* __restrict__ state_slots) {
    pdl_launch_dependents();
    pdl_wait(46);
    const int s = blockIdx.x, c = blockIdx.y * 128 + threadIdx.x;
    const int r0 = seq_starts[s], n = seq_starts[s + 1] - r0;
    if (n <= 0 || c >= C) return;
    conv_state_shift(proj + x_off, ld, C, taps, cstate + (size_t)state_slots[s] * (taps - 1) * C, r0, n, c);
}

VOB_EXPORT int vob_conv_state_update(const void* proj, int code, long ld, int x_off, int C, int taps, float* cstate,
                                     const int* seq_starts, const int* state_slots, int seqs, cudaStream_t stream) {
    if (seqs <= 0 || taps <= 1) return 0;
    if (C <= 0 || seqs > 0x7fffffff || (C + 127) / 128 > 65535) return VOB_ERR_BAD_ARG;
    VOB_DISPATCH_ELEM(code, return vob_launch(conv_state_update_kernel<ElemT>, dim3(seqs, (C + 127) / 128), dim3(128), 0, stream,
                                              (const ElemT*)proj, ld, x_off, C, taps, cstate, seq_starts, state_slots));
    return 0;
}

// ---------------------------------------------------------------------------------------------
// A short causal convolution over time on each channel, with the last taps - 1 inputs of a request kept in its state slot:
//   y[t, c] = (bias[c]) + sum_j w[j, c] * x[t - taps + 1 + j, c]      (w [taps, C]; x before this step's rows comes from the state,
//                                                                     which is zero at a request's start)
//   out[t, c] = act(y + (residual ? x[t, c] : 0)),   act: 0 none, 1 silu
// x is a column range of a projection output [T, ld] in the activations' type; out [T, ld_out] of type TO. The state is
// only read here (but see `single`): vob_conv_state_update moves it on behind this kernel. Rows with a negative position
// (padding) get zeros.
// Launch: grid (tokens, ceil(C / 128)), 128 threads, one channel each; the sum runs over the taps in order.
// ---------------------------------------------------------------------------------------------
template <typename T, typename TO>
__global__ void __launch_bounds__(128)
causal_conv_kernel(const T* __restrict__ x, long ld, int C, int taps, const float* __restrict__ w, const float* __restrict__ bias,
                   float* cstate, const int* __restrict__ positions, const int* __restrict__ row_seq,
                   const int* __restrict__ seq_starts, const int* __restrict__ state_slots, int residual, int act,
                   TO* __restrict__ out, long ld_out, int single) {
    pdl_launch_dependents();
    pdl_wait(49);
    const int t = blockIdx.x, c = blockIdx.y * 128 + threadIdx.x;
    if (c >= C) return;
    if (positions[t] < 0) {
        st_f(out + (size_t)t * ld_out + c, 0.f);
        return;
    }
    const int s = row_seq[t];
    const int i = t - seq_starts[s];                 // this row's place among the request's rows of the step
    float* st = cstate ? cstate + (size_t)state_slots[s] * (taps - 1) * C : nullptr;
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;
        const float v = i - back >= 0 ? ld_f(x + (size_t)(t - back) * ld + c) : st[(size_t)(taps - 1 + i - back) * C + c];
        acc = fmaf(w[(size_t)j * C + c], v, acc);
    }
    if (single && st) {      // the request's only row: this thread alone touches its channel of the state, and moves it on
        for (int m = 0; m + 2 < taps; ++m) st[(size_t)m * C + c] = st[(size_t)(m + 1) * C + c];
        st[(size_t)(taps - 2) * C + c] = ld_f(x + (size_t)t * ld + c);
    }
    if (residual) acc += ld_f(x + (size_t)t * ld + c);
    if (act == 1) acc = acc / (1.0f + expf(-acc));
    st_f(out + (size_t)t * ld_out + c, acc);
}

// The same, VEC neighbouring channels a thread (16 bytes of x at a time): C, the row strides and the addresses allow it.
template <typename T, typename TO, int VEC>
__global__ void __launch_bounds__(128)
causal_conv_vec_kernel(const T* __restrict__ x, long ld, int C, int taps, const float* __restrict__ w, const float* __restrict__ bias,
                       float* cstate, const int* __restrict__ positions, const int* __restrict__ row_seq,
                       const int* __restrict__ seq_starts, const int* __restrict__ state_slots, int residual, int act,
                       TO* __restrict__ out, long ld_out, int single) {
    pdl_launch_dependents();
    pdl_wait(49);
    const int t = blockIdx.x, c = (blockIdx.y * 128 + threadIdx.x) * VEC;
    if (c >= C) return;
    float acc[VEC];
    TO* o = out + (size_t)t * ld_out + c;
    if (positions[t] < 0) {
#pragma unroll
        for (int k = 0; k < (int)(VEC * sizeof(TO) / 16); ++k) reinterpret_cast<uint4*>(o)[k] = make_uint4(0u, 0u, 0u, 0u);
        return;
    }
    const int s = row_seq[t];
    const int i = t - seq_starts[s];
    float* st = cstate ? cstate + (size_t)state_slots[s] * (taps - 1) * C : nullptr;
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = bias ? bias[c + e] : 0.f;
    float cur[VEC];
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;
        float v[VEC];
        if (i - back >= 0) {
            const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)(t - back) * ld + c);
            const T* rv = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int e = 0; e < VEC; ++e) v[e] = ld_f(rv + e);
        } else {
            const float* sp = st + (size_t)(taps - 1 + i - back) * C + c;
#pragma unroll
            for (int e = 0; e < VEC; ++e) v[e] = sp[e];
        }
        const float4* wj = reinterpret_cast<const float4*>(w + (size_t)j * C + c);      // C and c are multiples of 4
#pragma unroll
        for (int e4 = 0; e4 < VEC / 4; ++e4) {
            const float4 w4 = wj[e4];
            acc[4 * e4] = fmaf(w4.x, v[4 * e4], acc[4 * e4]);
            acc[4 * e4 + 1] = fmaf(w4.y, v[4 * e4 + 1], acc[4 * e4 + 1]);
            acc[4 * e4 + 2] = fmaf(w4.z, v[4 * e4 + 2], acc[4 * e4 + 2]);
            acc[4 * e4 + 3] = fmaf(w4.w, v[4 * e4 + 3], acc[4 * e4 + 3]);
        }
        if (back == 0) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) cur[e] = v[e];
        } else if (single && st) {
            // the request's only row: every input before it came from the state, and this thread alone touches its channels
            // of it; what it has just read moves one place down (the oldest leaves)
            if (back < taps - 1) {
                float* sp = st + (size_t)(taps - 2 - back) * C + c;
#pragma unroll
                for (int e4 = 0; e4 < VEC / 4; ++e4) reinterpret_cast<float4*>(sp)[e4] = make_float4(v[4 * e4], v[4 * e4 + 1], v[4 * e4 + 2], v[4 * e4 + 3]);
            }
        }
    }
    if (single && st) {
        float* sp = st + (size_t)(taps - 2) * C + c;
#pragma unroll
        for (int e4 = 0; e4 < VEC / 4; ++e4) reinterpret_cast<float4*>(sp)[e4] = make_float4(cur[4 * e4], cur[4 * e4 + 1], cur[4 * e4 + 2], cur[4 * e4 + 3]);
    }
    __align__(16) TO ov[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
        float a = acc[e];
        if (residual) a += cur[e];
        if (act == 1) a = a / (1.0f + expf(-a));
        st_f(ov + e, a);
    }
#pragma unroll
    for (int k = 0; k < (int)(VEC * sizeof(TO) / 16); ++k) reinterpret_cast<uint4*>(o)[k] = reinterpret_cast<const uint4*>(ov)[k];
}

// `single`: the caller knows that every request brings exactly one row; the kernel then also moves the state on (what
// vob_conv_state_update does), each thread for the channels it has just read.
VOB_EXPORT int vob_causal_conv(const void* x, int code, long ld, int C, int taps, const float* w, const float* bias, float* cstate,
                               const int* positions, const int* row_seq, const int* seq_starts, const int* state_slots, int residual,
                               int act, void* out, int out_code, long ld_out, int T, int single, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (C <= 0 || taps < 1 || !w || (taps > 1 && !cstate) || (act != 0 && act != 1) || (C + 127) / 128 > 65535) return VOB_ERR_BAD_ARG;
    const dim3 grid(T, (C + 127) / 128);
    const int vec = code == VOB_BF16 ? 8 : 4;
    const int out_vec = out_code == VOB_BF16 ? 8 : 4;
    const bool by16 = C % vec == 0 && ld % vec == 0 && (((uintptr_t)x) & 15) == 0 && ld_out % out_vec == 0 && (((uintptr_t)out) & 15) == 0 &&
                      (((uintptr_t)w) & 15) == 0 && (((uintptr_t)cstate) & 15) == 0;
#define VOB_CONV(T_, TO_, V_)                                                                                                 \
    return by16 ? vob_launch(causal_conv_vec_kernel<T_, TO_, V_>, dim3(T, (C / V_ + 127) / 128), dim3(128), 0, stream, (const T_*)x, ld, C, \
                             taps, w, bias, cstate, positions, row_seq, seq_starts, state_slots, residual, act, (TO_*)out, ld_out, single) \
                : vob_launch(causal_conv_kernel<T_, TO_>, grid, dim3(128), 0, stream, (const T_*)x, ld, C, taps, w, bias, cstate,  \
                             positions, row_seq, seq_starts, state_slots, residual, act, (TO_*)out, ld_out, single)
    if (code == VOB_F32 && out_code == VOB_F32) VOB_CONV(float, float, 4);
    if (code == VOB_BF16 && out_code == VOB_BF16) VOB_CONV(__nv_bfloat16, __nv_bfloat16, 8);
    if (code == VOB_BF16 && out_code == VOB_F32) VOB_CONV(__nv_bfloat16, float, 8);
#undef VOB_CONV
    return VOB_ERR_BAD_ARG;
}

// ---------------------------------------------------------------------------------------------
// Step sizes and decays of a state-space mixer, per token and head, float32:
//   dt = softplus(raw + dt_bias[h]) (no clamp);   decay = exp(-exp(A_log[h]) * dt)
// raw: H columns of a projection output [T, ld]. Launch: ceil(T * H / 256) blocks of 256 threads.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
ssm_steps_kernel(const T* __restrict__ raw, long ld, const float* __restrict__ dt_bias, const float* __restrict__ a_log, int T_rows,
                 int H, float* __restrict__ dt_out, float* __restrict__ decay_out) {
    pdl_launch_dependents();
    pdl_wait(50);
    const long long e = (long long)blockIdx.x * 256 + threadIdx.x;
    if (e >= (long long)T_rows * H) return;
    const int t = (int)(e / H), h = (int)(e % H);
    const float z = ld_f(raw + (size_t)t * ld + h) + dt_bias[h];
    const float dt = z > 20.f ? z : log1pf(expf(z));       // beyond 20 the two agree to the last bit of a float
    dt_out[e] = dt;
    decay_out[e] = expf(-expf(a_log[h]) * dt);
}

VOB_EXPORT int vob_ssm_steps(const void* raw, int code, long ld, const float* dt_bias, const float* a_log, int T, int H, float* dt_out,
                             float* decay_out, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || !dt_bias || !a_log) return VOB_ERR_BAD_ARG;
    const long long n = (long long)T * H;
    VOB_DISPATCH_ELEM(code, return vob_launch(ssm_steps_kernel<ElemT>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream,
                                              (const ElemT*)raw, ld, dt_bias, a_log, T, H, dt_out, decay_out));
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Behind a state-space scan, per token: y = (o + skip[h] * x) * silu(z), then an RMS norm over each of `groups` equal
// parts of the row (each part by its own root mean square), times weight: the gate comes before the norm.
// o float32 [T, n]; x float32 columns of [T, ld_x]; z columns of a projection output [T, ld_z] in the activations' type;
// skip float32 [H] (one number per head of n / H features); weight float32 [n]; out [T, n] in the activations' type.
// Launch: grid (tokens, groups), 128 threads.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
ssm_post_kernel(const float* __restrict__ o, const float* __restrict__ x, long ld_x, const T* __restrict__ z, long ld_z,
                const float* __restrict__ skip, const float* __restrict__ weight, float eps, int n, int H, int groups,
                T* __restrict__ out, long ld_out) {
    pdl_launch_dependents();
    pdl_wait(51);
    __shared__ float red[4];
    extern __shared__ float yrow[];
    const int t = blockIdx.x, gsz = n / groups, c0 = blockIdx.y * gsz, hv = n / H, tid = threadIdx.x;
    float ss = 0.f;
    for (int c = tid; c < gsz; c += 128) {
        const int f = c0 + c;
        const float zv = ld_f(z + (size_t)t * ld_z + f);
        const float y = fmaf(skip[f / hv], x[(size_t)t * ld_x + f], o[(size_t)t * n + f]) * (zv / (1.0f + expf(-zv)));
        yrow[c] = y;
        ss = fmaf(y, y, ss);
    }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    const float inv = 1.0f / sqrtf(((red[0] + red[1]) + (red[2] + red[3])) / (float)gsz + eps);
    for (int c = tid; c < gsz; c += 128) st_f(out + (size_t)t * ld_out + c0 + c, yrow[c] * inv * weight[c0 + c]);
}

VOB_EXPORT int vob_ssm_post(const float* o, const float* x, long ld_x, const void* z, int code, long ld_z, const float* skip,
                            const float* weight, float eps, int T, int n, int H, int groups, void* out, long ld_out, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (n <= 0 || H <= 0 || groups <= 0 || n % H || n % groups || groups > 65535 || !skip || !weight) return VOB_ERR_BAD_ARG;
    const size_t smem = (size_t)(n / groups) * sizeof(float);
    if (smem > 40 * 1024) return VOB_ERR_UNSUPPORTED;
    VOB_DISPATCH_ELEM(code, return vob_launch(ssm_post_kernel<ElemT>, dim3(T, groups), dim3(128), smem, stream, o, x, ld_x, (const ElemT*)z,
                                              ld_z, skip, weight, eps, n, H, groups, (ElemT*)out, ld_out));
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Rotary positions and a scale, to float32: for every head of D features, feature i < rot / 2 is
// paired with feature i + rot / 2 and the pair (a, b) becomes (a cos - b sin, b cos + a sin) with
// the angle float(position) * inv_freq[i]; features from `rot` on pass unchanged; everything is
// multiplied by `scale`. src is a column range of a projection output [T, ld]; out [T, H * D].
// Rows with a negative position (padding) are written as zeros.
// Launch: one block of 128 threads per token.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
rotate_scale_kernel(const T* __restrict__ src, long ld, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                    int H, int D, int rot, float scale, float* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait(42);
    const int t = blockIdx.x;
    const int pos = positions[t];
    const T* row = src + (size_t)t * ld;
    float* o = out + (size_t)t * H * D;
    const int half = rot >> 1;
    for (int e = threadIdx.x; e < H * D; e += blockDim.x) {
        const int f = e % D;
        float v = 0.f;
        if (pos >= 0) {
            if (f < rot) {
                const int i = f < half ? f : f - half;
                const float ang = (float)pos * inv_freq[i];
                const float cs = cosf(ang), sn = sinf(ang);
                const float a = ld_f(row + e - f + i), b = ld_f(row + e - f + i + half);
                v = f < half ? a * cs - b * sn : b * cs + a * sn;
            } else {
                v = ld_f(row + e);
            }
            v *= scale;
        }
        o[e] = v;
    }
}

VOB_EXPORT int vob_rotate_scale(const void* src, int code, long ld, const int* positions, const float* inv_freq, int T, int H,
                                int D, int rot, float scale, float* out, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || D <= 0 || rot < 0 || rot > D || (rot & 1)) return VOB_ERR_BAD_ARG;
    VOB_DISPATCH_ELEM(code, return vob_launch(rotate_scale_kernel<ElemT>, dim3(T), dim3(128), 0, stream, (const ElemT*)src, ld,
                                              positions, inv_freq, H, D, rot, scale, out));
    return 0;
}

// ---------------------------------------------------------------------------------------------
// The scan. Grid (ceil(V / VT), H, requests); block VT * KS threads, lane = column * KS + q.
// r, k: [T, >= H * K] with row strides; v: [T, >= H * V]; w, b, u: float32 [T, H * K] (mode 0) or
// w = float32 [H] (mode 1); state float32 [slots, H, K, V]; o float32 [T, H * V].
// A request's rows are seq_starts[s] .. seq_starts[s + 1] - 1 (none: the block leaves at once and
// its state slot is not touched). VT = 128 / KS.
// ---------------------------------------------------------------------------------------------
template <int MODE, int KPT, int KS, typename TRK, typename TV>
__global__ void __launch_bounds__(128, 1)
recurrence_scan_kernel(const TRK* __restrict__ r, long ld_r, const TRK* __restrict__ k, long ld_k, const TV* __restrict__ v,
                       long ld_v, const float* __restrict__ w, const float* __restrict__ b, const float* __restrict__ u,
                       float* __restrict__ state, const int* __restrict__ seq_starts, const int* __restrict__ state_slots,
                       float* __restrict__ o, int H, int K, int V, int rk_div, const TV* __restrict__ conv_x, long ld_cx, int conv_c,
                       int conv_taps, float* __restrict__ conv_state) {
    // Every size of the tiling is a constant, so that staging a token is a few plain loads and stores: what one token
    // needs is one list of PER elements (r, k and in mode 0 w, b, u over KPAD channels, then v over VT columns), thread
    // t takes elements t, t + 128, ... of it (NPT per token), and the list of the next CT tokens is fetched into
    // registers while the staged tokens are worked on. The chain from token to token is what bounds a long portion.
    constexpr int KPAD = KS * KPT, VT = 128 / KS, NA = MODE == 0 ? 5 : MODE == 2 ? 3 : 2;
    constexpr int NB = MODE == 2 ? 1 : MODE == 3 ? 2 : 0;   // mode 2: one more element per token, the writing strength; mode 3: decay and step size
    // Lane q of a column holds key channels q * KPT .. q * KPT + KPT - 1. In shared memory a lane's channels lie
    // together (read four at a time), each lane's group padded by four floats so that the KS groups fall into
    // different banks: channel c of an array at (c / KPT) * (KPT + 4) + c % KPT.
    constexpr int GRP = KPT + 4, KPADP = KS * GRP;
    constexpr int PER = NA * KPADP + VT + 4 * NB, NPT = (NA * KPAD + VT + NB + 127) / 128;
    constexpr int CT = NPT >= 24 ? 1 : (24 / NPT > 8 ? 8 : 24 / NPT);
    pdl_launch_dependents();
    pdl_wait(43);
    const int s = blockIdx.z, h = blockIdx.y;
    const int hk = h / rk_div;                       // the head whose r and k this head reads
    const int r0 = seq_starts[s], r1 = seq_starts[s + 1];
    if (r1 <= r0) return;
    __shared__ __align__(16) float sm[CT * PER];     // token tt: [r | k | (w | b | u) | v | (strength)] at sm + tt * PER
    const int tid = threadIdx.x;
    if (MODE == 2 && conv_x) {
        // the convolutions' last inputs of this request (the kernel that read the old ones has completed)
        float* st = conv_state + (size_t)state_slots[s] * (conv_taps - 1) * conv_c;
        const int blocks = gridDim.x * gridDim.y;
        for (int c = (blockIdx.y * gridDim.x + blockIdx.x) * 128 + tid; c < conv_c; c += blocks * 128)
            conv_state_shift(conv_x, ld_cx, conv_c, conv_taps, st, r0, r1 - r0, c);
    }
    const int q = tid % KS, jj = tid / KS;
    const int j = blockIdx.x * VT + jj;
    const bool col = j < V;
    float* S_glob = state + ((size_t)state_slots[s] * H + h) * K * V;
    float S[KPT];
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
        const int c = q * KPT + i;
        S[i] = (col && c < K) ? S_glob[(size_t)c * V + j] : 0.f;
    }
    const float decay = MODE == 1 ? w[h] : 0.f;
    unsigned pre[CT * NPT];              // raw bits: converted when they are staged, not when they arrive
    auto fetch = [&](int c0, int n) {
#pragma unroll
        for (int tt = 0; tt < CT; ++tt) {
            const size_t row = (size_t)(c0 + tt);
#pragma unroll
            for (int i = 0; i < NPT; ++i) {
                const int x = tid + i * 128;            // which array and channel x is does not depend on the token
                unsigned val = 0u;                      // the bits of 0 in either type
                if (tt < n && x < NA * KPAD + VT + NB) {
                    if (x < NA * KPAD) {
                        const int a = x / KPAD, c = x % KPAD;
                        if (c < K) {
                            const size_t g = row * H * K + h * K + c;
                            val = a == 0 ? raw_ld(r + row * ld_r + hk * K + c) : a == 1 ? raw_ld(k + row * ld_k + hk * K + c)
                                : a == 2 ? raw_ld(w + g) : a == 3 ? raw_ld(b + g) : raw_ld(u + g);
                        }
                    } else if (x == NA * KPAD + VT) {
                        val = raw_ld(b + row * H + h);
                    } else if (MODE == 3 && x == NA * KPAD + VT + 1) {
                        val = raw_ld(u + row * H + h);
                    } else {
                        const int jv = blockIdx.x * VT + (x - NA * KPAD);
                        if (jv < V) val = raw_ld(v + row * ld_v + h * V + jv);
                    }
                }
                pre[tt * NPT + i] = val;
            }
        }
    };
    fetch(r0, min(CT, r1 - r0));
    for (int c0 = r0; c0 < r1; c0 += CT) {
        const int n = min(CT, r1 - c0);
        __syncthreads();                     // the tokens staged before have been used
#pragma unroll
        for (int tt = 0; tt < CT; ++tt)
#pragma unroll
            for (int i = 0; i < NPT; ++i) {
                const int x = tid + i * 128;
                if (x < NA * KPAD) {
                    const int a = x / KPAD, c = x % KPAD;
                    sm[tt * PER + a * KPADP + (c / KPT) * GRP + c % KPT] =
                        a < 2 ? raw_to_float<TRK>(pre[tt * NPT + i]) : __uint_as_float(pre[tt * NPT + i]);
                } else if (x < NA * KPAD + VT) {
                    sm[tt * PER + NA * KPADP + (x - NA * KPAD)] = raw_to_float<TV>(pre[tt * NPT + i]);
                } else if (NB && x == NA * KPAD + VT) {
                    sm[tt * PER + NA * KPADP + VT] = __uint_as_float(pre[tt * NPT + i]);
                } else if (NB == 2 && x == NA * KPAD + VT + 1) {
                    sm[tt * PER + NA * KPADP + VT + 1] = __uint_as_float(pre[tt * NPT + i]);
                }
            }
        __syncthreads();
        if (c0 + CT < r1) fetch(c0 + CT, min(CT, r1 - c0 - CT));
        for (int tt = 0; tt < n; ++tt) {
            const float4* pr = reinterpret_cast<const float4*>(sm + tt * PER + q * GRP);
            const float4* pk = reinterpret_cast<const float4*>(sm + tt * PER + KPADP + q * GRP);
            const float vj = sm[tt * PER + NA * KPADP + jj];
            float rr[KPT], kk[KPT];
#pragma unroll
            for (int i = 0; i < KPT / 4; ++i) {
                const float4 a = pr[i], c = pk[i];
                rr[4 * i] = a.x; rr[4 * i + 1] = a.y; rr[4 * i + 2] = a.z; rr[4 * i + 3] = a.w;
                kk[4 * i] = c.x; kk[4 * i + 1] = c.y; kk[4 * i + 2] = c.z; kk[4 * i + 3] = c.w;
            }
            if (MODE == 0) {
                const float4* pw = reinterpret_cast<const float4*>(sm + tt * PER + 2 * KPADP + q * GRP);
                const float4* pb = reinterpret_cast<const float4*>(sm + tt * PER + 3 * KPADP + q * GRP);
                const float4* pu = reinterpret_cast<const float4*>(sm + tt * PER + 4 * KPADP + q * GRP);
                // four partial sums: the chain of dependent additions is a quarter as long; their order is fixed
                float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
                for (int i = 0; i < KPT / 4; ++i) {
                    const float4 uu = pu[i];
                    d0 = fmaf(uu.x, S[4 * i], d0);
                    d1 = fmaf(uu.y, S[4 * i + 1], d1);
                    d2 = fmaf(uu.z, S[4 * i + 2], d2);
                    d3 = fmaf(uu.w, S[4 * i + 3], d3);
                }
                float dot = (d0 + d1) + (d2 + d3);
#pragma unroll
                for (int off = 1; off < KS; off <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
#pragma unroll
                for (int i = 0; i < KPT / 4; ++i) {
                    const float4 ww = pw[i], bb = pb[i];
                    S[4 * i] = fmaf(kk[4 * i], vj, fmaf(ww.x, S[4 * i], -(bb.x * dot)));
                    S[4 * i + 1] = fmaf(kk[4 * i + 1], vj, fmaf(ww.y, S[4 * i + 1], -(bb.y * dot)));
                    S[4 * i + 2] = fmaf(kk[4 * i + 2], vj, fmaf(ww.z, S[4 * i + 2], -(bb.z * dot)));
                    S[4 * i + 3] = fmaf(kk[4 * i + 3], vj, fmaf(ww.w, S[4 * i + 3], -(bb.w * dot)));
                }
            } else if (MODE == 2) {
                // Decay first, then the delta-rule write against the decayed state S'. The read-out sees the write:
                // o = (S' + k uu)^T r = S'^T r + (k . r) uu, so the three sums over key channels (k . S', r . S', k . r)
                // are taken in one pass and finished by ONE round of shuffles, and the token-to-token chain is
                // decay -> sums -> shuffles -> write (the read-out hangs off it instead of lengthening it).
                const float4* pw = reinterpret_cast<const float4*>(sm + tt * PER + 2 * KPADP + q * GRP);
                const float strength = sm[tt * PER + NA * KPADP + VT];
                float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f, e0 = 0.f, e1 = 0.f, e2 = 0.f, e3 = 0.f, f0 = 0.f, f1 = 0.f, f2 = 0.f, f3 = 0.f;
#pragma unroll
                for (int i = 0; i < KPT / 4; ++i) {
                    const float4 ww = pw[i];
                    S[4 * i] *= ww.x; S[4 * i + 1] *= ww.y; S[4 * i + 2] *= ww.z; S[4 * i + 3] *= ww.w;
                    d0 = fmaf(kk[4 * i], S[4 * i], d0);
                    d1 = fmaf(kk[4 * i + 1], S[4 * i + 1], d1);
                    d2 = fmaf(kk[4 * i + 2], S[4 * i + 2], d2);
                    d3 = fmaf(kk[4 * i + 3], S[4 * i + 3], d3);
                    e0 = fmaf(rr[4 * i], S[4 * i], e0);
                    e1 = fmaf(rr[4 * i + 1], S[4 * i + 1], e1);
                    e2 = fmaf(rr[4 * i + 2], S[4 * i + 2], e2);
                    e3 = fmaf(rr[4 * i + 3], S[4 * i + 3], e3);
                    f0 = fmaf(rr[4 * i], kk[4 * i], f0);
                    f1 = fmaf(rr[4 * i + 1], kk[4 * i + 1], f1);
                    f2 = fmaf(rr[4 * i + 2], kk[4 * i + 2], f2);
                    f3 = fmaf(rr[4 * i + 3], kk[4 * i + 3], f3);
                }
                float dot = (d0 + d1) + (d2 + d3), read = (e0 + e1) + (e2 + e3), rk = (f0 + f1) + (f2 + f3);
#pragma unroll
                for (int off = 1; off < KS; off <<= 1) {
                    dot += __shfl_xor_sync(0xffffffffu, dot, off);
                    read += __shfl_xor_sync(0xffffffffu, read, off);
                    rk += __shfl_xor_sync(0xffffffffu, rk, off);
                }
                const float uu = strength * (vj - dot);
#pragma unroll
                for (int i = 0; i < KPT; ++i) S[i] = fmaf(kk[i], uu, S[i]);
                if (q == 0 && col) o[(size_t)(c0 + tt) * H * V + h * V + j] = fmaf(rk, uu, read);
                continue;
            } else if (MODE == 3) {
                const float a = sm[tt * PER + NA * KPADP + VT], dv = sm[tt * PER + NA * KPADP + VT + 1] * vj;
#pragma unroll
                for (int i = 0; i < KPT; ++i) S[i] = fmaf(kk[i], dv, a * S[i]);
            } else {
#pragma unroll
                for (int i = 0; i < KPT; ++i) S[i] = fmaf(kk[i], vj, decay * S[i]);
            }
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
            for (int i = 0; i < KPT / 4; ++i) {
                a0 = fmaf(rr[4 * i], S[4 * i], a0);
                a1 = fmaf(rr[4 * i + 1], S[4 * i + 1], a1);
                a2 = fmaf(rr[4 * i + 2], S[4 * i + 2], a2);
                a3 = fmaf(rr[4 * i + 3], S[4 * i + 3], a3);
            }
            float acc = (a0 + a1) + (a2 + a3);
#pragma unroll
            for (int off = 1; off < KS; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            if (q == 0 && col) o[(size_t)(c0 + tt) * H * V + h * V + j] = acc;
        }
    }
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
        const int c = q * KPT + i;
        if (col && c < K) S_glob[(size_t)c * V + j] = S[i];
    }
}

// How the key channels are shared out: KS lanes per column (a power of two) with KPT state registers each:
// K <= 32: 4 x 8; <= 64: 4 x 16; <= 128: 8 x 16; <= 256: 16 x 16; <= 512: 32 x 16.
template <int MODE, typename TRK, typename TV>
static int scan_launch(const void* r, long ld_r, const void* k, long ld_k, const void* v, long ld_v, const float* w, const float* b,
                       const float* u, float* state, const int* seq_starts, const int* state_slots, float* o, int seqs, int H, int K,
                       int V, int rk_div, const void* conv_x, long ld_cx, int conv_c, int conv_taps, float* conv_state, cudaStream_t stream) {
#define VOB_SCAN(P, KS_)                                                                                                        \
    return vob_launch(recurrence_scan_kernel<MODE, P, KS_, TRK, TV>, dim3((V + 128 / KS_ - 1) / (128 / KS_), H, seqs), dim3(128), 0,  \
                      stream, (const TRK*)r, ld_r, (const TRK*)k, ld_k, (const TV*)v, ld_v, w, b, u, state, seq_starts, state_slots, o, \
                      H, K, V, rk_div, (const TV*)conv_x, ld_cx, conv_c, conv_taps, conv_state)
    if (K <= 32) VOB_SCAN(8, 4);
    if (K <= 64) VOB_SCAN(16, 4);
    if (K <= 128) VOB_SCAN(16, 8);
    if (K <= 256) VOB_SCAN(16, 16);
    VOB_SCAN(16, 32);
#undef VOB_SCAN
}

VOB_EXPORT int vob_recurrence_scan(int mode, const void* r, long ld_r, const void* k, long ld_k, int rk_code, const void* v, long ld_v,
                                   int v_code, const float* w, const float* b, const float* u, float* state, const int* seq_starts,
                                   const int* state_slots, float* o, int seqs, int H, int K, int V, int rk_div, const void* conv_x,
                                   long ld_cx, int conv_c, int conv_taps, float* conv_state, cudaStream_t stream) {
    if (seqs <= 0) return 0;
    if (H <= 0 || K <= 0 || V <= 0 || H > 65535 || seqs > 65535) return VOB_ERR_BAD_ARG;
    if (K > 512) return VOB_ERR_UNSUPPORTED;
    if (mode == 0 && (!w || !b || !u)) return VOB_ERR_BAD_ARG;
    if (mode == 1 && !w) return VOB_ERR_BAD_ARG;
    if (mode == 2 && (!w || !b)) return VOB_ERR_BAD_ARG;
    if (mode == 3 && (!b || !u)) return VOB_ERR_BAD_ARG;
    if (rk_div <= 0 || H % rk_div != 0 || (mode != 2 && mode != 3 && rk_div != 1)) return VOB_ERR_BAD_ARG;
    // conv_x (mode 2, optional): columns of the activations' type (v's) whose last conv_taps - 1 rows per request are
    // left in conv_state [slots, conv_taps - 1, conv_c]
    if (conv_x && (mode != 2 || conv_c <= 0 || conv_taps < 2 || !conv_state)) return VOB_ERR_BAD_ARG;
#define VOB_ARGS r, ld_r, k, ld_k, v, ld_v, w, b, u, state, seq_starts, state_slots, o, seqs, H, K, V, rk_div, conv_x, ld_cx, conv_c, conv_taps, conv_state, stream
    if (mode == 0 && rk_code == VOB_F32 && v_code == VOB_F32) return scan_launch<0, float, float>(VOB_ARGS);
    if (mode == 0 && rk_code == VOB_BF16 && v_code == VOB_BF16) return scan_launch<0, __nv_bfloat16, __nv_bfloat16>(VOB_ARGS);
    if (mode == 1 && rk_code == VOB_F32 && v_code == VOB_F32) return scan_launch<1, float, float>(VOB_ARGS);
    if (mode == 1 && rk_code == VOB_F32 && v_code == VOB_BF16) return scan_launch<1, float, __nv_bfloat16>(VOB_ARGS);
    if (mode == 2 && rk_code == VOB_F32 && v_code == VOB_F32) return scan_launch<2, float, float>(VOB_ARGS);
    if (mode == 2 && rk_code == VOB_F32 && v_code == VOB_BF16) return scan_launch<2, float, __nv_bfloat16>(VOB_ARGS);
    if (mode == 3 && rk_code == VOB_F32 && v_code == VOB_F32) return scan_launch<3, float, float>(VOB_ARGS);
#undef VOB_ARGS
    return VOB_ERR_BAD_ARG;
}

// ---------------------------------------------------------------------------------------------
// After the scan, per token and head: out = o / sqrt(mean(o^2) + eps) * weight * gate(g), with
// weight optional ([H * V] float32) and gate = sigmoid (0) or silu (1) of the gate projection g, a
// column range of a projection output [T, ld_g]. out [T, H * V] in the activations' type, rows `ld_out`
// apart, everything times `out_scale`.
// Launch: one block of 128 threads per (token, head).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
recurrence_post_kernel(const float* __restrict__ o, const T* __restrict__ g, long ld_g, const float* __restrict__ weight,
                       int gate_mode, float eps, int H, int V, T* __restrict__ out, long ld_out, float out_scale) {
    pdl_launch_dependents();
    pdl_wait(44);
    __shared__ float red[4];
    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const float* orow = o + (size_t)t * H * V + h * V;
    float ss = 0.f;
    for (int c = tid; c < V; c += blockDim.x) ss = fmaf(orow[c], orow[c], ss);
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    const float inv = 1.0f / sqrtf(((red[0] + red[1]) + (red[2] + red[3])) / (float)V + eps);
    for (int c = tid; c < V; c += blockDim.x) {
        const float gv = ld_f(g + (size_t)t * ld_g + h * V + c);
        const float sg = sigmoidf_(gv);
        float val = orow[c] * inv;
        if (weight) val *= weight[h * V + c];
        val *= gate_mode == 1 ? gv * sg : sg;
        st_f(out + (size_t)t * ld_out + h * V + c, val * out_scale);
    }
}

VOB_EXPORT int vob_recurrence_post(const float* o, const void* g, int code, long ld_g, const float* weight, int gate_mode, float eps,
                                   int T, int H, int V, void* out, long ld_out, float out_scale, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || V <= 0 || H > 65535 || (gate_mode != 0 && gate_mode != 1) || ld_out < (long)H * V) return VOB_ERR_BAD_ARG;
    VOB_DISPATCH_ELEM(code, return vob_launch(recurrence_post_kernel<ElemT>, dim3(T, H), dim3(128), 0, stream, o, (const ElemT*)g, ld_g,
                                              weight, gate_mode, eps, H, V, (ElemT*)out, ld_out, out_scale));
    return 0;
}
