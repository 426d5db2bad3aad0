// Softmax attention over a paged cache whose keys and values have sizes of their own, with the
// options a design may switch on one by one: rotary positions on part of each head, q and k brought
// to unit root mean square, a query factor that grows with the position, values mixed with those an
// earlier layer made of the same token, a window, blocks of positions, a cap on the scores, a bias that grows with the
// distance, a sink in the softmax, a sigmoid gate on the result.
//
// Two steps per call of a layer:
//   vob_flex_prep      per token: q, k, v (columns of one projection output) -> q' to a buffer, k' and
//                      v' to their cache slots;
//   vob_flex_attention per (row, head a), the row at position p of its request, g = a / (H / G):
//       s_j = (q'_a . K[j, g]) * scale          for keys j in [first, p], first = max(0, p + 1 - window), and with
//                                                `chunk` not before p - p % chunk (the query's own block of positions)
//       with `pool` (and a window): every block of `pool` positions that ends at or before p - window is one more key and
//                                                value, the means of the block's keys and values, in the same softmax
//       s_j <- cap * tanh(s_j / cap)  (cap > 0);   s_j <- s_j - r1_a * ln(1 + r2_a * (p - j))  (r1, r2 given)
//       den = sum_j exp(s_j) (+ exp(sink_a): a key with no value, counted once)
//       out_a = sum_j exp(s_j) V[j, g] / den    (* sigmoid(gate) * out_scale)
// The step's own keys are in the cache before they are read. Scores, softmax, angles, norms and the
// query factor are float32. Cache layout per layer: K [pages][G][page_size][D], V [pages][G][page_size][DV].
#include "common.cuh"
VOB_PDL_SWITCH(attention_flex)

// ---------------------------------------------------------------------------------------------
// Preparation. Grid (tokens, ceil((H + 2 G) / 8)), blocks of 256 threads: a warp takes one head of one token
// (q heads, then k heads, then v heads), lane l holding features l, l + 32, ... (heads up to 256 wide); a
// head is a short chain of loads, a reduction and stores, so many independent warps are what hides it, and
// the head's features are asked for before the token's position and slot are known (padding rows are rows of
// the projection like any other).
//   q, k:  the first `rot` features of a head are rotated, feature i with i + rot / 2, by
//          float(pos) * inv_freq[i]; then (unit_rms) the head is divided by sqrt(mean(x^2) + eps) and, where a
//          weight of D entries is given (`q_norm_w`, `k_norm_w`, shared by the heads), multiplied by it;
//          q is also multiplied by 1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1) (temp_every > 0).
//          With `q_pre_w` [H * D] / `k_pre_w` [G * D]: BEFORE the rotation the whole projection (all heads at once) is
//          divided by its root mean square, sqrt(mean over all its features of x^2 + eps), and multiplied by that weight.
//   v:     v_mode 1: the values are also left in `v_first` [T, G * DV] for later layers of this step;
//          v_mode 2: v <- (1 - lambda) v + lambda v_first, lambda = *vmix.
// Rows with a negative position (padding) are left alone; a negative slot skips the cache write. Without a cache
// (a layer that reads the keys and values another layer wrote) only the queries are prepared.
// ---------------------------------------------------------------------------------------------
// NI: features a lane holds of a q or k head, 32 * NI >= D.
template <typename T, int NI>
__global__ void __launch_bounds__(256, 4)
flex_prep_kernel(const T* __restrict__ proj, long ld, int q_off, int k_off, int v_off, const int* __restrict__ positions,
                 const int* __restrict__ slots, const float* __restrict__ inv_freq, int rot, int unit_rms, float eps,
                 float temp_coef, int temp_every, const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w,
                 const float* __restrict__ q_pre_w, const float* __restrict__ k_pre_w, const float* __restrict__ vmix, T* __restrict__ v_first, int v_mode, T* __restrict__ q_out, long ld_q, T* __restrict__ kcache, T* __restrict__ vcache, int H, int G, int D, int DV,
                 int page_size) {
    pdl_launch_dependents();
    pdl_wait(61);
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = positions[t];
    const int slot = slots ? slots[t] : -1;
    const T* row = proj + (size_t)t * ld;
    const int half = rot >> 1;
    {
        const int job = blockIdx.y * 8 + warp;
        if (job >= (kcache ? H + 2 * G : H)) return;       // no cache given: only the queries are prepared
        if (job < H + G) {
            const bool is_q = job < H;
            const int head = is_q ? job : job - H;
            const T* src = row + (is_q ? q_off : k_off) + (size_t)head * D;
            float x[NI], y[NI];                      // a feature and, where it is rotated, its partner
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                const int f = lane + 32 * i;
                x[i] = f < D ? ld_f(src + f) : 0.f;
                y[i] = f < rot ? ld_f(src + (f < half ? f + half : f - half)) : 0.f;
            }
            const float* pre_w = is_q ? q_pre_w : k_pre_w;
            if (pre_w) {
                // a norm over the WHOLE projection (all heads of q, or of k, at once) with a weight per feature, before the
                // rotation: every warp sums the projection's squares for itself (the same sum in the same order)
                const int n = (is_q ? H : G) * D;
                const T* base = row + (is_q ? q_off : k_off);
                float sq = 0.f;
                for (int f = lane; f < n; f += 32) {
                    const float v = ld_f(base + f);
                    sq = fmaf(v, v, sq);
                }
                const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)n + eps);
                const float* hw = pre_w + (size_t)head * D;
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    const int f = lane + 32 * i;
                    if (f < D) x[i] *= inv * hw[f];
                    if (f < rot) y[i] *= inv * hw[f < half ? f + half : f - half];
                }
            }
            if (pos < 0) return;
            const float fpos = (float)pos;
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                const int f = lane + 32 * i;
                if (f < rot) {
                    const float ang = fpos * inv_freq[f < half ? f : f - half];
                    const float sn = sinf(ang), cs = cosf(ang);
                    x[i] = f < half ? x[i] * cs - y[i] * sn : x[i] * cs + y[i] * sn;
                }
                ss = fmaf(x[i], x[i], ss);
            }
            float mul = 1.f;
            if (unit_rms) mul = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
            if (is_q && temp_every > 0) mul *= 1.0f + temp_coef * logf((float)((pos + 1) / temp_every + 1));
            const float* nw = is_q ? q_norm_w : k_norm_w;
            T* dst;
            if (is_q) {
                dst = q_out + (size_t)t * ld_q + (size_t)head * D;
            } else {
                if (slot < 0) return;
                dst = kcache + ((size_t)((slot / page_size) * G + head) * page_size + slot % page_size) * D;
            }
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                const int f = lane + 32 * i;
                if (f < D) st_f(dst + f, nw ? x[i] * mul * nw[f] : x[i] * mul);
            }
        } else {
            if (pos < 0) return;
            const int head = job - H - G;
            const T* src = row + v_off + (size_t)head * DV;
            T* vf = v_first ? v_first + ((size_t)t * G + head) * DV : nullptr;
            T* dst = slot >= 0 ? vcache + ((size_t)((slot / page_size) * G + head) * page_size + slot % page_size) * DV : nullptr;
            const float lam = v_mode == 2 ? *vmix : 0.f;
            for (int f = lane; f < DV; f += 32) {
                float v = ld_f(src + f);
                if (v_mode == 2) v = (1.0f - lam) * v + lam * ld_f(vf + f);
                if (v_mode == 1) st_f(vf + f, v);
                if (dst) st_f(dst + f, v);
            }
        }
    }
}

VOB_EXPORT int vob_flex_prep(const void* proj, int code, long ld, int q_off, int k_off, int v_off, const int* positions,
                             const int* slots, const float* inv_freq, int rot, int unit_rms, float eps, float temp_coef,
                             int temp_every, const float* q_norm_w, const float* k_norm_w, const float* q_pre_w, const float* k_pre_w,
                             const float* vmix, void* v_first,
                             int v_mode, void* q_out, long ld_q, void* kcache,
                             void* vcache, int T, int H, int G, int D, int DV, int page_size, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || G <= 0 || D <= 0 || DV <= 0 || page_size <= 0 || rot < 0 || rot > D || (rot & 1)) return VOB_ERR_BAD_ARG;
    if (D > 256) return VOB_ERR_UNSUPPORTED;
    if (rot > 0 && !inv_freq) return VOB_ERR_BAD_ARG;
    if ((v_mode == 1 || v_mode == 2) && !v_first) return VOB_ERR_BAD_ARG;
    if (v_mode == 2 && !vmix) return VOB_ERR_BAD_ARG;
    if ((H + 2 * G + 7) / 8 > 65535) return VOB_ERR_UNSUPPORTED;
#define VOB_PREP(NI_)                                                                                                                  \
    VOB_DISPATCH_ELEM(code, return vob_launch(flex_prep_kernel<ElemT, NI_>, dim3(T, (H + 2 * G + 7) / 8), dim3(256), 0, stream,              \
                                              (const ElemT*)proj, ld, q_off, k_off, v_off, positions, slots, inv_freq, rot, unit_rms, eps,  \
                                              temp_coef, temp_every, q_norm_w, k_norm_w, q_pre_w, k_pre_w, vmix, (ElemT*)v_first, v_mode, (ElemT*)q_out,  \
                                              ld_q, (ElemT*)kcache,                                                                      \
                                              (ElemT*)vcache, H, G, D, DV, page_size))
    if (D <= 32) VOB_PREP(1);
    else if (D <= 64) VOB_PREP(2);
    else if (D <= 128) VOB_PREP(4);
    else VOB_PREP(8);
#undef VOB_PREP
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Pooled entries. A row at position p with (p + 1) % pool == 0 ends the block b = p / pool of `pool` tokens: the mean of
// the block's cached keys and the mean of its cached values (float32 sums in token order, one division) are written to
// kpool / vpool, which are laid out like the caches, at the place a token at position b would have (a request that holds
// pages for its tokens holds that place too). Runs behind the kernel that wrote the step's keys and values; other rows
// leave at once. Launch: grid (rows, kv heads), 128 threads.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
pool_blocks_kernel(const T* __restrict__ kcache, const T* __restrict__ vcache, T* __restrict__ kpool, T* __restrict__ vpool,
                   const int* __restrict__ block_tables, int max_pages, const int* __restrict__ row_seq,
                   const int* __restrict__ positions, int G, int D, int DV, int page_size, int pool) {
    pdl_launch_dependents();
    pdl_wait(63);
    const int t = blockIdx.x, g = blockIdx.y;
    const int pos = positions[t];
    if (pos < 0 || (pos + 1) % pool != 0) return;
    const int* bt = block_tables + (size_t)row_seq[t] * max_pages;
    const int b = pos / pool, first = b * pool;
    const size_t dst = (size_t)(bt[b / page_size] * G + g) * page_size + b % page_size;
    const float inv = 1.0f / (float)pool;
    for (int d = threadIdx.x; d < D + DV; d += 128) {
        const bool key = d < D;
        const T* src = key ? kcache : vcache;
        const int w = key ? D : DV, c = key ? d : d - D;
        float acc = 0.f;
        for (int j = first; j <= pos; ++j)
            acc += ld_f(src + ((size_t)(bt[j / page_size] * G + g) * page_size + j % page_size) * w + c);
        st_f((key ? kpool : vpool) + dst * w + c, acc * inv);
    }
}

VOB_EXPORT int vob_pool_blocks(const void* kcache, const void* vcache, void* kpool, void* vpool, int code, const int* block_tables,
                               int max_pages, const int* row_seq, const int* positions, int T_rows, int G, int D, int DV, int page_size,
                               int pool, cudaStream_t stream) {
    if (T_rows <= 0) return 0;
    if (G <= 0 || G > 65535 || D <= 0 || DV <= 0 || page_size <= 0 || max_pages <= 0 || pool <= 0) return VOB_ERR_BAD_ARG;
    VOB_DISPATCH_ELEM(code, return vob_launch(pool_blocks_kernel<ElemT>, dim3(T_rows, G), dim3(128), 0, stream, (const ElemT*)kcache,
                                              (const ElemT*)vcache, (ElemT*)kpool, (ElemT*)vpool, block_tables, max_pages, row_seq, positions,
                                              G, D, DV, page_size, pool));
    return 0;
}

// ---------------------------------------------------------------------------------------------
// General kernel: one warp per (row, head). Keys are visited in chunks of 32: each lane scores one
// key against q held in shared memory, the warp agrees on the running maximum, then the 32 weighted
// value rows are summed with lane l holding value features l, l + 32, ... Any D, DV up to 256, any
// H, G, page size. This is the kernel of the 32-bit engine and the one the bfloat16 engine falls
// back to. A row's result depends only on its own q and keys, never on the batch around it: keys
// are walked from the first visible one in chunks that start there.
// Launch: ceil(T * H / 4) blocks of 128 threads; 4 * D floats of shared memory.
// ---------------------------------------------------------------------------------------------
template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    __device__ static inline void load(const float* p, float* o) {
        float4 v = *reinterpret_cast<const float4*>(p);
        o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
    }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static inline void load(const __nv_bfloat16* p, float* o) {
        uint4 v = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __bfloat1622float2(h[i]);
            o[2 * i] = f.x; o[2 * i + 1] = f.y;
        }
    }
};

__device__ __forceinline__ float flex_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

template <typename T>
__global__ void __launch_bounds__(128, 8)
flex_attention_warp_kernel(const T* __restrict__ q, long q_stride, T* __restrict__ out, long out_stride,
                           const T* __restrict__ kcache, const T* __restrict__ vcache, const int* __restrict__ block_tables,
                           int max_pages, const int* __restrict__ row_seq, const int* __restrict__ positions, int T_rows, int H,
                           int G, int D, int DV, int page_size, int window, float scale, const float* __restrict__ sink,
                           const T* __restrict__ gate, long gate_stride, float out_scale, int chunk, float softcap,
                           const float* __restrict__ dist_r1, const float* __restrict__ dist_r2, int pool) {
    pdl_launch_dependents();
    pdl_wait(62);
    extern __shared__ float qs_all[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * 4 + warp;
    if (w >= (long long)T_rows * H) return;          // whole warp leaves together
    const int row = (int)(w / H), head = (int)(w % H);
    const int g = head / (H / G);
    T* op = out + (size_t)row * out_stride + (size_t)head * DV;
    const int pos = positions[row];
    if (pos < 0) {                                   // a padding row: no keys, zero output
        for (int d = lane; d < DV; d += 32) st_f(op + d, 0.f);
        return;
    }
    float* qs = qs_all + warp * D;
    const T* qp = q + (size_t)row * q_stride + (size_t)head * D;
    for (int d = lane; d < D; d += 32) qs[d] = ld_f(qp + d);
    __syncwarp();
    const int seq = row_seq[row];
    const int* bt = block_tables + (size_t)seq * max_pages;
    int first = window > 0 ? max(0, pos + 1 - window) : 0;
    if (chunk > 0) first = max(first, pos - pos % chunk);
    const float r1 = dist_r1 ? dist_r1[head] : 0.f, r2 = dist_r1 ? dist_r2[head] : 0.f;

    constexpr int VN = Vec16<T>::N;
    const bool vec = D % VN == 0;                    // a key row then starts on a 16-byte boundary
    float m = -INFINITY, l = 0.f;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;

    if (pool > 0 && window > 0) {
        // Behind the window every block of `pool` positions that lies wholly before it counts as ONE key and value, the
        // means of its keys and of its values: q . mean(k) = mean(q . k), and its weight goes to each value divided by pool.
        // Block b is seen when b * pool + pool - 1 <= pos - window. A lane scores one block; no distance bias here.
        const int nblk = pos - window + 1 >= pool ? (pos - window + 1) / pool : 0;
        const float inv_pool = 1.0f / (float)pool;
        for (int b0 = 0; b0 < nblk; b0 += 32) {
            const int b = b0 + lane;
            const bool valid = b < nblk;
            float s = -INFINITY;
            if (valid) {
                float dot = 0.f;
                for (int jj = 0; jj < pool; ++jj) {
                    const int j = b * pool + jj;
                    const T* kp = kcache + (size_t)((bt[j / page_size] * G + g) * page_size + (j % page_size)) * D;
                    if (vec) {
                        for (int d = 0; d < D; d += VN) {
                            float kv[VN];
                            Vec16<T>::load(kp + d, kv);
#pragma unroll
                            for (int i = 0; i < VN; ++i) dot = fmaf(qs[d + i], kv[i], dot);
                        }
                    } else {
                        for (int d = 0; d < D; ++d) dot = fmaf(qs[d], ld_f(kp + d), dot);
                    }
                }
                s = dot * inv_pool * scale;
                if (softcap > 0.f) s = softcap * tanhf(s / softcap);
            }
            const float m_new = fmaxf(m, warp_max(s));
            const float p = valid ? expf(s - m_new) : 0.f;
            const float alpha = expf(m - m_new);
            l = l * alpha + warp_sum(p);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] *= alpha;
            m = m_new;
            const int nb = min(32, nblk - b0);
            for (int jb = 0; jb < nb; ++jb) {
                const float pj = __shfl_sync(0xffffffffu, p, jb) * inv_pool;
                for (int jj = 0; jj < pool; ++jj) {
                    const int j = (b0 + jb) * pool + jj;
                    const T* vp = vcache + (size_t)((bt[j / page_size] * G + g) * page_size + (j % page_size)) * DV;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int d = lane + 32 * i;
                        if (d < DV) acc[i] = fmaf(pj, ld_f(vp + d), acc[i]);
                    }
                }
            }
        }
    }
    for (int c0 = first; c0 <= pos; c0 += 32) {
        const int j = c0 + lane;
        const bool valid = j <= pos;
        int slot_row = 0;                            // row of key j in the [.., D] / [.., DV] view of the layer's cache
        float s = -INFINITY;
        if (valid) {
            const int page = bt[j / page_size];
            slot_row = (page * G + g) * page_size + (j % page_size);
            const T* kp = kcache + (size_t)slot_row * D;
            float dot = 0.f;
            if (vec) {
                for (int d = 0; d < D; d += VN) {
                    float kv[VN];
                    Vec16<T>::load(kp + d, kv);
#pragma unroll
                    for (int i = 0; i < VN; ++i) dot = fmaf(qs[d + i], kv[i], dot);
                }
            } else {
                for (int d = 0; d < D; ++d) dot = fmaf(qs[d], ld_f(kp + d), dot);
            }
            s = dot * scale;
            if (softcap > 0.f) s = softcap * tanhf(s / softcap);
            if (dist_r1) s -= r1 * log1pf(r2 * (float)(pos - j));
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float alpha = expf(m - m_new);         // 0 on the first chunk (m = -inf)
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] *= alpha;
        m = m_new;
        const int nk = min(32, pos - c0 + 1);
        for (int jj = 0; jj < nk; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int sr = __shfl_sync(0xffffffffu, slot_row, jj);
            const T* vp = vcache + (size_t)sr * DV;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int d = lane + 32 * i;
                if (d < DV) acc[i] = fmaf(pj, ld_f(vp + d), acc[i]);
            }
        }
    }
    if (sink) {                                      // one more term in the denominator, no value
        const float sk = sink[head];
        const float m_new = fmaxf(m, sk);
        const float alpha = expf(m - m_new);
        l = l * alpha + expf(sk - m_new);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] *= alpha;
    }
    const float inv_l = out_scale / l;
    const T* gp = gate ? gate + (size_t)row * gate_stride + (size_t)head * DV : nullptr;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int d = lane + 32 * i;
        if (d < DV) {
            float v = acc[i] * inv_l;
            if (gp) v *= flex_sigmoid(ld_f(gp + d));
            st_f(op + d, v);
        }
    }
}

VOB_EXPORT int vob_flex_attention(const void* q, long q_stride, void* out, long out_stride, const void* kcache, const void* vcache,
                                  int code, const int* block_tables, int max_pages, const int* row_seq, const int* positions,
                                  int T_rows, int H, int G, int D, int DV, int page_size, int window, float scale,
                                  const float* sink, const void* gate, long gate_stride, float out_scale, int chunk, float softcap,
                                  const float* dist_r1, const float* dist_r2, int pool, cudaStream_t stream) {
    if (T_rows <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G != 0 || page_size <= 0 || max_pages <= 0 || D <= 0 || DV <= 0) return VOB_ERR_BAD_ARG;
    if (D > 256 || DV > 256) return VOB_ERR_UNSUPPORTED;
    if (chunk < 0 || softcap < 0.f || (dist_r1 != nullptr) != (dist_r2 != nullptr) || pool < 0 || (pool > 0 && (window <= 0 || chunk > 0)))
        return VOB_ERR_BAD_ARG;
    const long long warps = (long long)T_rows * H;
    const long long blocks = (warps + 3) / 4;
    if (blocks > 0x7fffffffLL) return VOB_ERR_UNSUPPORTED;
    const size_t smem = 4 * (size_t)D * sizeof(float);
    VOB_DISPATCH_ELEM(code, return vob_launch(flex_attention_warp_kernel<ElemT>, dim3((unsigned)blocks), dim3(128), smem, stream,
                                              (const ElemT*)q, q_stride, (ElemT*)out, out_stride, (const ElemT*)kcache,
                                              (const ElemT*)vcache, block_tables, max_pages, row_seq, positions, T_rows, H, G, D, DV,
                                              page_size, window, scale, sink, (const ElemT*)gate, gate_stride, out_scale, chunk, softcap,
                                              dist_r1, dist_r2, pool));
    return 0;
}
