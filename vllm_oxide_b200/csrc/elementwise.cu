// Memory-bound row kernels of a decoder step: embedding gather, residual add + RMSNorm,
// rotary positions + cache write, SwiGLU.
//
// Conventions: the residual stream is float32 in both engines; `act` tensors (inputs of the
// matrix products, q/k/v, the cache) are float32 or bfloat16 by an element code. All
// reductions, rotation angles and the activation are float32. One block works on one row, so a
// row's result does not depend on what else is in the batch.
#include "common.cuh"
VOB_PDL_SWITCH(elementwise)

// ---------------------------------------------------------------------------------------------
// Embedding gather: out[t, :] = table[tokens[t], :] * scale (+ pos_table[positions[t], :])   (float32 out; scale 1 leaves
// the row as it is). The learned position vector is optional; a row with a negative position (padding) gets none.
// Reference op: crates/engine/src/backend/cpu/mod.rs:172-180.
// Launch: one block per token, 256 threads. Bound: memory (2 * h * 4 bytes per token).
// A token outside [0, vocab) writes zeros and raises *err_flag (the host checks ids first); so does a position
// beyond the table.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, int h, int vocab, int* err_flag, float scale,
                             const T* __restrict__ pos_table, const int* __restrict__ positions, int max_pos) {
    pdl_launch_dependents();
    pdl_wait(1);
    int t = blockIdx.x;
    int tok = tokens[t];
    int pos = pos_table ? positions[t] : -1;
    bool ok = tok >= 0 && tok < vocab && pos < max_pos;
    if (!ok && threadIdx.x == 0 && err_flag) atomicExch(err_flag, 1);
    const T* src = table + (size_t)(ok ? tok : 0) * h;
    const T* psrc = (ok && pos >= 0) ? pos_table + (size_t)pos * h : nullptr;
    float* dst = out + (size_t)t * h;
    for (int i = threadIdx.x; i < h; i += blockDim.x) {
        float v = ok ? ld_f(src + i) * scale : 0.f;
        if (psrc) v += ld_f(psrc + i);
        dst[i] = v;
    }
}

VOB_EXPORT int vob_embed(const void* table, int table_code, const int* tokens, float* out, int T, int h,
                         int vocab, int* err_flag, float scale, const void* pos_table, const int* positions, int max_pos,
                         cudaStream_t stream) {
    if (T <= 0) return 0;
    if (h <= 0 || vocab <= 0) return VOB_ERR_BAD_ARG;
    if (pos_table && (!positions || max_pos <= 0)) return VOB_ERR_BAD_ARG;
    if (!pos_table) max_pos = 0x7fffffff;
    VOB_DISPATCH_ELEM(table_code, return vob_launch(embed_kernel<ElemT>, dim3(T), dim3(256), 0, stream, (const ElemT*)table, tokens, out, h, vocab, err_flag, scale,
                                                    (const ElemT*)pos_table, positions, max_pos));
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Embedding gather that also prepares the first norm's input in folded form (see EPI_RESID in
// gemm_sm100.cu): resid[t] = table[token]; xn[t] = bf16(resid * next_w); ssq[tile][t] = the sum of
// squares of resid over features tile*128 .. +127. One block of 128 threads per token and tile (a
// block per token that walked the tiles took one memory round trip per tile: 14 us for a width of
// 2,048); the order of every sum is fixed.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
embed_fold_kernel(const T* __restrict__ table, const int* __restrict__ tokens, float* __restrict__ resid,
                  const float* __restrict__ next_w, __nv_bfloat16* __restrict__ xn, float* __restrict__ ssq, int ld_ssq, int h,
                  int vocab, int* err_flag) {
    pdl_launch_dependents();
    pdl_wait(1);
    __shared__ float red[4];
    const int t = blockIdx.x, tile = blockIdx.y;
    const int tok = tokens[t];
    const bool ok = tok >= 0 && tok < vocab;
    if (!ok && threadIdx.x == 0 && tile == 0 && err_flag) atomicExch(err_flag, 1);
    const T* src = table + (size_t)(ok ? tok : 0) * h;
    const int f = tile * 128 + threadIdx.x;
    float v = 0.f;
    if (f < h) {
        v = ok ? ld_f(src + f) : 0.f;
        resid[(size_t)t * h + f] = v;
        xn[(size_t)t * h + f] = __float2bfloat16_rn(v * next_w[f]);
    }
    float sq = warp_sum(v * v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
    __syncthreads();
    if (threadIdx.x == 0) ssq[(size_t)tile * ld_ssq + t] = (red[0] + red[1]) + (red[2] + red[3]);
}

VOB_EXPORT int vob_embed_fold(const void* table, int table_code, const int* tokens, float* resid, const float* next_w, void* xn,
                              float* ssq, int ld_ssq, int T, int h, int vocab, int* err_flag, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (h <= 0 || vocab <= 0 || ld_ssq < T) return VOB_ERR_BAD_ARG;
    if ((h + 127) / 128 > 65535) return VOB_ERR_UNSUPPORTED;
    VOB_DISPATCH_ELEM(table_code, return vob_launch(embed_fold_kernel<ElemT>, dim3(T, (h + 127) / 128), dim3(128), 0, stream, (const ElemT*)table, tokens,
                                                    resid, next_w, (__nv_bfloat16*)xn, ssq, ld_ssq, h, vocab, err_flag));
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Residual add + RMSNorm:
//   x = resid[src] (+ delta[src] (* dscale, per feature));  if no row list: resid[src] = x  (the residual sum, float32)
//   out[r] = w * (x * 1/sqrt(mean(x^2) + eps))
// Reference ops: add (crates/engine/src/backend/cpu/mod.rs:351-358) followed by rmsnorm
// (:182-197); the weight multiplies last, as there. With a row list (`rows`, R entries) only
// those rows are normalised (gather_rows + rmsnorm, crates/engine/src/model.rs:335-342) and
// the residual is left untouched.
// Launch: one block per output row, 256 threads, h floats of shared memory; the row is read
// once. Sum of squares: per-thread strided partial sums, then a fixed tree, so a row's value is
// the same in every batch. Bound: memory.
// ---------------------------------------------------------------------------------------------
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta,
                                   const float* __restrict__ weight, const int* __restrict__ rows,
                                   TO* __restrict__ out, int h, float eps, const float* __restrict__ dscale) {
    pdl_launch_dependents();
    pdl_wait(2);
    extern __shared__ float row[];
    __shared__ float red[32];
    int r = blockIdx.x;
    int src = rows ? rows[r] : r;
    float* x = resid + (size_t)src * h;
    const TD* d = delta ? delta + (size_t)src * h : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < h; i += blockDim.x) {
        float v = x[i];
        if (d) {
            v += dscale ? ld_f(d + i) * dscale[i] : ld_f(d + i);
            if (!rows) x[i] = v;
        }
        row[i] = v;
        ss += v * v;
    }
    ss = warp_sum(ss);
    int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) red[wid] = ss;
    __syncthreads();
    if (wid == 0) {
        float v = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
        v = warp_sum(v);
        if (lane == 0) red[0] = v;
    }
    __syncthreads();
    float mean_square = red[0] / (float)h;
    float inv = 1.0f / sqrtf(mean_square + eps);
    TO* o = out + (size_t)r * h;
    for (int i = threadIdx.x; i < h; i += blockDim.x) st_f(o + i, weight[i] * (row[i] * inv));
}

// Fast path for rows whose width is a multiple of 4 and fits NV float4 per thread: every load of
// the row is issued before anything depends on one (a row of a small batch is latency-bound, not
// bandwidth-bound), the row stays in registers, and the sums take the same fixed order for every
// row. Same arithmetic as the kernel above.
template <typename TD> struct Load4;
template <> struct Load4<float> {
    __device__ static inline float4 ld(const float* p) { return *reinterpret_cast<const float4*>(p); }
};
template <> struct Load4<__nv_bfloat16> {
    __device__ static inline float4 ld(const __nv_bfloat16* p) {
        uint2 u = *reinterpret_cast<const uint2*>(p);
        float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
};
template <typename TO> struct Store4;
template <> struct Store4<float> {
    __device__ static inline void st(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Store4<__nv_bfloat16> {
    __device__ static inline void st(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&a);
        u.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = u;
    }
};

template <typename TD, typename TO, int NV>
__global__ void __launch_bounds__(256)
add_rmsnorm_vec_kernel(float* __restrict__ resid, const TD* __restrict__ delta, const float* __restrict__ weight,
                       const int* __restrict__ rows, TO* __restrict__ out, int h, float eps, const float* __restrict__ dscale) {
    pdl_launch_dependents();
    pdl_wait(2);
    __shared__ float red[32];
    int r = blockIdx.x;
    int src = rows ? rows[r] : r;
    float* x = resid + (size_t)src * h;
    const TD* d = delta ? delta + (size_t)src * h : nullptr;
    int nvec = h >> 2;
    float4 v[NV], dv[NV], w[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        int i = threadIdx.x + k * 256;
        if (i < nvec) {
            v[k] = *reinterpret_cast<const float4*>(x + 4 * i);
            dv[k] = d ? Load4<TD>::ld(d + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (d && dscale) {
                const float4 sc = *reinterpret_cast<const float4*>(dscale + 4 * i);
                dv[k].x *= sc.x; dv[k].y *= sc.y; dv[k].z *= sc.z; dv[k].w *= sc.w;
            }
            w[k] = *reinterpret_cast<const float4*>(weight + 4 * i);
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        int i = threadIdx.x + k * 256;
        if (i < nvec) {
            v[k].x += dv[k].x; v[k].y += dv[k].y; v[k].z += dv[k].z; v[k].w += dv[k].w;
            if (d && !rows) *reinterpret_cast<float4*>(x + 4 * i) = v[k];
            ss += v[k].x * v[k].x; ss += v[k].y * v[k].y; ss += v[k].z * v[k].z; ss += v[k].w * v[k].w;
        }
    }
    ss = warp_sum(ss);
    int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) red[wid] = ss;
    __syncthreads();
    if (wid == 0) {
        float t = lane < 8 ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[0] = t;
    }
    __syncthreads();
    float inv = 1.0f / sqrtf(red[0] / (float)h + eps);
    TO* o = out + (size_t)r * h;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        int i = threadIdx.x + k * 256;
        if (i < nvec)
            Store4<TO>::st(o + 4 * i, make_float4(w[k].x * (v[k].x * inv), w[k].y * (v[k].y * inv),
                                                  w[k].z * (v[k].z * inv), w[k].w * (v[k].w * inv)));
    }
}

template <typename TD, typename TO>
static int launch_add_rmsnorm(float* resid, const void* delta, const float* weight, const int* rows, void* out, int R,
                              int h, float eps, const float* dscale, cudaStream_t stream) {
    bool aligned = (h % 4 == 0) && (((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)out | (uintptr_t)dscale) % 16 == 0);
    int nv = (h / 4 + 255) / 256;
    if (aligned && nv <= 8) {
#define VEC(NV) return vob_launch(add_rmsnorm_vec_kernel<TD, TO, NV>, dim3(R), dim3(256), 0, stream, resid, (const TD*)delta, weight, rows, (TO*)out, h, eps, dscale)
        if (nv <= 1) VEC(1); else if (nv <= 2) VEC(2); else if (nv <= 4) VEC(4); else VEC(8);
#undef VEC
    }
    size_t smem = (size_t)h * sizeof(float);
    if (smem > 48 * 1024) return VOB_ERR_UNSUPPORTED;
    return vob_launch(add_rmsnorm_kernel<TD, TO>, dim3(R), dim3(256), smem, stream, resid, (const TD*)delta, weight, rows, (TO*)out, h, eps, dscale);
}

VOB_EXPORT int vob_add_rmsnorm(float* resid, const void* delta, int delta_code, const float* weight,
                               const int* rows, void* out, int out_code, int R, int h, float eps,
                               const float* dscale, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (h <= 0) return VOB_ERR_BAD_ARG;
    if (!delta) delta_code = VOB_F32;
    if (out_code == VOB_F32) {
        if (delta_code == VOB_F32) return launch_add_rmsnorm<float, float>(resid, delta, weight, rows, out, R, h, eps, dscale, stream);
        if (delta_code == VOB_BF16) return launch_add_rmsnorm<__nv_bfloat16, float>(resid, delta, weight, rows, out, R, h, eps, dscale, stream);
    } else if (out_code == VOB_BF16) {
        if (delta_code == VOB_F32) return launch_add_rmsnorm<float, __nv_bfloat16>(resid, delta, weight, rows, out, R, h, eps, dscale, stream);
        if (delta_code == VOB_BF16) return launch_add_rmsnorm<__nv_bfloat16, __nv_bfloat16>(resid, delta, weight, rows, out, R, h, eps, dscale, stream);
    }
    return VOB_ERR_BAD_ARG;
}

// ---------------------------------------------------------------------------------------------
// Rotary positions on q and k, and the cache write of k and v, in one pass over a token's
// q/k/v rows:
//   theta_i = float(pos) * inv_freq[i]         (float32 product; cosf/sinf precise versions)
//   x1' = x1*cos - x2*sin ; x2' = x2*cos + x1*sin   with x1 = x[:hd/2], x2 = x[hd/2:] per head
//   K[page, kvh, off, :] = k'[kvh],  V[page, kvh, off, :] = v[kvh],  slot = page*page_size+off
// Reference ops: rope (crates/engine/src/backend/cpu/rope.rs:64-99) on q and k, then write_kv
// (crates/engine/src/backend/cpu/mod.rs:257-285), in that order before attention
// (crates/engine/src/model.rs:307-311). q is rotated in place. A page holds
// [kv_heads][page_size][head_dim], so one (page, head) is one contiguous tile.
// `slots` may be null (rotate only); a negative slot skips that token's write.
// `inv_freq` may be null (no rotation: the part has no position encoding).
// Launch: grid (tokens, ceil((H+KV)*hd/2 / 128)), one thread per (head, pair); each thread takes
// the sine and cosine of its own angle. Bound: memory.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
rope_kv_write_kernel(T* __restrict__ q, long long q_stride, T* __restrict__ k, long long k_stride,
                     const T* __restrict__ v, long long v_stride, const int* __restrict__ positions,
                     const int* __restrict__ slots, const float* __restrict__ inv_freq, T* __restrict__ kcache,
                     T* __restrict__ vcache, int H, int KV, int hd, int page_size) {
    // one thread per (head, pair i): heads 0..H-1 are q heads, H..H+KV-1 are k heads (with their v)
    pdl_launch_dependents();
    pdl_wait(4);
    int t = blockIdx.x;
    int half = hd >> 1;
    int e = blockIdx.y * blockDim.x + threadIdx.x;
    int nheads = H + (k ? KV : 0);
    if (e >= nheads * half) return;
    int head = e / half, i = e - head * half;
    float c = 1.f, s = 0.f;
    if (inv_freq) {
        float theta = (float)positions[t] * inv_freq[i];
        c = cosf(theta);
        s = sinf(theta);
    }
    if (head < H) {
        T* x = q + (size_t)t * q_stride + (size_t)head * hd;
        if (inv_freq) {
            float a = ld_f(x + i), b = ld_f(x + half + i);
            st_f(x + i, a * c - b * s);
            st_f(x + half + i, b * c + a * s);
        }
        return;
    }
    int kh = head - H;
    T* x = k + (size_t)t * k_stride + (size_t)kh * hd;
    float a = ld_f(x + i), b = ld_f(x + half + i);
    float ra = a, rb = b;
    if (inv_freq) {
        ra = a * c - b * s;
        rb = b * c + a * s;
        st_f(x + i, ra);
        st_f(x + half + i, rb);
    }
    int slot = slots ? slots[t] : -1;
    if (slot >= 0) {
        size_t page = (size_t)(slot / page_size);
        int off = slot % page_size;
        size_t base = ((page * KV + kh) * page_size + off) * (size_t)hd;
        const T* vr = v + (size_t)t * v_stride + (size_t)kh * hd;
        st_f(kcache + base + i, ra);
        st_f(kcache + base + half + i, rb);
        vcache[base + i] = vr[i];
        vcache[base + half + i] = vr[half + i];
    }
}

// The same for many tokens: one block per token, thread (pair i, head group): the sine and cosine
// of the pair's angle are taken once and reused for every head the thread walks over, instead
// of once per (head, pair).
template <typename T>
__global__ void __launch_bounds__(128)
rope_kv_write_token_kernel(T* __restrict__ q, long long q_stride, T* __restrict__ k, long long k_stride,
                           const T* __restrict__ v, long long v_stride, const int* __restrict__ positions,
                           const int* __restrict__ slots, const float* __restrict__ inv_freq, T* __restrict__ kcache,
                           T* __restrict__ vcache, int H, int KV, int hd, int page_size) {
    pdl_launch_dependents();
    pdl_wait(4);
    const int t = blockIdx.x;
    const int half = hd >> 1;
    const int groups = blockDim.x / half;          // head groups that work side by side
    const int i = threadIdx.x % half, hg = threadIdx.x / half;
    if (hg >= groups) return;
    float c = 1.f, s = 0.f;
    if (inv_freq) {
        float theta = (float)positions[t] * inv_freq[i];
        c = cosf(theta);
        s = sinf(theta);
    }
    if (inv_freq) {
        T* qr = q + (size_t)t * q_stride;
        for (int head = hg; head < H; head += groups) {
            T* x = qr + (size_t)head * hd;
            float a = ld_f(x + i), b = ld_f(x + half + i);
            st_f(x + i, a * c - b * s);
            st_f(x + half + i, b * c + a * s);
        }
    }
    if (!k) return;
    const int slot = slots ? slots[t] : -1;
    const size_t page = slot >= 0 ? (size_t)(slot / page_size) : 0;
    const int off = slot >= 0 ? slot % page_size : 0;
    for (int kh = hg; kh < KV; kh += groups) {
        T* x = k + (size_t)t * k_stride + (size_t)kh * hd;
        float a = ld_f(x + i), b = ld_f(x + half + i);
        float ra = a, rb = b;
        if (inv_freq) {
            ra = a * c - b * s;
            rb = b * c + a * s;
            st_f(x + i, ra);
            st_f(x + half + i, rb);
        }
        if (slot >= 0) {
            size_t base = ((page * KV + kh) * page_size + off) * (size_t)hd;
            const T* vr = v + (size_t)t * v_stride + (size_t)kh * hd;
            st_f(kcache + base + i, ra);
            st_f(kcache + base + half + i, rb);
            vcache[base + i] = vr[i];
            vcache[base + half + i] = vr[half + i];
        }
    }
}

// The same with 16-byte accesses, ROPE_TOK tokens per block: every thread takes 16-byte pieces of
// heads: it first requests all of its pieces (the first half of a head, the half that pairs with it
// and, for a k head, the pieces of v that go to the cache with it), so that a block has its whole
// traffic in flight at once; while they are on their way the tokens' sines and cosines go to shared
// memory once; then the pieces are rotated and stored. Needs 16-byte aligned rows.
constexpr int ROPE_TOK = 4;
constexpr int ROPE_THREADS = 256;
constexpr int ROPE_MAX_UNITS = 4;                  // pieces per thread handled in one go

template <typename T>
__global__ void __launch_bounds__(ROPE_THREADS)
rope_kv_write_token_vec_kernel(T* __restrict__ q, long long q_stride, T* __restrict__ k, long long k_stride,
                               const T* __restrict__ v, long long v_stride, const int* __restrict__ positions,
                               const int* __restrict__ slots, const float* __restrict__ inv_freq, T* __restrict__ kcache,
                               T* __restrict__ vcache, int T_, int H, int KV, int hd, int page_size) {
    constexpr int E = 16 / sizeof(T);              // elements per 16 bytes
    pdl_launch_dependents();
    pdl_wait(4);
    extern __shared__ float s_cs[];                // [ROPE_TOK][half] cosines, then as many sines
    const int t0 = blockIdx.x * ROPE_TOK;
    const int ntok = min(ROPE_TOK, T_ - t0);
    const int half = hd >> 1;
    float* sc = s_cs;
    float* ss = s_cs + ROPE_TOK * half;
    const int chunks = half / E;                   // 16-byte pieces per half head
    const int heads = H + (k ? KV : 0);            // q heads, then k heads
    const int per_tok = heads * chunks;
    const int total = ntok * per_tok;
    uint4 ua[ROPE_MAX_UNITS], ub[ROPE_MAX_UNITS], va[ROPE_MAX_UNITS], vb[ROPE_MAX_UNITS];
    T* pa[ROPE_MAX_UNITS];
    long long cb[ROPE_MAX_UNITS];                  // where in the cache a piece of a k head (and of its v) goes; -1: nowhere
    // every piece a thread handles in one round is requested before anything is computed
    auto load_round = [&](int base) {
#pragma unroll
        for (int j = 0; j < ROPE_MAX_UNITS; ++j) {
            const int u = base + j * ROPE_THREADS + threadIdx.x;
            pa[j] = nullptr;
            cb[j] = -1;
            if (u < total) {
                const int tt = u / per_tok, r = u - tt * per_tok, head = r / chunks, ch = r - head * chunks;
                pa[j] = head < H ? q + (size_t)(t0 + tt) * q_stride + (size_t)head * hd + ch * E
                                 : k + (size_t)(t0 + tt) * k_stride + (size_t)(head - H) * hd + ch * E;
                ua[j] = *reinterpret_cast<const uint4*>(pa[j]);
                ub[j] = *reinterpret_cast<const uint4*>(pa[j] + half);
                if (head >= H) {
                    const int kh = head - H;
                    const int slot = slots ? slots[t0 + tt] : -1;
                    if (slot >= 0) {
                        cb[j] = (long long)(((((size_t)(slot / page_size)) * KV + kh) * page_size + slot % page_size) * (size_t)hd) + ch * E;
                        const T* vr = v + (size_t)(t0 + tt) * v_stride + (size_t)kh * hd + ch * E;
                        va[j] = *reinterpret_cast<const uint4*>(vr);
                        vb[j] = *reinterpret_cast<const uint4*>(vr + half);
                    }
                }
            }
        }
    };
    auto finish_round = [&](int base) {
#pragma unroll
        for (int j = 0; j < ROPE_MAX_UNITS; ++j) {
            const int u = base + j * ROPE_THREADS + threadIdx.x;
            if (u >= total) continue;
            const int tt = u / per_tok, r = u - tt * per_tok, head = r / chunks, ch = r - head * chunks;
            uint4 ra = ua[j], rb = ub[j];
            if (inv_freq) {
                const T* a = reinterpret_cast<const T*>(&ua[j]);
                const T* b = reinterpret_cast<const T*>(&ub[j]);
                T* oa = reinterpret_cast<T*>(&ra);
                T* ob = reinterpret_cast<T*>(&rb);
                const float* c = sc + tt * half + ch * E;
                const float* sn = ss + tt * half + ch * E;
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    const float x = ld_f(a + e), y = ld_f(b + e);
                    st_f(oa + e, x * c[e] - y * sn[e]);
                    st_f(ob + e, y * c[e] + x * sn[e]);
                }
                *reinterpret_cast<uint4*>(pa[j]) = ra;
                *reinterpret_cast<uint4*>(pa[j] + half) = rb;
            }
            if (cb[j] >= 0) {
                *reinterpret_cast<uint4*>(kcache + cb[j]) = ra;
                *reinterpret_cast<uint4*>(kcache + cb[j] + half) = rb;
                *reinterpret_cast<uint4*>(vcache + cb[j]) = va[j];
                *reinterpret_cast<uint4*>(vcache + cb[j] + half) = vb[j];
            }
        }
    };
    load_round(0);
    // the tokens' cosines and sines, while the first round's pieces are on their way
    for (int u = threadIdx.x; u < ntok * half; u += ROPE_THREADS) {
        const int tt = u / half, i = u - tt * half;
        float c = 1.f, s = 0.f;
        if (inv_freq) {
            float theta = (float)positions[t0 + tt] * inv_freq[i];
            c = cosf(theta);
            s = sinf(theta);
        }
        sc[u] = c;
        ss[u] = s;
    }
    __syncthreads();
    finish_round(0);
    for (int base = ROPE_THREADS * ROPE_MAX_UNITS; base < total; base += ROPE_THREADS * ROPE_MAX_UNITS) {
        load_round(base);
        finish_round(base);
    }
}

VOB_EXPORT int vob_rope_kv_write(void* q, long long q_stride, void* k, long long k_stride, const void* v,
                                 long long v_stride, const int* positions, const int* slots,
                                 const float* inv_freq, void* kcache, void* vcache, int code, int T, int H,
                                 int KV, int hd, int page_size, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hd <= 0 || (hd & 1) || H <= 0 || KV < 0 || page_size <= 0) return VOB_ERR_BAD_ARG;
    if (k && slots && (!kcache || !vcache || !v)) return VOB_ERR_BAD_ARG;
    const int esz = code == VOB_BF16 ? 2 : 4;
    auto aligned = [&](const void* p, long long stride) { return !p || (((uintptr_t)p & 15) == 0 && (stride * esz) % 16 == 0); };
    if (T >= 64 && (hd / 2) % (16 / esz) == 0 && aligned(q, q_stride) && aligned(k, k_stride) && aligned(v, v_stride) &&
        aligned(kcache, hd) && aligned(vcache, hd)) {
        // many tokens, 16-byte aligned rows: sines and cosines once per token, 16-byte accesses
        VOB_DISPATCH_ELEM(code, return vob_launch(rope_kv_write_token_vec_kernel<ElemT>, dim3((T + ROPE_TOK - 1) / ROPE_TOK),
            dim3(ROPE_THREADS), (size_t)ROPE_TOK * hd * sizeof(float), stream, (ElemT*)q, q_stride, (ElemT*)k, k_stride,
            (const ElemT*)v, v_stride, positions, slots, inv_freq, (ElemT*)kcache, (ElemT*)vcache, T, H, KV, hd, page_size));
    }
    if (T >= 64 && hd / 2 <= 128) {
        // many tokens: a block per token, sines and cosines shared across heads
        VOB_DISPATCH_ELEM(code, return vob_launch(rope_kv_write_token_kernel<ElemT>, dim3(T), dim3(128), 0, stream,
            (ElemT*)q, q_stride, (ElemT*)k, k_stride, (const ElemT*)v, v_stride, positions, slots, inv_freq,
            (ElemT*)kcache, (ElemT*)vcache, H, KV, hd, page_size));
    }
    int pairs = (H + (k ? KV : 0)) * (hd / 2);
    dim3 grid(T, (pairs + 127) / 128);
    if (grid.y > 65535) return VOB_ERR_UNSUPPORTED;
    VOB_DISPATCH_ELEM(code, return vob_launch(rope_kv_write_kernel<ElemT>, grid, dim3(128), 0, stream,
        (ElemT*)q, q_stride, (ElemT*)k, k_stride, (const ElemT*)v, v_stride, positions, slots, inv_freq,
        (ElemT*)kcache, (ElemT*)vcache, H, KV, hd, page_size));
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Gated activation: out[t, j] = act(gate) * up, gate = in[t, j], up = in[t, I + j].
// ACT 0, SwiGLU: gate / (1 + exp(-gate)) * up
// (divide, then multiply by up, as crates/engine/src/backend/cpu/mod.rs:341-349).
// ACT 1, the tanh form of gelu: 0.5 gate (1 + tanh(sqrt(2/pi) (gate + 0.044715 gate^3))) * up. The input is
// the output of one fused [gate; up] matrix product, row stride `in_stride` elements.
// Launch: grid (T, ceil(I/256)). Bound: memory.
// ---------------------------------------------------------------------------------------------
template <int ACT> __device__ __forceinline__ float glu_act(float g) {
    if (ACT == 1) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    return g / (1.0f + expf(-g));
}

template <typename T, int ACT>
__global__ void swiglu_kernel(const T* __restrict__ in, long long in_stride, T* __restrict__ out, int I) {
    pdl_launch_dependents();
    pdl_wait(5);
    int j = blockIdx.y * blockDim.x + threadIdx.x;
    if (j >= I) return;
    const T* r = in + (size_t)blockIdx.x * in_stride;
    float g = ld_f(r + j), u = ld_f(r + I + j);
    st_f(out + (size_t)blockIdx.x * I + j, glu_act<ACT>(g) * u);
}

// 16 bytes per load: 8 bfloat16 or 4 float per thread (I a multiple of that, rows 16-byte aligned).
template <typename T, int N, int ACT>
__global__ void swiglu_vec_kernel(const T* __restrict__ in, long long in_stride, T* __restrict__ out, int I) {
    pdl_launch_dependents();
    pdl_wait(5);
    int j = (blockIdx.y * blockDim.x + threadIdx.x) * N;
    if (j >= I) return;
    const T* r = in + (size_t)blockIdx.x * in_stride;
    uint4 gu = *reinterpret_cast<const uint4*>(r + j);
    uint4 uu = *reinterpret_cast<const uint4*>(r + I + j);
    const T* g = reinterpret_cast<const T*>(&gu);
    const T* u = reinterpret_cast<const T*>(&uu);
    uint4 ov;
    T* o = reinterpret_cast<T*>(&ov);
#pragma unroll
    for (int e = 0; e < N; ++e) {
        float gf = ld_f(g + e), uf = ld_f(u + e);
        st_f(o + e, glu_act<ACT>(gf) * uf);
    }
    *reinterpret_cast<uint4*>(out + (size_t)blockIdx.x * I + j) = ov;
}

template <typename T, int ACT>
static int launch_swiglu(const void* in, long long in_stride, void* out, int T_rows, int I, cudaStream_t stream) {
    constexpr int N = 16 / sizeof(T);
    bool vec = (I % N == 0) && (in_stride % N == 0) && (((uintptr_t)in | (uintptr_t)out) % 16 == 0);
    if (vec) {
        int per = 256 * N;
        if ((I + per - 1) / per > 65535) return VOB_ERR_UNSUPPORTED;
        dim3 grid(T_rows, (I + per - 1) / per);
        return vob_launch(swiglu_vec_kernel<T, N, ACT>, grid, dim3(256), 0, stream, (const T*)in, in_stride, (T*)out, I);
    } else {
        if ((I + 255) / 256 > 65535) return VOB_ERR_UNSUPPORTED;
        dim3 grid(T_rows, (I + 255) / 256);
        return vob_launch(swiglu_kernel<T, ACT>, grid, dim3(256), 0, stream, (const T*)in, in_stride, (T*)out, I);
    }
}

VOB_EXPORT int vob_swiglu(const void* in, long long in_stride, void* out, int code, int T, int I,
                          cudaStream_t stream) {
    if (T <= 0) return 0;
    if (I <= 0) return VOB_ERR_BAD_ARG;
    if (code == VOB_F32) return launch_swiglu<float, 0>(in, in_stride, out, T, I, stream);
    if (code == VOB_BF16) return launch_swiglu<__nv_bfloat16, 0>(in, in_stride, out, T, I, stream);
    return VOB_ERR_BAD_ARG;
}

// The same with the activation chosen by `act` (0 silu, 1 the tanh form of gelu).
VOB_EXPORT int vob_glu(const void* in, long long in_stride, void* out, int code, int T, int I, int act,
                       cudaStream_t stream) {
    if (T <= 0) return 0;
    if (I <= 0 || (act != 0 && act != 1)) return VOB_ERR_BAD_ARG;
    if (act == 0) return vob_swiglu(in, in_stride, out, code, T, I, stream);
    if (code == VOB_F32) return launch_swiglu<float, 1>(in, in_stride, out, T, I, stream);
    if (code == VOB_BF16) return launch_swiglu<__nv_bfloat16, 1>(in, in_stride, out, T, I, stream);
    return VOB_ERR_BAD_ARG;
}

// ---------------------------------------------------------------------------------------------
// The clamped gate of a feed-forward: g = min(gate, limit), u = clamp(up, -limit, limit), out = g * sigmoid(1.702 g) * (u + 1).
// in [T, >= 2 I] (gate columns, then up columns, rows `in_stride` apart), out [T, I]. Grid (T, ceil(I / 256)).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
glu_clamped_kernel(const T* __restrict__ in, long long in_stride, T* __restrict__ out, int I, float limit) {
    pdl_launch_dependents();
    pdl_wait(5);
    const int j = blockIdx.y * 256 + threadIdx.x;
    if (j >= I) return;
    const T* r = in + (size_t)blockIdx.x * in_stride;
    const float g = fminf(ld_f(r + j), limit), u = fminf(fmaxf(ld_f(r + I + j), -limit), limit);
    st_f(out + (size_t)blockIdx.x * I + j, g / (1.0f + expf(-1.702f * g)) * (u + 1.0f));
}

VOB_EXPORT int vob_glu_clamped(const void* in, long long in_stride, void* out, int code, int T, int I, float limit, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (I <= 0 || !(limit > 0.f) || (I + 255) / 256 > 65535) return VOB_ERR_BAD_ARG;
    VOB_DISPATCH_ELEM(code, return vob_launch(glu_clamped_kernel<ElemT>, dim3(T, (I + 255) / 256), dim3(256), 0, stream, (const ElemT*)in,
                                              in_stride, (ElemT*)out, I, limit));
    return 0;
}

// ---------------------------------------------------------------------------------------------
// A stream that is a learned weighted sum over depth. `stack` float32 [T, slots, h] keeps the embedding's output (slot 0)
// and every layer's result so far; `x` float32 [T, h] holds the newest result:
//   stack[t, n] = x[t];   x[t] = sum over j = 0 .. n of w[j] * stack[t, j]      (j in order, float32)
// With `first` the kernel only files x as slot 0 (n = 0, x unchanged). Launch: grid (T, ceil(h / 256)).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
depth_average_kernel(float* __restrict__ stack, float* __restrict__ x, const float* __restrict__ w, int slots, int h, int n, int first) {
    pdl_launch_dependents();
    pdl_wait(7);
    const int t = blockIdx.x, c = blockIdx.y * 256 + threadIdx.x;
    if (c >= h) return;
    float* base = stack + (size_t)t * slots * h + c;
    const float cur = x[(size_t)t * h + c];
    base[(size_t)n * h] = cur;
    if (first) return;
    float acc = 0.f;
    for (int j = 0; j < n; ++j) acc = fmaf(w[j], base[(size_t)j * h], acc);
    x[(size_t)t * h + c] = fmaf(w[n], cur, acc);
}

VOB_EXPORT int vob_depth_average(float* stack, float* x, const float* w, int T, int slots, int h, int n, int first, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (h <= 0 || slots <= 0 || n < 0 || n >= slots || (!first && !w) || (h + 255) / 256 > 65535) return VOB_ERR_BAD_ARG;
    return vob_launch(depth_average_kernel, dim3(T, (h + 255) / 256), dim3(256), 0, stream, stack, x, w, slots, h, n, first);
}

// ---------------------------------------------------------------------------------------------
// Layer norm with weight and bias (`bias` null: none), LN(z) = (z - mean) / sqrt(mean((z - mean)^2) + eps) * w + b, in two arrangements:
//   delta given:  y = LN(delta[r]);  resid[r] += y  (the residual takes the NORMED result of a sub-layer, float32);
//                 copy[r] = resid[r] in the activations' type, if `copy` is given (what the next sub-layer reads)
//   delta null:   out[r] = LN(resid[rows ? rows[r] : r])   (the model's last norm on the wanted rows)
// Launch: one block of 256 threads per row, h floats of shared memory; the mean first, then the mean of the squared
// deviations from it, each a strided partial sum per thread and a fixed tree, so a row's value is the same in every batch.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float block_sum_256(float v, float* red) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    __syncthreads();                       // red may still be read from the call before
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += red[i];
    return t;
}

template <typename T> __device__ __forceinline__ void ld4_f(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void ld4_f<float>(const float* p, float (&v)[4]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
template <> __device__ __forceinline__ void ld4_f<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 a = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&a.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&a.y);
    v[0] = __bfloat162float(lo.x); v[1] = __bfloat162float(lo.y); v[2] = __bfloat162float(hi.x); v[3] = __bfloat162float(hi.y);
}
template <typename T> __device__ __forceinline__ void st4_f(T* p, const float (&v)[4]);
template <> __device__ __forceinline__ void st4_f<float>(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void st4_f<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
    uint2 a;
    a.x = *reinterpret_cast<const unsigned*>(&lo);
    a.y = *reinterpret_cast<const unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = a;
}

// What the kernel can do on its way behind resid[r] += LN(delta[r]) (a kernel parameter: what is not asked for costs nothing):
//   * the stream as a weighted sum over depth (see depth_average_kernel, the same sums in the same order): the new row is
//     filed as entry `depth_n` of `stack` [T, depth_slots, h] and replaced by sum_j depth_w[j] * entry j, j = 0 .. depth_n;
//   * the last taps - 1 inputs of a short convolution that ran in front of the sub-layer (`conv_x` [T, h], what the
//     convolution read, in delta's type): the block of a request's last row of the step leaves them in the request's state
//     slot, new[m] = x_(n - (taps - 1) + m) if that row is of this step, else old[m + n] (m ascending, in place). Every
//     kernel that read the old state has completed by now.
struct NormTail {
    float* stack;
    const float* depth_w;
    int depth_slots, depth_n;
    const void* conv_x;
    float* conv_state;
    int taps;
    const int* row_seq;
    const int* seq_starts;
    const int* state_slots;
    const int* positions;
};

// BY4: the row's length is a multiple of 4 and every row starts where four features can be read at once; a thread
// then takes four neighbouring features a turn (its partial sums run over them in order).
template <typename TD, typename TO, bool BY4>
__global__ void __launch_bounds__(256)
layernorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta, const float* __restrict__ weight,
                 const float* __restrict__ bias, const int* __restrict__ rows, TO* __restrict__ out, int h, float eps, NormTail tail) {
    pdl_launch_dependents();
    pdl_wait(5);
    extern __shared__ __align__(16) float row[];
    __shared__ float red[8];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* x = resid + (size_t)src * h;
    const TD* d = delta ? delta + (size_t)r * h : nullptr;
    float s = 0.f;
    if (BY4) {
        for (int i = threadIdx.x * 4; i < h; i += 1024) {
            float v[4];
            if (d) ld4_f<TD>(d + i, v); else ld4_f<float>(x + i, v);
            st4_f<float>(row + i, v);
            s += v[0]; s += v[1]; s += v[2]; s += v[3];
        }
    } else {
        for (int i = threadIdx.x; i < h; i += blockDim.x) {
            const float v = d ? ld_f(d + i) : x[i];
            row[i] = v;
            s += v;
        }
    }
    const float mean = block_sum_256(s, red) / (float)h;
    float ss = 0.f;
    if (BY4) {
        for (int i = threadIdx.x * 4; i < h; i += 1024) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float c = row[i + k] - mean;
                ss = fmaf(c, c, ss);
            }
        }
    } else {
        for (int i = threadIdx.x; i < h; i += blockDim.x) {
            const float c = row[i] - mean;
            ss = fmaf(c, c, ss);
        }
    }
    const float inv = 1.0f / sqrtf(block_sum_256(ss, red) / (float)h + eps);
    TO* o = out ? out + (size_t)r * h : nullptr;
    if (BY4) {
        for (int i = threadIdx.x * 4; i < h; i += 1024) {
            const float4 w4 = *reinterpret_cast<const float4*>(weight + i);
            const float4 r4 = *reinterpret_cast<const float4*>(row + i);
            float4 y = make_float4((r4.x - mean) * inv * w4.x, (r4.y - mean) * inv * w4.y, (r4.z - mean) * inv * w4.z,
                                   (r4.w - mean) * inv * w4.w);
            if (bias) {
                const float4 b4 = *reinterpret_cast<const float4*>(bias + i);
                y.x += b4.x; y.y += b4.y; y.z += b4.z; y.w += b4.w;
            }
            if (d) {
                const float4 x4 = *reinterpret_cast<const float4*>(x + i);
                y.x += x4.x; y.y += x4.y; y.z += x4.z; y.w += x4.w;
                *reinterpret_cast<float4*>(x + i) = y;
            }
            if (o) {
                const float yv[4] = {y.x, y.y, y.z, y.w};
                st4_f<TO>(o + i, yv);
            }
        }
    } else {
        for (int i = threadIdx.x; i < h; i += blockDim.x) {
            float y = (row[i] - mean) * inv * weight[i] + (bias ? bias[i] : 0.f);
            if (d) {
                y += x[i];
                x[i] = y;
            }
            if (o) st_f(o + i, y);
        }
    }
    if (tail.stack) {
        __syncthreads();       // the row's new values, whoever wrote them
        float* base = tail.stack + (size_t)r * tail.depth_slots * h;
        const int dn = tail.depth_n;
        if (BY4) {
            for (int i = threadIdx.x * 4; i < h; i += 1024) {
                const float4 cur = *reinterpret_cast<const float4*>(x + i);
                *reinterpret_cast<float4*>(base + (size_t)dn * h + i) = cur;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
                for (int j = 0; j < dn; ++j) {
                    const float wj = tail.depth_w[j];
                    const float4 e = *reinterpret_cast<const float4*>(base + (size_t)j * h + i);
                    acc.x = fmaf(wj, e.x, acc.x); acc.y = fmaf(wj, e.y, acc.y); acc.z = fmaf(wj, e.z, acc.z); acc.w = fmaf(wj, e.w, acc.w);
                }
                const float wn = tail.depth_w[dn];
                *reinterpret_cast<float4*>(x + i) = make_float4(fmaf(wn, cur.x, acc.x), fmaf(wn, cur.y, acc.y), fmaf(wn, cur.z, acc.z),
                                                                fmaf(wn, cur.w, acc.w));
            }
        } else {
            for (int i = threadIdx.x; i < h; i += blockDim.x) {
                const float cur = x[i];
                base[(size_t)dn * h + i] = cur;
                float acc = 0.f;
                for (int j = 0; j < dn; ++j) acc = fmaf(tail.depth_w[j], base[(size_t)j * h + i], acc);
                x[i] = fmaf(tail.depth_w[dn], cur, acc);
            }
        }
    }
    if (tail.conv_state && tail.positions[r] >= 0) {
        const int s = tail.row_seq[r];
        const int r0 = tail.seq_starts[s], r1 = tail.seq_starts[s + 1];
        if (r == r1 - 1) {
            // a thread owns whole columns of the state: it reads a column's new entries (independent loads), then writes them
            const int n = r1 - r0, keep = tail.taps - 1;
            const TD* cx = reinterpret_cast<const TD*>(tail.conv_x);
            float* st = tail.conv_state + (size_t)tail.state_slots[s] * keep * h;
            if (keep <= 8) {
#pragma unroll 2
                for (int c = threadIdx.x; c < h; c += blockDim.x) {
                    float v[8];
#pragma unroll
                    for (int m = 0; m < 8; ++m) {
                        const int tau = n - keep + m;
                        if (m < keep) v[m] = tau >= 0 ? ld_f(cx + (size_t)(r0 + tau) * h + c) : st[(size_t)(m + n) * h + c];
                    }
#pragma unroll
                    for (int m = 0; m < 8; ++m)
                        if (m < keep) st[(size_t)m * h + c] = v[m];
                }
            } else {
                for (int c = threadIdx.x; c < h; c += blockDim.x)
                    for (int m = 0; m < keep; ++m) {
                        const int tau = n - keep + m;
                        st[(size_t)m * h + c] = tau >= 0 ? ld_f(cx + (size_t)(r0 + tau) * h + c) : st[(size_t)(m + n) * h + c];
                    }
            }
        }
    }
}

static int layernorm_launch(float* resid, const void* delta, int delta_code, const float* weight, const float* bias,
                            const int* rows, void* out, int out_code, int R, int h, float eps, NormTail tail, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (h <= 0 || !weight || (delta && rows) || (!delta && !out)) return VOB_ERR_BAD_ARG;
    const size_t smem = (size_t)h * sizeof(float);
    if (smem > 48 * 1024) return VOB_ERR_UNSUPPORTED;
    if (!delta) delta_code = VOB_F32;
    if (!out) out_code = VOB_F32;
    const bool by4 = h % 4 == 0 && ((((uintptr_t)resid) | ((uintptr_t)weight) | ((uintptr_t)bias)) & 15) == 0 && (((uintptr_t)delta) & 15) == 0 &&
                     (((uintptr_t)out) & 15) == 0 && (((uintptr_t)tail.stack) & 15) == 0;
#define VOB_LN(TD_, TO_)                                                                                                             \
    return by4 ? vob_launch(layernorm_kernel<TD_, TO_, true>, dim3(R), dim3(256), smem, stream, resid, (const TD_*)delta, weight, bias, rows, \
                            (TO_*)out, h, eps, tail)                                                                                 \
               : vob_launch(layernorm_kernel<TD_, TO_, false>, dim3(R), dim3(256), smem, stream, resid, (const TD_*)delta, weight, bias, rows, \
                            (TO_*)out, h, eps, tail)
    if (delta_code == VOB_F32 && out_code == VOB_F32) VOB_LN(float, float);
    if (delta_code == VOB_BF16 && out_code == VOB_BF16) VOB_LN(__nv_bfloat16, __nv_bfloat16);
    if (delta_code == VOB_F32 && out_code == VOB_BF16) VOB_LN(float, __nv_bfloat16);
    if (delta_code == VOB_BF16 && out_code == VOB_F32) VOB_LN(__nv_bfloat16, float);
#undef VOB_LN
    return VOB_ERR_BAD_ARG;
}

VOB_EXPORT int vob_layernorm(float* resid, const void* delta, int delta_code, const float* weight, const float* bias,
                             const int* rows, void* out, int out_code, int R, int h, float eps, cudaStream_t stream) {
    return layernorm_launch(resid, delta, delta_code, weight, bias, rows, out, out_code, R, h, eps, NormTail{}, stream);
}

// resid[r] += LN(delta[r]) with what `NormTail` describes done on the way: the weighted sum over depth (stack non-null:
// depth_w float32 [depth_n + 1], 0 < depth_n < depth_slots) and / or a convolution's state moved on (conv_state non-null:
// float32 [slots, taps - 1, h]; conv_x [R, h] in delta's type; row_seq, positions int32 [R], seq_starts, state_slots per request).
VOB_EXPORT int vob_layernorm_tail(float* resid, const void* delta, int delta_code, const float* weight, const float* bias, int R, int h,
                                  float eps, float* stack, const float* depth_w, int depth_slots, int depth_n, const void* conv_x,
                                  float* conv_state, int taps, const int* row_seq, const int* seq_starts, const int* state_slots,
                                  const int* positions, cudaStream_t stream) {
    if (!delta) return VOB_ERR_BAD_ARG;
    if (stack && (!depth_w || depth_n <= 0 || depth_n >= depth_slots)) return VOB_ERR_BAD_ARG;
    if (conv_state && (!conv_x || taps < 2 || !row_seq || !seq_starts || !state_slots || !positions)) return VOB_ERR_BAD_ARG;
    const NormTail tail{stack, depth_w, depth_slots, depth_n, conv_x, conv_state, taps, row_seq, seq_starts, state_slots, positions};
    return layernorm_launch(resid, delta, delta_code, weight, bias, nullptr, nullptr, 0, R, h, eps, tail, stream);
}

// ---------------------------------------------------------------------------------------------
// The float32 residual in the activations' type: out[i] = in[i] (rounded to nearest even for bfloat16). What a
// sub-layer that reads the residual itself is given where nothing before it has left such a copy.
// ---------------------------------------------------------------------------------------------
template <typename TO>
__global__ void __launch_bounds__(256) cast_rows_kernel(const float* __restrict__ in, TO* __restrict__ out, long long n) {
    pdl_launch_dependents();
    pdl_wait(6);
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i < n) st_f(out + i, in[i]);
}

VOB_EXPORT int vob_cast_rows(const float* in, void* out, int out_code, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const long long blocks = (n + 255) / 256;
    if (blocks > 0x7fffffffLL) return VOB_ERR_UNSUPPORTED;
    VOB_DISPATCH_ELEM(out_code, return vob_launch(cast_rows_kernel<ElemT>, dim3((unsigned)blocks), dim3(256), 0, stream, in, (ElemT*)out, n));
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Activations of a feed-forward that is not gated, element by element, float32 arithmetic:
//   act 0, xIELU with two numbers ap = params[0] > 0 and an = params[1]:
//       z > 0:  ap z^2 + z / 2;      z <= 0:  an (exp(z) - 1 - z) + z / 2
// in [T, I] with a row stride, out [T, I] contiguous (may be `in` itself when that is contiguous).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float xielu_f(float z, float ap, float an) {
    return z > 0.f ? fmaf(ap * z, z, 0.5f * z) : fmaf(an, expm1f(z) - z, 0.5f * z);
}

template <typename T>
__global__ void __launch_bounds__(256)
act_kernel(const T* __restrict__ in, long long in_stride, T* __restrict__ out, int I, int act, const float* __restrict__ params) {
    pdl_launch_dependents();
    pdl_wait(7);
    const int t = blockIdx.x;
    const int j = blockIdx.y * 256 + threadIdx.x;
    if (j >= I) return;
    const float ap = params[0], an = params[1];
    const float z = ld_f(in + (size_t)t * in_stride + j);
    st_f(out + (size_t)t * I + j, xielu_f(z, ap, an));
}

// Rows whose length and addresses allow 16-byte accesses: a thread takes 16 bytes of a row a turn.
template <typename T>
__global__ void __launch_bounds__(256)
act_vec_kernel(const T* __restrict__ in, long long in_stride, T* __restrict__ out, int I, int act, const float* __restrict__ params) {
    pdl_launch_dependents();
    pdl_wait(7);
    constexpr int PER = 16 / sizeof(T);
    const int t = blockIdx.x;
    const int j = (blockIdx.y * 256 + threadIdx.x) * PER;
    if (j >= I) return;
    const float ap = params[0], an = params[1];
    const T* src = in + (size_t)t * in_stride + j;
    T* dst = out + (size_t)t * I + j;
#pragma unroll
    for (int k = 0; k < PER; k += 4) {
        float v[4];
        ld4_f<T>(src + k, v);
#pragma unroll
        for (int m = 0; m < 4; ++m) v[m] = xielu_f(v[m], ap, an);
        st4_f<T>(dst + k, v);
    }
}

VOB_EXPORT int vob_act(const void* in, long long in_stride, void* out, int code, int T, int I, int act, const float* params,
                       cudaStream_t stream) {
    if (T <= 0) return 0;
    if (I <= 0 || act != 0 || !params) return VOB_ERR_BAD_ARG;
    const int per = code == VOB_BF16 ? 8 : 4;
    if (I % per == 0 && in_stride % per == 0 && ((((uintptr_t)in) | ((uintptr_t)out)) & 15) == 0) {
        const int by = (I / per + 255) / 256;
        if (by > 65535) return VOB_ERR_UNSUPPORTED;
        VOB_DISPATCH_ELEM(code, return vob_launch(act_vec_kernel<ElemT>, dim3(T, by), dim3(256), 0, stream, (const ElemT*)in, in_stride,
                                                  (ElemT*)out, I, act, params));
        return 0;
    }
    if ((I + 255) / 256 > 65535) return VOB_ERR_UNSUPPORTED;
    VOB_DISPATCH_ELEM(code, return vob_launch(act_kernel<ElemT>, dim3(T, (I + 255) / 256), dim3(256), 0, stream, (const ElemT*)in, in_stride,
                                              (ElemT*)out, I, act, params));
    return 0;
}
