// Attention over a latent cache: per token the pages hold ONE latent vector c (width L, shared by
// all heads, already normalised) and ONE rotated key part (width R, shared by all heads), not
// keys and values per head. A head's key is [W_uk c | rotated part] and its value W_uv c, but
// neither is ever built: with q_lat = W_uk^T q_plain (done by the caller as a matrix product)
//     score(i, j) = (q_lat_i . c_j + q_rot_i . kr_j) * scale,   out_lat_i = sum_j softmax_j(score) c_j
// and the caller applies W_uv to out_lat. Causal: row i of a request sees the keys 0 .. position(i)
// of that request, all read from the pages (the step's own tokens were written first).
//
// vob_latent_prep: per token, c = weight * x / sqrt(mean(x^2) + eps) of the first L columns of the
// down projection and the rotary positions on its last R columns, both written to the token's cache
// slot; the rotated query part of every head to a float32 buffer.
// vob_latent_attend: scores, softmax weights and the weighted sum in float32, keys in page order
// from the first, in tiles staged in shared memory; one warp per head, a block takes up to 8 heads
// of one row, so a key tile is read once for all of them. The order of every sum depends only on the row's
// position, never on how the request was cut into steps or on the batch around it. Steps of few rows
// (single tokens) share a row's keys over `splits` blocks, whose partial results a second small kernel
// puts together in a fixed order.
#include "common.cuh"
#include <math.h>
VOB_PDL_SWITCH(latent_attention)

// proj [T, ld]: the query of head h at columns q_off + h * (D + R) (D plain features, then R to be
// rotated); the down projection at columns down_off .. + L + R. lat [pages, 1, page, L], kr [pages,
// 1, page, R] in the cache's type TC. q_rot float32 [T, H, R]. Rows with position < 0 write nothing
// (their q_rot is zero); a slot < 0 writes no cache.
// Launch: one block of 128 threads per token.
template <typename T, typename TC>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const T* __restrict__ proj, long ld, int q_off, int H, int D, int R, int down_off, int L,
                   const float* __restrict__ norm_w, float eps, const int* __restrict__ positions, const int* __restrict__ slots,
                   const float* __restrict__ inv_freq, TC* __restrict__ lat, TC* __restrict__ kr, float* __restrict__ q_rot) {
    pdl_launch_dependents();
    pdl_wait(45);
    __shared__ float red[4];
    const int t = blockIdx.x, tid = threadIdx.x;
    const int pos = positions[t];
    const T* row = proj + (size_t)t * ld;
    const int half = R >> 1;
    float* qo = q_rot + (size_t)t * H * R;
    for (int e = tid; e < H * R; e += blockDim.x) {
        float v = 0.f;
        if (pos >= 0) {
            const int h = e / R, f = e - h * R;
            const int i = f < half ? f : f - half;
            const float ang = (float)pos * inv_freq[i];
            const float cs = cosf(ang), sn = sinf(ang);
            const T* qh = row + q_off + (size_t)h * (D + R) + D;
            const float a = ld_f(qh + i), b = ld_f(qh + i + half);
            v = f < half ? a * cs - b * sn : b * cs + a * sn;
        }
        qo[e] = v;
    }
    const int slot = slots ? slots[t] : -1;
    if (pos < 0 || slot < 0) return;
    const T* down = row + down_off;
    float ss = 0.f;
    for (int i = tid; i < L; i += blockDim.x) {
        const float x = ld_f(down + i);
        ss = fmaf(x, x, ss);
    }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    const float inv = 1.0f / sqrtf(((red[0] + red[1]) + (red[2] + red[3])) / (float)L + eps);
    TC* lo = lat + (size_t)slot * L;
    for (int i = tid; i < L; i += blockDim.x) st_f(lo + i, norm_w[i] * (ld_f(down + i) * inv));
    TC* ko = kr + (size_t)slot * R;
    for (int f = tid; f < R; f += blockDim.x) {
        const int i = f < half ? f : f - half;
        const float ang = (float)pos * inv_freq[i];
        const float cs = cosf(ang), sn = sinf(ang);
        const float a = ld_f(down + L + i), b = ld_f(down + L + i + half);
        st_f(ko + f, f < half ? a * cs - b * sn : b * cs + a * sn);
    }
}

VOB_EXPORT int vob_latent_prep(const void* proj, int code, long ld, int q_off, int H, int D, int R, int down_off, int L,
                               const float* norm_w, float eps, const int* positions, const int* slots, const float* inv_freq,
                               void* lat, void* kr, int cache_code, float* q_rot, int T, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || D < 0 || R <= 0 || (R & 1) || L <= 0 || code != cache_code) return VOB_ERR_BAD_ARG;
    VOB_DISPATCH_ELEM(code, return vob_launch(latent_prep_kernel<ElemT, ElemT>, dim3(T), dim3(128), 0, stream, (const ElemT*)proj, ld,
                                              q_off, H, D, R, down_off, L, norm_w, eps, positions, slots, inv_freq, (ElemT*)lat,
                                              (ElemT*)kr, q_rot));
    return 0;
}

// q_lat float32, element (t, h, i) at t * q_ts + h * q_hs + i; q_rot float32 [T, H, R]; out_lat of type
// TO, element (t, h, i) at t * o_ts + h * o_hs + i. NL = ceil(L / 32) registers per lane for q_lat and
// for the weighted sum. Grid (rows, ceil(H / warps)); a block has `warps` warps, one head each.
template <int NL, typename TC, typename TO>
__global__ void __launch_bounds__(256, 1)
latent_attend_kernel(const float* __restrict__ q_lat, long q_ts, long q_hs, const float* __restrict__ q_rot,
                     const TC* __restrict__ lat, const TC* __restrict__ kr, const int* __restrict__ block_tables, int max_pages,
                     const int* __restrict__ row_seq, const int* __restrict__ positions, int page_size, int H, int L, int R,
                     float scale, int KT, TO* __restrict__ out, long o_ts, long o_hs, int splits, float* __restrict__ part, int window) {
    pdl_launch_dependents();
    pdl_wait(46);
    extern __shared__ float tile[];                 // [KT][L + R]
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y * (blockDim.x >> 5) + warp;
    const bool head = h < H;
    const int pos = positions[t];
    TO* orow = out + (size_t)t * o_ts + (size_t)(head ? h : 0) * o_hs;
    // with splits > 1 block z takes the z-th share of the row's keys and leaves (max, sum, weighted sum) in `part`
    // [T, H, splits, L + 2]; the shares depend on the row's position and `splits` only
    float* prow = part + (((size_t)t * H + (head ? h : 0)) * splits + blockIdx.z) * (L + 2);
    if (pos < 0) {
        if (head && splits == 1)
            for (int i = lane; i < L; i += 32) st_f(orow + i, 0.f);
        if (head && splits > 1 && lane == 0) { prow[0] = -INFINITY; prow[1] = 0.f; }
        return;
    }
    const int* table = block_tables + (size_t)row_seq[t] * max_pages;
    const int W = L + R;
    float ql[NL], qr[4], acc[NL];
#pragma unroll
    for (int i = 0; i < NL; ++i) {
        const int c = lane + 32 * i;
        ql[i] = (head && c < L) ? q_lat[(size_t)t * q_ts + (size_t)h * q_hs + c] : 0.f;
        acc[i] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = lane + 32 * i;
        qr[i] = (head && c < R) ? q_rot[((size_t)t * H + h) * R + c] : 0.f;
    }
    float m = -INFINITY, l = 0.f;
    // the keys a row sees: all up to its own, or with a window only the last `window` of them
    const int first = window > 0 ? max(0, pos + 1 - window) : 0;
    const int share = ((pos - first + splits) / splits + KT - 1) / KT * KT;      // keys per block, whole tiles
    const int nkeys = min(pos + 1, first + (int)(blockIdx.z + 1) * share);
    for (int k0 = first + blockIdx.z * share; k0 < nkeys; k0 += KT) {
        const int n = min(KT, nkeys - k0);
        __syncthreads();
        // a warp copies whole keys (one page lookup per key, then consecutive elements)
        for (int kk = warp; kk < n; kk += (int)(blockDim.x >> 5)) {
            const int key = k0 + kk;
            const size_t slot = (size_t)table[key / page_size] * page_size + key % page_size;
            float* dst = tile + kk * W;
            for (int c = lane; c < L; c += 32) dst[c] = ld_f(lat + slot * L + c);
            for (int c = lane; c < R; c += 32) dst[L + c] = ld_f(kr + slot * R + c);
        }
        __syncthreads();
        // four keys at a time: their dot products and reductions are independent chains
        for (int kk = 0; kk < n; kk += 4) {
            float sc[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float* kv = tile + min(kk + j, n - 1) * W;
                float a = 0.f;
#pragma unroll
                for (int i = 0; i < NL; ++i) {
                    const int c = lane + 32 * i;
                    if (c < L) a = fmaf(ql[i], kv[c], a);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int c = lane + 32 * i;
                    if (c < R) a = fmaf(qr[i], kv[L + c], a);
                }
                sc[j] = a;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
                for (int j = 0; j < 4; ++j) sc[j] += __shfl_xor_sync(0xffffffffu, sc[j], o);
            }
            float mn = m;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                sc[j] = kk + j < n ? sc[j] * scale : -INFINITY;
                mn = fmaxf(mn, sc[j]);
            }
            const float corr = expf(m - mn);            // exp(-inf) = 0 at the first keys
            float p[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) p[j] = expf(sc[j] - mn);
            l = fmaf(l, corr, (p[0] + p[1]) + (p[2] + p[3]));
#pragma unroll
            for (int i = 0; i < NL; ++i) {
                const int c = lane + 32 * i;
                float a = acc[i] * corr;
                if (c < L) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) a = fmaf(p[j], tile[min(kk + j, n - 1) * W + c], a);
                }
                acc[i] = a;
            }
            m = mn;
        }
    }
    if (head && splits == 1) {
        const float inv = 1.0f / l;
#pragma unroll
        for (int i = 0; i < NL; ++i) {
            const int c = lane + 32 * i;
            if (c < L) st_f(orow + c, acc[i] * inv);
        }
    }
    if (head && splits > 1) {
        if (lane == 0) { prow[0] = m; prow[1] = l; }
#pragma unroll
        for (int i = 0; i < NL; ++i) {
            const int c = lane + 32 * i;
            if (c < L) prow[2 + c] = acc[i];
        }
    }
}

// The shares of a row's keys put together, in share order: out = sum_z acc_z e^(m_z - M) / sum_z l_z e^(m_z - M).
// Launch: one warp per (row, head).
template <typename TO>
__global__ void __launch_bounds__(32)
latent_merge_kernel(const float* __restrict__ part, const int* __restrict__ positions, int H, int L, int splits,
                    TO* __restrict__ out, long o_ts, long o_hs) {
    pdl_launch_dependents();
    pdl_wait(47);
    const int t = blockIdx.x, h = blockIdx.y, lane = threadIdx.x;
    TO* orow = out + (size_t)t * o_ts + (size_t)h * o_hs;
    const float* p = part + ((size_t)t * H + h) * splits * (L + 2);
    if (positions[t] < 0) {
        for (int i = lane; i < L; i += 32) st_f(orow + i, 0.f);
        return;
    }
    float M = -INFINITY;
    for (int z = 0; z < splits; ++z) M = fmaxf(M, p[(size_t)z * (L + 2)]);
    float l = 0.f;
    for (int z = 0; z < splits; ++z) l = fmaf(p[(size_t)z * (L + 2) + 1], expf(p[(size_t)z * (L + 2)] - M), l);
    const float inv = 1.0f / l;
    for (int i = lane; i < L; i += 32) {
        float a = 0.f;
        for (int z = 0; z < splits; ++z) {
            const float* pz = p + (size_t)z * (L + 2);
            if (pz[1] > 0.f) a = fmaf(pz[2 + i], expf(pz[0] - M), a);
        }
        st_f(orow + i, a * inv);
    }
}

VOB_EXPORT int vob_latent_attend(const float* q_lat, long q_ts, long q_hs, const float* q_rot, const void* lat, const void* kr,
                                 int cache_code, const int* block_tables, int max_pages, const int* row_seq, const int* positions,
                                 int page_size, int T, int H, int L, int R, float scale, void* out, int out_code, long o_ts, long o_hs,
                                 int splits, float* part, int window, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (window < 0) return VOB_ERR_BAD_ARG;
    if (H <= 0 || L <= 0 || R <= 0 || page_size <= 0 || max_pages <= 0 || cache_code != out_code) return VOB_ERR_BAD_ARG;
    if (splits < 1 || splits > 65535 || (splits > 1 && !part) || H > 65535) return VOB_ERR_BAD_ARG;
    if (L > 1024 || R > 128) return VOB_ERR_UNSUPPORTED;
    const int warps = H < 8 ? H : 8;
    const int W = L + R;
    int KT = (int)(40 * 1024 / ((size_t)W * 4));
    KT = KT > 32 ? 32 : KT < 1 ? 1 : KT;
    const size_t smem = (size_t)KT * W * 4;
    dim3 grid(T, (H + warps - 1) / warps, splits), block(32 * warps);
    const int nl = (L + 31) / 32;
    int status = VOB_ERR_BAD_ARG;
#define VOB_LA(N, TC)                                                                                                          \
    status = vob_launch(latent_attend_kernel<N, TC, TC>, grid, block, smem, stream, q_lat, q_ts, q_hs, q_rot, (const TC*)lat, \
                        (const TC*)kr, block_tables, max_pages, row_seq, positions, page_size, H, L, R, scale, KT, (TC*)out, o_ts, o_hs, \
                        splits, part, window)
#define VOB_LA_N(TC)                       \
    do {                                   \
        if (nl <= 4) { VOB_LA(4, TC); }        \
        else if (nl <= 8) { VOB_LA(8, TC); }   \
        else if (nl <= 16) { VOB_LA(16, TC); } \
        else { VOB_LA(32, TC); }               \
        if (status == 0 && splits > 1)         \
            status = vob_launch(latent_merge_kernel<TC>, dim3(T, H), dim3(32), 0, stream, (const float*)part, positions, H, L, splits, \
                                (TC*)out, o_ts, o_hs);                                                                          \
    } while (0)
    if (cache_code == VOB_F32) VOB_LA_N(float);
    else if (cache_code == VOB_BF16) VOB_LA_N(__nv_bfloat16);
#undef VOB_LA_N
#undef VOB_LA
    return status;
}


// ---------------------------------------------------------------------------------------------
// Prompt portions in bfloat16 on the tensor cores (mma.sync m16n8k16, operands by ldmatrix). A block takes 16
// consecutive tokens of one request and HB heads; a head has WPH warps, each of which owns a share of the latent
// columns of O (at most 256) and computes the head's S = Q K^T for itself. A tile of 32 keys ([c | kr], L + R
// wide, bfloat16, rows padded by 16 bytes so that ldmatrix meets no bank conflict) is brought into shared memory
// once for all of them; the next tile is fetched into registers meanwhile. S, the softmax (float32, running
// maximum and sum per row), P (bfloat16, taken straight from S's registers as the next product's A operand) and
// O (float32) never leave the registers. Needs L and R multiples of 16. Rows are a request's seq_starts[s] + 16
// * tile ..; their positions are consecutive, so the tile's last row bounds the keys and every row masks what
// lies behind its own position.
// ---------------------------------------------------------------------------------------------
#define VOB_LTC_BN 32
#define VOB_LTC_PRE 10        // 16-byte pieces of the next key tile a thread holds ahead (the rest of a tile is copied when it is due)

__device__ __forceinline__ void ldsm_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma_bf16_16816(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}

// NT16: groups of 16 latent columns a warp owns at most (its O accumulator is NT16 * 8 registers).
template <int NT16>
__global__ void __launch_bounds__(256, 1)
latent_attend_tc_kernel(const float* __restrict__ q_lat, long q_ts, long q_hs, const float* __restrict__ q_rot,
                        const __nv_bfloat16* __restrict__ lat, const __nv_bfloat16* __restrict__ kr, const int* __restrict__ block_tables,
                        int max_pages, const int* __restrict__ seq_starts, const int* __restrict__ positions, int page_size, int H, int L,
                        int R, float scale, __nv_bfloat16* __restrict__ out, long o_ts, long o_hs, int WPH, int colsw, int window) {
    constexpr int BN = VOB_LTC_BN;
    pdl_launch_dependents();
    pdl_wait(48);
    const int s = blockIdx.z, NW = blockDim.x >> 5, HB = NW / WPH;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hh = warp / WPH, wsub = warp - hh * WPH;
    const int h = blockIdx.y * HB + hh;
    const bool head = h < H;
    const int r0 = seq_starts[s] + blockIdx.x * 16, r1 = seq_starts[s + 1];
    if (r0 >= r1) return;
    const int nrows = min(16, r1 - r0);
    const int D = L + R, DP = D + 8;
    extern __shared__ __align__(128) unsigned char ltc_smem[];
    __nv_bfloat16* Kt = reinterpret_cast<__nv_bfloat16*>(ltc_smem);                               // [BN][DP]
    __nv_bfloat16* Q = Kt + (size_t)BN * DP + (size_t)hh * 16 * DP;                                // [16][DP] per head
    for (int e = lane + 32 * wsub; e < 16 * D; e += 32 * WPH) {
        const int i = e / D, c = e - i * D;
        float v = 0.f;
        if (head && i < nrows)
            v = c < L ? q_lat[(size_t)(r0 + i) * q_ts + (size_t)h * q_hs + c] : q_rot[((size_t)(r0 + i) * H + h) * R + (c - L)];
        Q[i * DP + c] = __float2bfloat16_rn(v);
    }
    const int pos0 = positions[r0], pos_hi = pos0 + nrows - 1;
    // with a window a row sees only its last `window` keys: the tile's first row bounds the keys from below (pages before
    // that may have been given back and are never addressed), and the walk starts at the tile of BN keys that holds it, so
    // that a row's keys fall into the same tiles however the prompt was cut
    const int key_lo = window > 0 ? max(0, pos0 + 1 - window) : 0;
    const int k_start = key_lo / BN * BN;
    const int* table = block_tables + (size_t)s * max_pages;
    // this warp's latent columns, in groups of 16
    const int col0 = wsub * colsw;
    const int n16 = max(0, min(colsw, L - col0)) / 16;
    const int g = lane >> 2, t4 = lane & 3;          // this thread's rows g and g + 8, columns 2 * t4, + 1 of every 8
    float o[NT16 * 2][4];
#pragma unroll
    for (int i = 0; i < NT16 * 2; ++i) { o[i][0] = 0.f; o[i][1] = 0.f; o[i][2] = 0.f; o[i][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;       // l: this thread's share of the row sums
    const bool row0 = g < nrows, row1 = g + 8 < nrows;
    const int lat_chunks = L / 8, kr_chunks = R / 8;            // 16-byte pieces of a key
    // The key tile as a list of 16-byte pieces, BN keys x (lat_chunks + kr_chunks) pieces: thread t takes pieces
    // t, t + threads, ... The NEXT tile's pieces are fetched into registers while this tile is worked on.
    const int pieces = lat_chunks + kr_chunks, tile_pieces = BN * pieces;
    const int dp_pieces = DP / 8;                    // a row of Kt in 16-byte pieces (DP is a multiple of 8)
    uint4 nxt[VOB_LTC_PRE];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int i = 0; i < VOB_LTC_PRE; ++i) {
            const int x = (int)threadIdx.x + i * (int)blockDim.x;
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (x < tile_pieces) {
                const int kk = x / pieces, c = x - kk * pieces;
                const int key = k0 + kk;
                if (key <= pos_hi && key >= key_lo) {
                    const size_t slot = (size_t)table[key / page_size] * page_size + key % page_size;
                    val = c < lat_chunks ? reinterpret_cast<const uint4*>(lat + slot * L)[c]
                                         : reinterpret_cast<const uint4*>(kr + slot * R)[c - lat_chunks];
                }
            }
            nxt[i] = val;
        }
    };
    fetch(k_start);
    for (int k0 = k_start; k0 <= pos_hi; k0 += BN) {
        __syncthreads();
#pragma unroll
        for (int i = 0; i < VOB_LTC_PRE; ++i) {
            const int x = (int)threadIdx.x + i * (int)blockDim.x;
            if (x < tile_pieces) {
                const int kk = x / pieces, c = x - kk * pieces;
                reinterpret_cast<uint4*>(Kt)[(size_t)kk * dp_pieces + c] = nxt[i];
            }
        }
        // what of a tile the registers do not hold (small blocks, wide keys) is copied now
        for (int x = (int)threadIdx.x + VOB_LTC_PRE * (int)blockDim.x; x < tile_pieces; x += (int)blockDim.x) {
            const int kk = x / pieces, c = x - kk * pieces;
            const int key = k0 + kk;
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (key <= pos_hi && key >= key_lo) {
                const size_t slot = (size_t)table[key / page_size] * page_size + key % page_size;
                val = c < lat_chunks ? reinterpret_cast<const uint4*>(lat + slot * L)[c]
                                     : reinterpret_cast<const uint4*>(kr + slot * R)[c - lat_chunks];
            }
            reinterpret_cast<uint4*>(Kt)[(size_t)kk * dp_pieces + c] = val;
        }
        if (k0 + BN <= pos_hi) fetch(k0 + BN);
        __syncthreads();
        if (!head) continue;
        // S = Q K^T: 16 rows x 32 keys, four accumulator tiles of 8 keys
        float sc[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) { sc[j][0] = 0.f; sc[j][1] = 0.f; sc[j][2] = 0.f; sc[j][3] = 0.f; }
#pragma unroll 2
        for (int ks = 0; ks < D / 16; ++ks) {
            unsigned a0, a1, a2, a3;
            ldsm_x4(a0, a1, a2, a3, Q + (size_t)(lane & 15) * DP + ks * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int jp = 0; jp < 2; ++jp) {            // keys 16 * jp .. + 15: two accumulator tiles
                unsigned b0, b1, b2, b3;
                ldsm_x4(b0, b1, b2, b3, Kt + (size_t)(16 * jp + (lane >> 4) * 8 + (lane & 7)) * DP + ks * 16 + ((lane >> 3) & 1) * 8);
                mma_bf16_16816(sc[2 * jp], a0, a1, a2, a3, b0, b1);
                mma_bf16_16816(sc[2 * jp + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        // the softmax of rows g and g + 8 over this tile's keys
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = k0 + 8 * j + 2 * t4 + e;
                const bool in0 = key <= pos0 + g && (window <= 0 || key > pos0 + g - window);
                const bool in1 = key <= pos0 + g + 8 && (window <= 0 || key > pos0 + g + 8 - window);
                sc[j][e] = (row0 && in0) ? sc[j][e] * scale : -INFINITY;
                sc[j][2 + e] = (row1 && in1) ? sc[j][2 + e] * scale : -INFINITY;
                mx0 = fmaxf(mx0, sc[j][e]);
                mx1 = fmaxf(mx1, sc[j][2 + e]);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const bool none0 = mn0 == -INFINITY, none1 = mn1 == -INFINITY;
        const float corr0 = none0 ? 1.f : expf(m0 - mn0), corr1 = none1 ? 1.f : expf(m1 - mn1);
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                sc[j][e] = none0 ? 0.f : expf(sc[j][e] - mn0);
                sc[j][2 + e] = none1 ? 0.f : expf(sc[j][2 + e] - mn1);
                sum0 += sc[j][e];
                sum1 += sc[j][2 + e];
            }
        }
        l0 = fmaf(l0, corr0, sum0);
        l1 = fmaf(l1, corr1, sum1);
        m0 = mn0;
        m1 = mn1;
        // P as the A operand of the second product: the accumulator tiles of 8 keys pair up into 16 keys
        unsigned pa[2][4];
#pragma unroll
        for (int jp = 0; jp < 2; ++jp) {
            pa[jp][0] = pack_bf16(sc[2 * jp][0], sc[2 * jp][1]);
            pa[jp][1] = pack_bf16(sc[2 * jp][2], sc[2 * jp][3]);
            pa[jp][2] = pack_bf16(sc[2 * jp + 1][0], sc[2 * jp + 1][1]);
            pa[jp][3] = pack_bf16(sc[2 * jp + 1][2], sc[2 * jp + 1][3]);
        }
        // O = O * corr + P C over this warp's latent columns
#pragma unroll
        for (int n = 0; n < NT16; ++n) {
            if (n < n16) {
                o[2 * n][0] *= corr0; o[2 * n][1] *= corr0; o[2 * n][2] *= corr1; o[2 * n][3] *= corr1;
                o[2 * n + 1][0] *= corr0; o[2 * n + 1][1] *= corr0; o[2 * n + 1][2] *= corr1; o[2 * n + 1][3] *= corr1;
#pragma unroll
                for (int jp = 0; jp < 2; ++jp) {
                    unsigned b0, b1, b2, b3;
                    ldsm_x4_trans(b0, b1, b2, b3, Kt + (size_t)(16 * jp + ((lane >> 3) & 1) * 8 + (lane & 7)) * DP + col0 + 16 * n + (lane >> 4) * 8);
                    mma_bf16_16816(o[2 * n], pa[jp][0], pa[jp][1], pa[jp][2], pa[jp][3], b0, b1);
                    mma_bf16_16816(o[2 * n + 1], pa[jp][0], pa[jp][1], pa[jp][2], pa[jp][3], b2, b3);
                }
            }
        }
    }
    if (!head) return;
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = 1.0f / l0, inv1 = 1.0f / l1;
#pragma unroll
    for (int n = 0; n < NT16 * 2; ++n) {
        if (n < 2 * n16) {
            const int c = col0 + 8 * n + 2 * t4;
            if (row0)
                *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(r0 + g) * o_ts + (size_t)h * o_hs + c) = __floats2bfloat162_rn(o[n][0] * inv0, o[n][1] * inv0);
            if (row1)
                *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(r0 + g + 8) * o_ts + (size_t)h * o_hs + c) = __floats2bfloat162_rn(o[n][2] * inv1, o[n][3] * inv1);
        }
    }
}

// The shape of a block of the tensor-core kernel: warps per head (each with at most 256 latent columns, a multiple of
// 16), the columns per warp, and heads per block (0: the sizes do not fit the kernel).
static int ltc_shape(int H, int L, int R, int* wph, int* colsw) {
    if (L % 16 || R % 16 || L <= 0 || R <= 0 || L > 1024) return 0;
    *wph = (L + 255) / 256;
    *colsw = ((L / 16 + *wph - 1) / *wph) * 16;
    const size_t DP = (size_t)L + R + 8;
    const size_t shared = (size_t)VOB_LTC_BN * DP * 2, per_head = 16 * DP * 2;
    int hb = 8 / *wph;                                   // at most eight warps
    while (hb > 1 && shared + hb * per_head > 100 * 1024) --hb;
    if (shared + hb * per_head > 200 * 1024) return 0;
    return hb > H ? H : hb;
}

VOB_EXPORT int vob_latent_attend_tc_supported(int H, int L, int R) {
    int wph, colsw;
    return ltc_shape(H, L, R, &wph, &colsw) > 0 ? 1 : 0;
}

// q_lat, q_rot, out and the caches as for vob_latent_attend (bfloat16 caches and out only; out's strides even);
// seq_starts int32 [seqs + 1]; max_new: no request brings more rows than this.
VOB_EXPORT int vob_latent_attend_tc(const float* q_lat, long q_ts, long q_hs, const float* q_rot, const void* lat, const void* kr,
                                    const int* block_tables, int max_pages, const int* seq_starts, const int* positions, int page_size,
                                    int seqs, int max_new, int H, int L, int R, float scale, void* out, long o_ts, long o_hs,
                                    int window, cudaStream_t stream) {
    if (seqs <= 0 || max_new <= 0) return 0;
    if (window < 0) return VOB_ERR_BAD_ARG;
    int wph, colsw;
    const int hb = ltc_shape(H, L, R, &wph, &colsw);
    if (hb <= 0) return VOB_ERR_UNSUPPORTED;
    if (page_size <= 0 || max_pages <= 0 || seqs > 65535 || (H + hb - 1) / hb > 65535 || (o_ts & 1) || (o_hs & 1) || ((uintptr_t)out & 3))
        return VOB_ERR_BAD_ARG;
    const size_t DP = (size_t)L + R + 8;
    const size_t smem = (size_t)VOB_LTC_BN * DP * 2 + (size_t)hb * 16 * DP * 2;
    dim3 grid((max_new + 15) / 16, (H + hb - 1) / hb, seqs), block(32 * hb * wph);
#define VOB_LTC(N)                                                                                                              \
    do {                                                                                                                        \
        cudaError_t e = cudaFuncSetAttribute(latent_attend_tc_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return (int)e;                                                                                    \
        return vob_launch(latent_attend_tc_kernel<N>, grid, block, smem, stream, q_lat, q_ts, q_hs, q_rot, (const __nv_bfloat16*)lat, \
                          (const __nv_bfloat16*)kr, block_tables, max_pages, seq_starts, positions, page_size, H, L, R, scale,  \
                          (__nv_bfloat16*)out, o_ts, o_hs, wph, colsw, window);                                                 \
    } while (0)
    if (colsw <= 64) VOB_LTC(4);
    if (colsw <= 128) VOB_LTC(8);
    VOB_LTC(16);
#undef VOB_LTC
}
