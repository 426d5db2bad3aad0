// A feed-forward made of many small experts of which every token uses a few.
//
//   vob_moe_route    per token: router logits z = W_r x (float32 sums in feature order), scores s = softmax(z) over
//                    all experts; the experts form `n_groups` runs of neighbours, a run scores as its best expert, only
//                    experts of the `keep` best runs stand for election (n_groups <= 1: all do); the `top` experts with
//                    the largest scores are chosen (a tie goes to the lower index), their weights are their own scores
//                    (times 1 / their sum where `renorm` is set).
//   vob_moe_align    the (token, choice) pairs put in order of their expert, every expert's run padded to whole tiles
//                    of VOB_MOE_BM rows, with the expert of every tile.
//   vob_moe_gate_up  per tile: h = act(W_gate[e] x) * (W_up[e] x) for the tile's pairs (x gathered by token).
//   vob_moe_down     per tile: y[pair] = weight[pair] * (W_down[e] h[pair]), float32.
//   vob_moe_combine  out[token] = sum over the token's choices, in the order they were chosen, of y.
//
// A pair's arithmetic never depends on which other pairs share its tile or where in its expert's run it lies: every
// output element is one chain of multiply-adds over the features in order (float32 accumulation), and a token's choices
// are added in the order of its own list. So the result of a token is the same in every batch.
// Two forms of the two products: plain multiply-adds (float32 engines, and any size) and mma.sync tensor-core tiles
// (bfloat16 operands, float32 accumulation).
#include "common.cuh"
#include <mma.h>
VOB_PDL_SWITCH(moe)

#define VOB_MOE_BM 32

// ---------------------------------------------------------------------------------------------
// Routing. Four tokens per block, one warp per token for the election; 2 E floats of shared memory per token.
// Rows with a negative position (padding) choose nothing: their indices are -1.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}

template <typename T> __device__ __forceinline__ void moe_ld4(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void moe_ld4<float>(const float* p, float (&v)[4]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
template <> __device__ __forceinline__ void moe_ld4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 a = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&a.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&a.y);
    v[0] = __bfloat162float(lo.x); v[1] = __bfloat162float(lo.y); v[2] = __bfloat162float(hi.x); v[3] = __bfloat162float(hi.y);
}

// The block's four warps first share out the experts: a warp reads an expert's router row once and multiplies it with
// the rows of all four tokens (a lane's chain runs over its own features in order, whoever the other tokens are; rows
// whose width and addresses allow are read four features at a time). Then warp w holds the election of token w.
template <typename T>
__global__ void __launch_bounds__(128)
moe_route_kernel(const T* __restrict__ x, long ld_x, const float* __restrict__ w_router, const int* __restrict__ positions,
                 int T_rows, int width, int E, int top, int n_groups, int keep, int renorm, int* __restrict__ idx_out,
                 float* __restrict__ w_out) {
    pdl_launch_dependents();
    pdl_wait(71);
    extern __shared__ float sc_all[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * 4;
    const T* rows[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) rows[k] = x + (size_t)min(t0 + k, T_rows - 1) * ld_x;
    const bool by4 = width % 4 == 0 && ld_x % 4 == 0 && (((uintptr_t)x) & (4 * sizeof(T) - 1)) == 0 && (((uintptr_t)w_router) & 15) == 0;
    for (int e = warp; e < E; e += 4) {
        const float* wr = w_router + (size_t)e * width;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        if (by4) {
#pragma unroll 2
            for (int i = lane * 4; i < width; i += 128) {
                const float4 w4 = *reinterpret_cast<const float4*>(wr + i);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    float v[4];
                    moe_ld4<T>(rows[k] + i, v);
                    acc[k] = fmaf(v[0], w4.x, acc[k]); acc[k] = fmaf(v[1], w4.y, acc[k]);
                    acc[k] = fmaf(v[2], w4.z, acc[k]); acc[k] = fmaf(v[3], w4.w, acc[k]);
                }
            }
        } else {
            for (int i = lane; i < width; i += 32) {
                const float w1 = wr[i];
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[k] = fmaf(ld_f(rows[k] + i), w1, acc[k]);
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float total = warp_sum(acc[k]);
            if (lane == 0) sc_all[(size_t)k * 2 * E + e] = total;
        }
    }
    __syncthreads();
    const int t = t0 + warp;
    if (t >= T_rows) return;
    if (positions && positions[t] < 0) {
        for (int k = lane; k < top; k += 32) { idx_out[(size_t)t * top + k] = -1; w_out[(size_t)t * top + k] = 0.f; }
        return;
    }
    float* sc = sc_all + (size_t)warp * 2 * E;       // scores, then the working copy the election strikes names from
    float* cand = sc + E;
    __syncwarp();
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, sc[e]);
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) sum += expf(sc[e] - m);
    sum = warp_sum(sum);
    for (int e = lane; e < E; e += 32) {
        const float s = expf(sc[e] - m) / sum;
        sc[e] = s;
        cand[e] = (n_groups > 1) ? -1.f : s;         // with groups: nobody stands until the group is kept
    }
    __syncwarp();
    if (n_groups > 1) {
        const int per = E / n_groups;
        // a group's score sits in its first expert's place of a second working row: reuse idx via registers instead
        for (int round = 0; round < keep; ++round) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            for (int g = lane; g < n_groups; g += 32) {
                if (cand[g * per] >= 0.f) continue;                 // group already kept (its experts stand)
                float gv = -INFINITY;
                for (int j = 0; j < per; ++j) gv = fmaxf(gv, sc[g * per + j]);
                if (gv > bv) { bv = gv; bi = g; }
            }
            warp_argmax(bv, bi);
            __syncwarp();
            if (bi != 0x7fffffff)
                for (int j = lane; j < per; j += 32) cand[bi * per + j] = sc[bi * per + j];
            __syncwarp();
        }
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float c = cand[e];
            if (c >= 0.f && c > bv) { bv = c; bi = e; }
        }
        warp_argmax(bv, bi);
        __syncwarp();
        if (lane == 0) {
            idx_out[(size_t)t * top + k] = bi != 0x7fffffff ? bi : -1;
            w_out[(size_t)t * top + k] = bi != 0x7fffffff ? bv : 0.f;
            if (bi != 0x7fffffff) cand[bi] = -2.f;
        }
        if (bi != 0x7fffffff) total += bv;
        __syncwarp();
    }
    if (renorm && lane == 0 && total > 0.f)
        for (int k = 0; k < top; ++k) w_out[(size_t)t * top + k] /= total;
}

VOB_EXPORT int vob_moe_route(const void* x, int code, long ld_x, const float* w_router, const int* positions, int T, int width, int E,
                             int top, int n_groups, int keep, int renorm, int* idx_out, float* w_out, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (width <= 0 || E <= 0 || top <= 0 || top > E) return VOB_ERR_BAD_ARG;
    if (n_groups > 1 && (E % n_groups != 0 || keep <= 0 || keep > n_groups || top > keep * (E / n_groups))) return VOB_ERR_BAD_ARG;
    const size_t smem = (size_t)4 * 2 * E * sizeof(float);
    if (smem > 48 * 1024) return VOB_ERR_UNSUPPORTED;
    VOB_DISPATCH_ELEM(code, return vob_launch(moe_route_kernel<ElemT>, dim3((T + 3) / 4), dim3(128), smem, stream, (const ElemT*)x, ld_x, w_router,
                                              positions, T, width, E, top, n_groups, keep, renorm, idx_out, w_out));
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Ordering. One block of 1024 threads. idx [P] (P = tokens * top; -1: no pair) ->
//   sorted [cap]: pair numbers expert by expert, each expert's run padded with -1 to a multiple of the tile's rows
//   (32, or 128 for the large tiles of the pipelined products);
//   tile_expert [cap / rows]: the expert of every tile (-1 behind the last one);  meta[0] = tiles in use.
// cap >= P rounded up + E * rows. Where a pair lands inside its expert's run is decided by atomics and may
// differ from run to run; no result depends on it.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ idx, int P, int E, int* __restrict__ sorted, int cap, int* __restrict__ tile_expert,
                 int* __restrict__ meta, int bm) {
    pdl_launch_dependents();
    pdl_wait(72);
    extern __shared__ int sh[];
    int* count = sh;            // [E]
    int* start = sh + E;        // [E + 1] padded starts
    int* cursor = sh + 2 * E + 1;
    for (int e = threadIdx.x; e < E; e += blockDim.x) { count[e] = 0; cursor[e] = 0; }
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = idx[p];
        if (e >= 0 && e < E) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            start[e] = at;
            at += (count[e] + bm - 1) / bm * bm;
        }
        start[E] = at;
        meta[0] = at / bm;
    }
    __syncthreads();
    const int used = start[E];
    for (int i = threadIdx.x; i < cap; i += blockDim.x) sorted[i] = -1;
    for (int i = threadIdx.x; i < cap / bm; i += blockDim.x) tile_expert[i] = -1;
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x)
        for (int tl = start[e] / bm; tl < start[e + 1] / bm; ++tl) tile_expert[tl] = e;
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = idx[p];
        if (e >= 0 && e < E) sorted[start[e] + atomicAdd(&cursor[e], 1)] = p;
    }
    (void)used;
}

VOB_EXPORT int vob_moe_align(const int* idx, int P, int E, int* sorted, int cap, int* tile_expert, int* meta, int tile_rows, cudaStream_t stream) {
    const int bm = tile_rows;
    if (bm != VOB_MOE_BM && bm != 128) return VOB_ERR_BAD_ARG;
    if (P <= 0) return 0;
    if (E <= 0 || cap % bm != 0 || cap < (P + bm - 1) / bm * bm + E * bm) return VOB_ERR_BAD_ARG;
    const size_t smem = (size_t)(3 * E + 1) * sizeof(int);
    if (smem > 48 * 1024) return VOB_ERR_UNSUPPORTED;
    return vob_launch(moe_align_kernel, dim3(1), dim3(1024), smem, stream, idx, P, E, sorted, cap, tile_expert, meta, bm);
}

// ---------------------------------------------------------------------------------------------
// The experts' first product with the gate, plain multiply-adds. Grid (tiles, ceil(ff / 32)); 256 threads; thread
// (ty, tx) of 16 x 16 owns rows ty, ty + 16 and hidden columns tx, tx + 16 of the tile, gate and up of each.
// w_gu [E, 2 ff, width]: an expert's gate rows, then its up rows. act 0: silu.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float moe_silu(float g) { return g / (1.0f + expf(-g)); }
// The gate on a hidden value. act 0: silu(g) * u. act 1 (clamped): g' = min(g, limit), u' = clamp(u, -limit, limit),
// g' * sigmoid(1.702 g') * (u' + 1).
__device__ __forceinline__ float moe_gate(float g, float u, int act, float limit) {
    if (act == 0) return moe_silu(g) * u;
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
}
// a float32 sum as the activations' type holds it
template <typename T> __device__ __forceinline__ float moe_rounded(float v);
template <> __device__ __forceinline__ float moe_rounded<float>(float v) { return v; }
template <> __device__ __forceinline__ float moe_rounded<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <typename T>
__global__ void __launch_bounds__(256, 2)
moe_gate_up_kernel(const T* __restrict__ x, long ld_x, const T* __restrict__ w_gu, const int* __restrict__ sorted,
                   const int* __restrict__ tile_expert, int top, int width, int ff, T* __restrict__ h_out, int act, float limit) {
    pdl_launch_dependents();
    pdl_wait(73);
    const int tile = blockIdx.x;
    const int e = tile_expert[tile];
    if (e < 0) return;
    __shared__ float As[VOB_MOE_BM][33], Bg[32][33], Bu[32][33];
    __shared__ int pair_of[VOB_MOE_BM];
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    if (tid < VOB_MOE_BM) pair_of[tid] = sorted[tile * VOB_MOE_BM + tid];
    __syncthreads();
    const int col0 = blockIdx.y * 32;
    const T* wg = w_gu + (size_t)e * 2 * ff * width;
    const T* wu = wg + (size_t)ff * width;
    float g[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, u[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    for (int k0 = 0; k0 < width; k0 += 32) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int el = tid + 256 * i, r = el >> 5, c = el & 31;
            const int p = pair_of[r];
            const bool kin = k0 + c < width;
            As[r][c] = (p >= 0 && kin) ? ld_f(x + (size_t)(p / top) * ld_x + k0 + c) : 0.f;
            const bool cin = col0 + r < ff && kin;
            Bg[r][c] = cin ? ld_f(wg + (size_t)(col0 + r) * width + k0 + c) : 0.f;
            Bu[r][c] = cin ? ld_f(wu + (size_t)(col0 + r) * width + k0 + c) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 32; ++kk) {
            const float a0 = As[ty][kk], a1 = As[ty + 16][kk];
            const float g0 = Bg[tx][kk], g1 = Bg[tx + 16][kk], u0 = Bu[tx][kk], u1 = Bu[tx + 16][kk];
            g[0][0] = fmaf(a0, g0, g[0][0]); g[0][1] = fmaf(a0, g1, g[0][1]);
            g[1][0] = fmaf(a1, g0, g[1][0]); g[1][1] = fmaf(a1, g1, g[1][1]);
            u[0][0] = fmaf(a0, u0, u[0][0]); u[0][1] = fmaf(a0, u1, u[0][1]);
            u[1][0] = fmaf(a1, u0, u[1][0]); u[1][1] = fmaf(a1, u1, u[1][1]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int p = pair_of[ty + 16 * i];
        if (p < 0) continue;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int c = col0 + tx + 16 * j;
            // the two products are rounded to the activations' type before the gate, as separate products would be
            if (c < ff) st_f(h_out + (size_t)p * ff + c, moe_gate(moe_rounded<T>(g[i][j]), moe_rounded<T>(u[i][j]), act, limit));
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The experts' second product, plain multiply-adds. Grid (tiles, ceil(width / 64)); thread (ty, tx) owns rows ty, ty + 16
// and columns tx, tx + 16, tx + 32, tx + 48. w_down [E, width, ff]. y float32 [P, width] = weight[pair] * sum.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256, 2)
moe_down_kernel(const T* __restrict__ h, const T* __restrict__ w_down, const int* __restrict__ sorted,
                const int* __restrict__ tile_expert, const float* __restrict__ pair_w, int width, int ff, float* __restrict__ y) {
    pdl_launch_dependents();
    pdl_wait(74);
    const int tile = blockIdx.x;
    const int e = tile_expert[tile];
    if (e < 0) return;
    __shared__ float As[VOB_MOE_BM][33], Bs[64][33];
    __shared__ int pair_of[VOB_MOE_BM];
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    if (tid < VOB_MOE_BM) pair_of[tid] = sorted[tile * VOB_MOE_BM + tid];
    __syncthreads();
    const int col0 = blockIdx.y * 64;
    const T* wd = w_down + (size_t)e * width * ff;
    float acc[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < ff; k0 += 32) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int el = tid + 256 * i, r = el >> 5, c = el & 31;
            const int p = pair_of[r];
            As[r][c] = (p >= 0 && k0 + c < ff) ? ld_f(h + (size_t)p * ff + k0 + c) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int el = tid + 256 * i, r = el >> 5, c = el & 31;
            Bs[r][c] = (col0 + r < width && k0 + c < ff) ? ld_f(wd + (size_t)(col0 + r) * ff + k0 + c) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < 32; ++kk) {
            const float a0 = As[ty][kk], a1 = As[ty + 16][kk];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float b = Bs[tx + 16 * j][kk];
                acc[0][j] = fmaf(a0, b, acc[0][j]);
                acc[1][j] = fmaf(a1, b, acc[1][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int p = pair_of[ty + 16 * i];
        if (p < 0) continue;
        const float wgt = pair_w[p];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = col0 + tx + 16 * j;
            if (c < width) y[(size_t)p * width + c] = wgt * acc[i][j];
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Tensor-core forms of the two products (bfloat16 operands, float32 accumulation): warp-level 16 x 16 x 16 tiles
// through the wmma interface. A block of 128 threads (4 warps) takes one tile of 32 pairs and 64 output columns:
// warp w owns columns 16 w .. 16 w + 15 and both 16-row halves. The A tile (gathered rows) and the B tiles are staged
// in shared memory 64 features at a time. Every output element is still one accumulation over the features in
// order, whatever else the tile holds.
// ---------------------------------------------------------------------------------------------
using namespace nvcuda;
#define VOB_MOE_TK 64
#define VOB_MOE_LDS (VOB_MOE_TK + 8)      // row length in shared memory: 16-byte multiples, rows fall into different banks

__device__ __forceinline__ void moe_stage_rows(__nv_bfloat16 (*dst)[VOB_MOE_LDS], int rows, const __nv_bfloat16* const* src_rows,
                                               int k0, int K) {
    // rows x 64 features, 8 at a time (16 bytes) where the row allows, else one by one; absent rows and features are zeros
    for (int el = threadIdx.x; el < rows * (VOB_MOE_TK / 8); el += blockDim.x) {
        const int r = el / (VOB_MOE_TK / 8), c = (el % (VOB_MOE_TK / 8)) * 8;
        const __nv_bfloat16* s = src_rows[r];
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (s) {
            if (k0 + c + 8 <= K && (((uintptr_t)(s + k0 + c)) & 15) == 0) {
                v = *reinterpret_cast<const uint4*>(s + k0 + c);
            } else {
                __nv_bfloat16 tmp[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) tmp[i] = k0 + c + i < K ? s[k0 + c + i] : __float2bfloat16_rn(0.f);
                v = *reinterpret_cast<const uint4*>(tmp);
            }
        }
        *reinterpret_cast<uint4*>(&dst[r][c]) = v;
    }
}

__global__ void __launch_bounds__(128)
moe_gate_up_tc_kernel(const __nv_bfloat16* __restrict__ x, long ld_x, const __nv_bfloat16* __restrict__ w_gu,
                      const int* __restrict__ sorted, const int* __restrict__ tile_expert, int top, int width, int ff,
                      __nv_bfloat16* __restrict__ h_out, int act, float limit) {
    pdl_launch_dependents();
    pdl_wait(75);
    const int tile = blockIdx.x;
    const int e = tile_expert[tile];
    if (e < 0) return;
    __shared__ __align__(32) __nv_bfloat16 As[VOB_MOE_BM][VOB_MOE_LDS], Bg[64][VOB_MOE_LDS], Bu[64][VOB_MOE_LDS];
    __shared__ __align__(32) float Cs[4][2][16 * 16];
    __shared__ int pair_of[VOB_MOE_BM];
    __shared__ const __nv_bfloat16* a_rows[VOB_MOE_BM];
    __shared__ const __nv_bfloat16* g_rows[64];
    __shared__ const __nv_bfloat16* u_rows[64];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int col0 = blockIdx.y * 64;
    const __nv_bfloat16* wg = w_gu + (size_t)e * 2 * ff * width;
    const __nv_bfloat16* wu = wg + (size_t)ff * width;
    if (tid < VOB_MOE_BM) {
        const int p = sorted[tile * VOB_MOE_BM + tid];
        pair_of[tid] = p;
        a_rows[tid] = p >= 0 ? x + (size_t)(p / top) * ld_x : nullptr;
    }
    if (tid < 64) {
        g_rows[tid] = col0 + tid < ff ? wg + (size_t)(col0 + tid) * width : nullptr;
        u_rows[tid] = col0 + tid < ff ? wu + (size_t)(col0 + tid) * width : nullptr;
    }
    __syncthreads();
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> cg[2], cu[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) { wmma::fill_fragment(cg[i], 0.f); wmma::fill_fragment(cu[i], 0.f); }
    for (int k0 = 0; k0 < width; k0 += VOB_MOE_TK) {
        moe_stage_rows(As, VOB_MOE_BM, a_rows, k0, width);
        moe_stage_rows(Bg, 64, g_rows, k0, width);
        moe_stage_rows(Bu, 64, u_rows, k0, width);
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < VOB_MOE_TK; kk += 16) {
            wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> bg, bu;
            wmma::load_matrix_sync(bg, &Bg[warp * 16][kk], VOB_MOE_LDS);
            wmma::load_matrix_sync(bu, &Bu[warp * 16][kk], VOB_MOE_LDS);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> a;
                wmma::load_matrix_sync(a, &As[16 * i][kk], VOB_MOE_LDS);
                wmma::mma_sync(cg[i], a, bg, cg[i]);
                wmma::mma_sync(cu[i], a, bu, cu[i]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        wmma::store_matrix_sync(Cs[warp][0], cg[i], 16, wmma::mem_row_major);
        wmma::store_matrix_sync(Cs[warp][1], cu[i], 16, wmma::mem_row_major);
        __syncwarp();
        for (int el = lane; el < 256; el += 32) {
            const int r = el >> 4, c = el & 15;
            const int p = pair_of[16 * i + r], col = col0 + warp * 16 + c;
            if (p >= 0 && col < ff) {
                const float gr = __bfloat162float(__float2bfloat16_rn(Cs[warp][0][el]));
                const float ur = __bfloat162float(__float2bfloat16_rn(Cs[warp][1][el]));
                h_out[(size_t)p * ff + col] = __float2bfloat16_rn(moe_gate(gr, ur, act, limit));
            }
        }
        __syncwarp();
    }
}

__global__ void __launch_bounds__(128)
moe_down_tc_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ w_down, const int* __restrict__ sorted,
                   const int* __restrict__ tile_expert, const float* __restrict__ pair_w, int width, int ff, float* __restrict__ y) {
    pdl_launch_dependents();
    pdl_wait(76);
    const int tile = blockIdx.x;
    const int e = tile_expert[tile];
    if (e < 0) return;
    __shared__ __align__(32) __nv_bfloat16 As[VOB_MOE_BM][VOB_MOE_LDS], Bs[64][VOB_MOE_LDS];
    __shared__ __align__(32) float Cs[4][16 * 16];
    __shared__ int pair_of[VOB_MOE_BM];
    __shared__ const __nv_bfloat16* a_rows[VOB_MOE_BM];
    __shared__ const __nv_bfloat16* b_rows[64];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int col0 = blockIdx.y * 64;
    const __nv_bfloat16* wd = w_down + (size_t)e * width * ff;
    if (tid < VOB_MOE_BM) {
        const int p = sorted[tile * VOB_MOE_BM + tid];
        pair_of[tid] = p;
        a_rows[tid] = p >= 0 ? h + (size_t)p * ff : nullptr;
    }
    if (tid < 64) b_rows[tid] = col0 + tid < width ? wd + (size_t)(col0 + tid) * ff : nullptr;
    __syncthreads();
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> cc[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) wmma::fill_fragment(cc[i], 0.f);
    for (int k0 = 0; k0 < ff; k0 += VOB_MOE_TK) {
        moe_stage_rows(As, VOB_MOE_BM, a_rows, k0, ff);
        moe_stage_rows(Bs, 64, b_rows, k0, ff);
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < VOB_MOE_TK; kk += 16) {
            wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> b;
            wmma::load_matrix_sync(b, &Bs[warp * 16][kk], VOB_MOE_LDS);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> a;
                wmma::load_matrix_sync(a, &As[16 * i][kk], VOB_MOE_LDS);
                wmma::mma_sync(cc[i], a, b, cc[i]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        wmma::store_matrix_sync(Cs[warp], cc[i], 16, wmma::mem_row_major);
        __syncwarp();
        for (int el = lane; el < 256; el += 32) {
            const int r = el >> 4, c = el & 15;
            const int p = pair_of[16 * i + r], col = col0 + warp * 16 + c;
            if (p >= 0 && col < width) y[(size_t)p * width + col] = pair_w[p] * Cs[warp][el];
        }
        __syncwarp();
    }
}

// ---------------------------------------------------------------------------------------------
// The same two products for rows that 16-byte copies can fetch (K a multiple of 8, 16-byte aligned rows): tiles of BM
// pairs (32: four warps; 128: eight warps, two along the rows) and 128 weight rows (gate_up: 64 gate and the 64 up rows
// of the same hidden columns; down: 128 output columns), 32 features a stage, STAGES stages in flight through cp.async
// (absent rows and features behind K arrive as zeros). The order of a sum is the one of the kernels above: 16
// features a step, in order.
// ---------------------------------------------------------------------------------------------
#define VOB_MOE_PK 32
#define VOB_MOE_PLD (VOB_MOE_PK + 8)

__device__ __forceinline__ void moe_cp16(void* dst, const void* src, int bytes) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void moe_cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void moe_cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

template <int BM, int STAGES, bool DOWN>
__global__ void __launch_bounds__(BM == 128 ? 256 : 128)
moe_pipe_kernel(const __nv_bfloat16* __restrict__ a, long ld_a, int a_div, const __nv_bfloat16* __restrict__ w,
                const int* __restrict__ sorted, const int* __restrict__ tile_expert, const float* __restrict__ pair_w,
                int K, int N, void* __restrict__ out, int act, float limit) {
    pdl_launch_dependents();
    pdl_wait(DOWN ? 76 : 75);
    constexpr int WR = BM == 128 ? 2 : 1;             // warps along the rows
    constexpr int NT = 128 * WR;
    constexpr int RF = BM / WR / 16;                   // 16-row fragments a warp owns
    constexpr int ROWS = BM + 128;                     // rows of a stage: the pairs, then the weight rows
    constexpr int CHUNKS = (ROWS * (VOB_MOE_PK / 8) + NT - 1) / NT;
    const int tile = blockIdx.x;
    const int e = tile_expert[tile];
    if (e < 0) return;
    extern __shared__ __align__(128) unsigned char moe_smem[];
    __nv_bfloat16* stages = reinterpret_cast<__nv_bfloat16*>(moe_smem);
    __shared__ int pair_of[BM];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, wc = warp & 3, wr = warp >> 2;
    const int col0 = blockIdx.y * (DOWN ? 128 : 64);
    // the rows this thread fetches, the same in every stage
    const __nv_bfloat16* src[CHUNKS];
    int dst_off[CHUNKS], feat[CHUNKS];
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) {
        const int el = tid + NT * i;
        const int r = el / (VOB_MOE_PK / 8), c = (el % (VOB_MOE_PK / 8)) * 8;
        src[i] = nullptr;
        dst_off[i] = -1;
        feat[i] = c;
        if (r >= ROWS) continue;
        dst_off[i] = r * VOB_MOE_PLD + c;
        if (r < BM) {
            const int p = sorted[tile * BM + r];
            if (c == 0) pair_of[r] = p;
            if (p >= 0) src[i] = a + (size_t)(p / a_div) * ld_a;
        } else {
            const int j = r - BM;
            if (DOWN) {
                if (col0 + j < N) src[i] = w + ((size_t)e * N + col0 + j) * K;
            } else {
                const int col = col0 + (j & 63);
                if (col < N) src[i] = w + ((size_t)e * 2 * N + (j < 64 ? 0 : N) + col) * K;
            }
        }
    }
    auto fetch = [&](int stage, int k0) {
        __nv_bfloat16* base = stages + (size_t)stage * ROWS * VOB_MOE_PLD;
#pragma unroll
        for (int i = 0; i < CHUNKS; ++i) {
            if (dst_off[i] < 0) continue;
            const int left = (K - k0 - feat[i]) * 2;
            const int bytes = src[i] ? max(0, min(16, left)) : 0;
            moe_cp16(base + dst_off[i], bytes > 0 ? (const void*)(src[i] + k0 + feat[i]) : (const void*)w, bytes);
        }
    };
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> c0[RF], c1[RF];
#pragma unroll
    for (int i = 0; i < RF; ++i) { wmma::fill_fragment(c0[i], 0.f); wmma::fill_fragment(c1[i], 0.f); }
    const int nk = (K + VOB_MOE_PK - 1) / VOB_MOE_PK;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < nk) fetch(s, s * VOB_MOE_PK);
        moe_cp_commit();
    }
    for (int it = 0; it < nk; ++it) {
        moe_cp_wait<STAGES - 2>();
        __syncthreads();                                // stage `it` has arrived for everyone; stage `it - 1` is read by nobody
        if (it + STAGES - 1 < nk) fetch((it + STAGES - 1) % STAGES, (it + STAGES - 1) * VOB_MOE_PK);
        moe_cp_commit();
        const __nv_bfloat16* As = stages + (size_t)(it % STAGES) * ROWS * VOB_MOE_PLD;
        const __nv_bfloat16* Bs = As + BM * VOB_MOE_PLD;
#pragma unroll
        for (int kk = 0; kk < VOB_MOE_PK; kk += 16) {
            wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> b0, b1;
            wmma::load_matrix_sync(b0, Bs + (wc * 16) * VOB_MOE_PLD + kk, VOB_MOE_PLD);
            wmma::load_matrix_sync(b1, Bs + (64 + wc * 16) * VOB_MOE_PLD + kk, VOB_MOE_PLD);
#pragma unroll
            for (int i = 0; i < RF; ++i) {
                wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> fa;
                wmma::load_matrix_sync(fa, As + (wr * (BM / WR) + 16 * i) * VOB_MOE_PLD + kk, VOB_MOE_PLD);
                wmma::mma_sync(c0[i], fa, b0, c0[i]);
                wmma::mma_sync(c1[i], fa, b1, c1[i]);
            }
        }
    }
    moe_cp_wait<0>();
    __syncthreads();                                    // the stages are free: each warp takes 2 KB of them for its results
    float* Cs = reinterpret_cast<float*>(moe_smem) + warp * 512;
#pragma unroll
    for (int i = 0; i < RF; ++i) {
        wmma::store_matrix_sync(Cs, c0[i], 16, wmma::mem_row_major);
        wmma::store_matrix_sync(Cs + 256, c1[i], 16, wmma::mem_row_major);
        __syncwarp();
        for (int el = lane; el < 256; el += 32) {
            const int r = el >> 4, c = el & 15;
            const int p = pair_of[wr * (BM / WR) + 16 * i + r];
            if (p < 0) continue;
            if (DOWN) {
                float* y = reinterpret_cast<float*>(out);
                const float wgt = pair_w[p];
                const int ca = col0 + wc * 16 + c, cb = ca + 64;
                if (ca < N) y[(size_t)p * N + ca] = wgt * Cs[el];
                if (cb < N) y[(size_t)p * N + cb] = wgt * Cs[256 + el];
            } else {
                const int col = col0 + wc * 16 + c;
                if (col < N) {
                    const float gr = __bfloat162float(__float2bfloat16_rn(Cs[el]));
                    const float ur = __bfloat162float(__float2bfloat16_rn(Cs[256 + el]));
                    reinterpret_cast<__nv_bfloat16*>(out)[(size_t)p * N + col] = __float2bfloat16_rn(moe_gate(gr, ur, act, limit));
                }
            }
        }
        __syncwarp();
    }
}

template <int BM, int STAGES, bool DOWN>
static int moe_pipe_launch(dim3 grid, cudaStream_t stream, const __nv_bfloat16* a, long ld_a, int a_div, const __nv_bfloat16* w,
                           const int* sorted, const int* tile_expert, const float* pair_w, int K, int N, void* out, int act = 0, float limit = 0.f) {
    const size_t smem = (size_t)STAGES * (BM + 128) * VOB_MOE_PLD * sizeof(__nv_bfloat16);
    static bool raised = false;
    if (!raised) {
        cudaError_t err = cudaFuncSetAttribute(moe_pipe_kernel<BM, STAGES, DOWN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
        raised = true;
    }
    return vob_launch(moe_pipe_kernel<BM, STAGES, DOWN>, grid, dim3(BM == 128 ? 256 : 128), smem, stream, a, ld_a, a_div, w, sorted,
                      tile_expert, pair_w, K, N, out, act, limit);
}

static inline bool moe_rows_by16(const void* p, long ld, int K) { return K % 8 == 0 && ld % 8 == 0 && (((uintptr_t)p) & 15) == 0; }

// `tensor_cores` (bfloat16 only): the wmma forms, the pipelined one where the rows allow 16-byte copies. `tile_rows`: the rows
// of a tile as the ordering made them (32; 128 only with the pipelined form). `max_tiles` = rows of `sorted` / tile_rows: the
// grid covers them all and tiles behind the last one in use leave at once.
VOB_EXPORT int vob_moe_gate_up(const void* x, int code, long ld_x, const void* w_gu, const int* sorted, const int* tile_expert,
                               int max_tiles, int tile_rows, int top, int width, int ff, void* h_out, int tensor_cores, int act, float limit,
                               cudaStream_t stream) {
    if (max_tiles <= 0) return 0;
    if (top <= 0 || width <= 0 || ff <= 0 || (act != 0 && act != 1)) return VOB_ERR_BAD_ARG;
    if (tile_rows != VOB_MOE_BM && !(tile_rows == 128 && tensor_cores)) return VOB_ERR_BAD_ARG;
    if (tensor_cores) {
        if (code != VOB_BF16) return VOB_ERR_BAD_ARG;
        if ((ff + 63) / 64 > 65535) return VOB_ERR_UNSUPPORTED;
        const dim3 grid(max_tiles, (ff + 63) / 64);
        const __nv_bfloat16 *xa = (const __nv_bfloat16*)x, *wa = (const __nv_bfloat16*)w_gu;
        if (moe_rows_by16(x, ld_x, width) && moe_rows_by16(w_gu, width, width)) {
            if (tile_rows == 128) return moe_pipe_launch<128, 3, false>(grid, stream, xa, ld_x, top, wa, sorted, tile_expert, nullptr, width, ff, h_out, act, limit);
            return moe_pipe_launch<32, 4, false>(grid, stream, xa, ld_x, top, wa, sorted, tile_expert, nullptr, width, ff, h_out, act, limit);
        }
        if (tile_rows != VOB_MOE_BM) return VOB_ERR_UNSUPPORTED;
        return vob_launch(moe_gate_up_tc_kernel, grid, dim3(128), 0, stream, xa, ld_x, wa, sorted, tile_expert, top, width, ff,
                          (__nv_bfloat16*)h_out, act, limit);
    }
    if ((ff + 31) / 32 > 65535) return VOB_ERR_UNSUPPORTED;
    VOB_DISPATCH_ELEM(code, return vob_launch(moe_gate_up_kernel<ElemT>, dim3(max_tiles, (ff + 31) / 32), dim3(256), 0, stream, (const ElemT*)x,
                                              ld_x, (const ElemT*)w_gu, sorted, tile_expert, top, width, ff, (ElemT*)h_out, act, limit));
    return 0;
}

VOB_EXPORT int vob_moe_down(const void* h, int code, const void* w_down, const int* sorted, const int* tile_expert, const float* pair_w,
                            int max_tiles, int tile_rows, int width, int ff, float* y, int tensor_cores, cudaStream_t stream) {
    if (max_tiles <= 0) return 0;
    if (width <= 0 || ff <= 0) return VOB_ERR_BAD_ARG;
    if (tile_rows != VOB_MOE_BM && !(tile_rows == 128 && tensor_cores)) return VOB_ERR_BAD_ARG;
    if ((width + 63) / 64 > 65535) return VOB_ERR_UNSUPPORTED;
    if (tensor_cores) {
        if (code != VOB_BF16) return VOB_ERR_BAD_ARG;
        const __nv_bfloat16 *ha = (const __nv_bfloat16*)h, *wa = (const __nv_bfloat16*)w_down;
        if (moe_rows_by16(h, ff, ff) && moe_rows_by16(w_down, ff, ff)) {
            const dim3 grid(max_tiles, (width + 127) / 128);
            if (tile_rows == 128) return moe_pipe_launch<128, 3, true>(grid, stream, ha, ff, 1, wa, sorted, tile_expert, pair_w, ff, width, y);
            return moe_pipe_launch<32, 4, true>(grid, stream, ha, ff, 1, wa, sorted, tile_expert, pair_w, ff, width, y);
        }
        if (tile_rows != VOB_MOE_BM) return VOB_ERR_UNSUPPORTED;
        return vob_launch(moe_down_tc_kernel, dim3(max_tiles, (width + 63) / 64), dim3(128), 0, stream, ha, wa, sorted, tile_expert, pair_w,
                          width, ff, y);
    }
    VOB_DISPATCH_ELEM(code, return vob_launch(moe_down_kernel<ElemT>, dim3(max_tiles, (width + 63) / 64), dim3(256), 0, stream, (const ElemT*)h,
                                              (const ElemT*)w_down, sorted, tile_expert, pair_w, width, ff, y));
    return 0;
}

// ---------------------------------------------------------------------------------------------
// out[t, c] = sum_k y[t * top + k, c] over the token's choices in their order (k ascending) (+ shared[t, c] * sigmoid(shared_gate[t]),
// where a shared expert's result [T, width] and its gate, one number per token `ld_gate` apart, are given), in the activations' type;
// a token without choices (padding) gets zeros. Grid (tokens, ceil(width / 256)).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ idx, int top, int width, T* __restrict__ out,
                   const T* __restrict__ shared, const T* __restrict__ shared_gate, long ld_gate) {
    pdl_launch_dependents();
    pdl_wait(77);
    const int t = blockIdx.x, c = blockIdx.y * 256 + threadIdx.x;
    if (c >= width) return;
    float acc = 0.f;
    for (int k = 0; k < top; ++k)
        if (idx[(size_t)t * top + k] >= 0) acc += y[((size_t)t * top + k) * width + c];
    if (shared) {       // an expert every token uses, times the sigmoid of one number per token
        float sv = ld_f(shared + (size_t)t * width + c);
        if (shared_gate) sv *= 1.0f / (1.0f + expf(-ld_f(shared_gate + (size_t)t * ld_gate)));
        acc += sv;
    }
    st_f(out + (size_t)t * width + c, acc);
}

VOB_EXPORT int vob_moe_combine(const float* y, const int* idx, int T, int top, int width, void* out, int code, const void* shared,
                               const void* shared_gate, long ld_gate, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (top <= 0 || width <= 0 || (width + 255) / 256 > 65535) return VOB_ERR_BAD_ARG;
    VOB_DISPATCH_ELEM(code, return vob_launch(moe_combine_kernel<ElemT>, dim3(T, (width + 255) / 256), dim3(256), 0, stream, y, idx, top, width,
                                              (ElemT*)out, (const ElemT*)shared, (const ElemT*)shared_gate, ld_gate));
    return 0;
}
