// Mixture of experts: routing, the grouping of (token, choice) pairs by expert, the experts' products
// over those groups, and the weighted sum of a token's choices.
//
//   router    the router's logits z = Wr x (float products, float sums) and the routing below, in one kernel.
//   route     (the routing alone, from ready-made logits) scores = softmax(router logits) over all experts (float), or with
//             score = 1 the sigmoid of every logit by itself.  Experts form `n_groups` equal groups of
//             neighbours; a group counts by its best score, only experts of the `keep` best groups can be chosen
//             (n_groups <= 1: all can), and the `top` best of them are.  The weights are the chosen experts' scores as
//             they are, or divided by their sum (renorm).  Equal scores: the lower index wins.
//   sort      a counting sort of the A = T * top assignments by expert: sorted[] lists assignment ids (t * top + k)
//             expert by expert; tiles[] cuts every expert's run into row tiles of MOE_BM for the products.
//   gemm      for every row tile, rows of X (chosen through `sorted`) times the tile's expert's matrix.  Mode 0:
//             X = the tokens' activations (row a / top), W = [gate; up] of the expert, result h = silu(g) * u at the
//             sorted place.  Mode 1: X = h at the sorted place, W = down, result at the assignment's own row a.
//             CUDA cores, float accumulation in ascending k per output element: a row's result does not depend on
//             its place in a tile nor on what else is in the step.
//   combine   y[t] = sum_k weight[t, k] * out[t * top + k], ascending k.
//
// The bfloat16 path runs the two products on the tcgen05 product's grouped mode instead (gemm_tcgen05.cu).  For that
// the sort lays the assignments out in padded order: every expert's rows start at a multiple of the token tile's
// height, so that a token tile belongs to one expert (sort_padded: row_of[a], the row of assignment a; src_token[r], the
// token whose activations row r holds, -1 for padding; tile_group[i], the expert of tile i, -1 for unused tiles), a
// gather copies the tokens' activations into that order (padding rows zero), and combine follows row_of.
#include <math.h>
#define IK_FAMILY 2
#include "common.cuh"

namespace {

constexpr int MOE_BM = 64, MOE_BN = 64, MOE_BK = 16, MOE_TM = 4, MOE_TN = 4;

// ------------------------------------------------------------------------------------------ route
// One warp routes one token.  sc [E]: the token's router logits on entry (any memory the warp may write), its scores
// with the taken ones marked on exit; gb [n_groups]: scratch.
__device__ __forceinline__ void route_token(float* sc, float* gb, int lane, int* __restrict__ chosen, float* __restrict__ weight,
                                            int E, int top, int ng, int keep, int renorm, int score) {
    if (score == 1) {                 // every expert's score is the sigmoid of its own logit
        for (int e = lane; e < E; e += 32) sc[e] = 1.0f / (1.0f + expf(-sc[e]));
    } else {
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, sc[e]);
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) { const float p = expf(sc[e] - m); sc[e] = p; sum += p; }
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float inv = 1.0f / sum;
        for (int e = lane; e < E; e += 32) sc[e] *= inv;
    }
    __syncwarp();
    // warp-wide argmax over n values v(i) >= 0 (taken ones are marked -1); the lower index wins a tie
    auto argmax = [&](const float* v, int n) -> int {
        float bv = -2.f; int bi = 0x7fffffff;
        for (int i = lane; i < n; i += 32) if (v[i] > bv) { bv = v[i]; bi = i; }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        return bi;
    };
    if (ng) {
        const int per = E / ng;
        for (int g = lane; g < ng; g += 32) {
            float b = -1.f;
            for (int i = 0; i < per; i++) b = fmaxf(b, sc[g * per + i]);
            gb[g] = b;
        }
        __syncwarp();
        // groups that are kept are marked by -1; then the others' experts are struck out
        for (int k = 0; k < keep; k++) {
            const int g = argmax(gb, ng);
            if (lane == 0) gb[g] = -1.f;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32) if (gb[e / per] != -1.f) sc[e] = -(sc[e] + 2.f);     // struck out: -(s + 2) <= -2
        __syncwarp();
    }
    float wsum = 0.f;
    for (int k = 0; k < top; k++) {
        const int e = argmax(sc, E);
        const float s = sc[e];
        wsum += s;
        __syncwarp();
        if (lane == 0) { chosen[k] = e; weight[k] = s; sc[e] = -1.f; }
        __syncwarp();
    }
    if (renorm && lane == 0) for (int k = 0; k < top; k++) weight[k] /= wsum;
}

// From ready-made logits: one warp per token.  smem: scores [E] then group bests [n_groups] per warp.
__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, int* __restrict__ chosen, float* __restrict__ weight, int T, int E,
                 int top, int n_groups, int keep, int renorm, int score) {
    ik_pdl_wait();
    IK_AFTER_WAIT(logits);
    ik_pdl_launch_dependents();
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= T) return;
    const int ng = n_groups > 1 ? n_groups : 0;
    float* sc = sm + (size_t)warp * (E + ng);
    for (int e = lane; e < E; e += 32) sc[e] = logits[(size_t)t * E + e];
    __syncwarp();
    route_token(sc, sc + E, lane, chosen + (size_t)t * top, weight + (size_t)t * top, E, top, ng, keep, renorm, score);
}

// The router's product and the routing in one kernel.  A block takes TOK tokens: their activations go to shared memory
// as floats; warp w forms the logits of experts w, w + warps, ...: its lanes stride over K four elements at a time (a weight
// row is read once per block, 512 bytes per warp and load), each lane keeps one partial sum per token, added over its k in
// ascending order and then across the lanes by a fixed tree, so a logit depends on its token and expert alone.  Then a warp
// routes each token.  Everything in float.  K a multiple of 4.  smem: x [TOK][K], logits [TOK][E + n_groups].
// Few tokens (decode): one token a block and 32 warps, so that a token's experts are spread over many warps.
template <int TOK, int THREADS, typename TX>
__global__ void __launch_bounds__(THREADS)
moe_router_kernel(const TX* __restrict__ x, const float* __restrict__ wr, int* __restrict__ chosen, float* __restrict__ weight,
                  int T, int K, int E, int top, int n_groups, int keep, int renorm, int score, int ldx) {
    ik_pdl_wait();
    IK_AFTER_WAIT(x);
    ik_pdl_launch_dependents();
    extern __shared__ __align__(16) float sm[];
    const int ng = n_groups > 1 ? n_groups : 0;
    float* xs = sm;                                   // [TOK][K]
    float* lg = sm + (size_t)TOK * K;                 // [TOK][E + ng]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * TOK;
    constexpr int V = 16 / (int)sizeof(TX);            // activations per 16-byte load
    if (K % V == 0 && ldx % V == 0 && ((uintptr_t)x % 16) == 0) {
        const int KV = K / V;
        #pragma unroll 4
        for (int idx = threadIdx.x; idx < TOK * KV; idx += THREADS) {
            const int i = idx / KV, kv = idx - i * KV;
            float* dst = xs + (size_t)i * K + kv * V;
            if (t0 + i < T) {
                const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)(t0 + i) * ldx + kv * V);
                const TX* e = reinterpret_cast<const TX*>(&raw);
                #pragma unroll
                for (int j = 0; j < V; j++) dst[j] = ik_ld(e, j);
            } else {
                #pragma unroll
                for (int j = 0; j < V; j++) dst[j] = 0.f;
            }
        }
    } else {
        for (int idx = threadIdx.x; idx < TOK * K; idx += THREADS) {
            const int i = idx / K, k = idx - i * K;
            xs[idx] = t0 + i < T ? ik_ld(x, (size_t)(t0 + i) * ldx + k) : 0.f;
        }
    }
    __syncthreads();
    const int K4 = K >> 2;
    const float4* xs4 = reinterpret_cast<const float4*>(xs);
    // four experts a pass: an activation read from shared memory serves four products
    constexpr int EB = 4, NW = THREADS / 32;
    for (int e0 = warp; e0 < E; e0 += NW * EB) {
        const float4* w4[EB];
        #pragma unroll
        for (int j = 0; j < EB; j++) w4[j] = reinterpret_cast<const float4*>(wr + (size_t)min(e0 + j * NW, E - 1) * K);
        float acc[EB][TOK];
        #pragma unroll
        for (int j = 0; j < EB; j++)
            #pragma unroll
            for (int i = 0; i < TOK; i++) acc[j][i] = 0.f;
        #pragma unroll 2
        for (int k = lane; k < K4; k += 32) {
            float4 wv[EB];
            #pragma unroll
            for (int j = 0; j < EB; j++) wv[j] = (j == 0 || e0 + j * NW < E) ? __ldg(w4[j] + k) : make_float4(0.f, 0.f, 0.f, 0.f);
            #pragma unroll
            for (int i = 0; i < TOK; i++) {
                const float4 xv = xs4[i * K4 + k];
                #pragma unroll
                for (int j = 0; j < EB; j++)
                    acc[j][i] = fmaf(xv.w, wv[j].w, fmaf(xv.z, wv[j].z, fmaf(xv.y, wv[j].y, fmaf(xv.x, wv[j].x, acc[j][i]))));
            }
        }
        #pragma unroll
        for (int j = 0; j < EB; j++) {
            const int e = e0 + j * NW;
            if (e >= E) break;
            #pragma unroll
            for (int i = 0; i < TOK; i++) {
                float v = acc[j][i];
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0) lg[i * (E + ng) + e] = v;
            }
        }
    }
    __syncthreads();
    for (int i = warp; i < TOK; i += THREADS / 32) {
        const int t = t0 + i;
        if (t >= T) continue;
        float* sc = lg + (size_t)i * (E + ng);
        route_token(sc, sc + E, lane, chosen + (size_t)t * top, weight + (size_t)t * top, E, top, ng, keep, renorm, score);
    }
}

// ------------------------------------------------------------------------------------------ sort
// One block.  offsets [E + 1], sorted [A], tiles [max_tiles][2] = (expert, first sorted place), n_tiles [1].
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ chosen, int* __restrict__ offsets, int* __restrict__ sorted, int* __restrict__ tiles,
                int* __restrict__ n_tiles, int A, int E, int max_tiles) {
    ik_pdl_wait();
    IK_AFTER_WAIT(chosen);
    ik_pdl_launch_dependents();
    extern __shared__ int cnt[];         // [E] counts, then [E] cursors
    int* cur = cnt + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int a = threadIdx.x; a < A; a += blockDim.x) {
        const int e = chosen[a];
        if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, nt = 0;
        for (int e = 0; e < E; e++) {
            offsets[e] = at;
            cur[e] = at;
            for (int r = 0; r < cnt[e] && nt < max_tiles; r += MOE_BM) { tiles[2 * nt] = e; tiles[2 * nt + 1] = at + r; nt++; }
            at += cnt[e];
        }
        offsets[E] = at;
        *n_tiles = nt;
    }
    __syncthreads();
    for (int a = threadIdx.x; a < A; a += blockDim.x) {
        const int e = chosen[a];
        if (e >= 0 && e < E) sorted[atomicAdd(&cur[e], 1)] = a;
    }
}

// ------------------------------------------------------------------------------------------ products
template <typename TX, typename TW, typename TY, int MODE>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const TX* __restrict__ X, const TW* __restrict__ W, TY* __restrict__ Y, const int* __restrict__ offsets,
                const int* __restrict__ sorted, const int* __restrict__ tiles, const int* __restrict__ n_tiles, int top,
                int N, int K, int ldx, int ldy, const float* __restrict__ row_scale, int act) {
    ik_pdl_wait();
    IK_AFTER_WAIT(X);
    IK_AFTER_WAIT(offsets);
    IK_AFTER_WAIT(sorted);
    IK_AFTER_WAIT(tiles);
    IK_AFTER_WAIT(n_tiles);
    ik_pdl_launch_dependents();
    if ((int)blockIdx.y >= *n_tiles) return;
    constexpr int NW = MODE == 0 ? 2 : 1;                  // mode 0 carries gate and up of the same columns
    __shared__ float xs[MOE_BK][MOE_BM + 1];
    __shared__ float ws[NW][MOE_BK][MOE_BN + 1];
    __shared__ int src_row[MOE_BM], dst_row[MOE_BM];
    __shared__ float in_scale[MOE_BM];
    const int e = tiles[2 * blockIdx.y], p0 = tiles[2 * blockIdx.y + 1];
    const int rows = min(MOE_BM, offsets[e + 1] - p0);
    const int n0 = blockIdx.x * MOE_BN;
    // expert e's matrix: mode 0 [2N, K] (gate j in row 2j, up j in row 2j + 1), mode 1 [N, K]
    const TW* We = W + (size_t)e * (MODE == 0 ? 2 : 1) * N * K;
    if (threadIdx.x < MOE_BM) {
        const int r = threadIdx.x;
        const int a = r < rows ? sorted[p0 + r] : -1;
        src_row[r] = a < 0 ? -1 : (MODE != 1 ? a / top : p0 + r);
        dst_row[r] = a < 0 ? -1 : (MODE != 1 ? p0 + r : a);
        in_scale[r] = (a >= 0 && row_scale) ? row_scale[a] : 1.0f;
    }
    __syncthreads();
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc[NW][MOE_TM][MOE_TN];
    #pragma unroll
    for (int w = 0; w < NW; w++)
        #pragma unroll
        for (int i = 0; i < MOE_TM; i++)
            #pragma unroll
            for (int j = 0; j < MOE_TN; j++) acc[w][i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += MOE_BK) {
        #pragma unroll
        for (int l = 0; l < 4; l++) {
            const int idx = threadIdx.x + l * 256;
            const int r = idx / MOE_BK, c = idx % MOE_BK, k = k0 + c;
            const int sr = src_row[r];
            xs[c][r] = (sr >= 0 && k < K) ? (MODE == 2 ? ik_round_to<TX>(ik_ld(X, (size_t)sr * ldx + k) * in_scale[r]) : ik_ld(X, (size_t)sr * ldx + k)) : 0.f;
            #pragma unroll
            for (int w = 0; w < NW; w++)
                ws[w][c][r] = (n0 + r < N && k < K) ? ik_ld(We, ((size_t)(MODE == 0 ? 2 : 1) * (n0 + r) + w) * K + k) : 0.f;
        }
        __syncthreads();
        #pragma unroll
        for (int kk = 0; kk < MOE_BK; kk++) {
            float a[MOE_TM];
            #pragma unroll
            for (int i = 0; i < MOE_TM; i++) a[i] = xs[kk][ty * MOE_TM + i];
            #pragma unroll
            for (int w = 0; w < NW; w++) {
                float b[MOE_TN];
                #pragma unroll
                for (int j = 0; j < MOE_TN; j++) b[j] = ws[w][kk][tx + 16 * j];
                #pragma unroll
                for (int i = 0; i < MOE_TM; i++)
                    #pragma unroll
                    for (int j = 0; j < MOE_TN; j++) acc[w][i][j] = fmaf(a[i], b[j], acc[w][i][j]);
            }
        }
        __syncthreads();
    }
    #pragma unroll
    for (int i = 0; i < MOE_TM; i++) {
        const int dr = dst_row[ty * MOE_TM + i];
        if (dr < 0) continue;
        #pragma unroll
        for (int j = 0; j < MOE_TN; j++) {
            const int n = n0 + tx + 16 * j;
            if (n >= N) continue;
            const float v = MODE == 0 ? ik_swiglu(acc[0][i][j], acc[NW - 1][i][j]) : MODE == 2 ? ik_plain_act_value(acc[0][i][j], act) : acc[0][i][j];
            ik_st(Y, (size_t)dr * ldy + n, v);
        }
    }
}

// ------------------------------------------------------------------------------------------ padded order
// One block.  row_of [A], src_token [n_tiles * bn], tile_group [n_tiles].
__global__ void __launch_bounds__(1024)
moe_sort_padded_kernel(const int* __restrict__ chosen, int* __restrict__ row_of, int* __restrict__ src_token,
                       int* __restrict__ tile_group, int A, int E, int top, int bn, int n_tiles, int* __restrict__ src_assign) {
    ik_pdl_wait();
    IK_AFTER_WAIT(chosen);
    ik_pdl_launch_dependents();
    extern __shared__ int cnt[];         // [E] counts, then [E] cursors
    int* cur = cnt + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    for (int r = threadIdx.x; r < n_tiles * bn; r += blockDim.x) src_token[r] = -1;
    __syncthreads();
    for (int a = threadIdx.x; a < A; a += blockDim.x) {
        const int e = chosen[a];
        if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int nt = 0;
        for (int e = 0; e < E; e++) {
            cur[e] = nt * bn;
            for (int r = 0; r < cnt[e] && nt < n_tiles; r += bn) tile_group[nt++] = e;
        }
        for (; nt < n_tiles; nt++) tile_group[nt] = -1;
    }
    __syncthreads();
    for (int a = threadIdx.x; a < A; a += blockDim.x) {
        const int e = chosen[a];
        if (e < 0 || e >= E) { row_of[a] = 0; continue; }
        const int r = atomicAdd(&cur[e], 1);
        row_of[a] = r;
        if (r < n_tiles * bn) {
            src_token[r] = a / top;
            if (src_assign) src_assign[r] = a;            // (read only where src_token is not -1)
        }
    }
}

// xp[r, :] = x[src_token[r], :], zeros where src_token[r] < 0; rows of d bfloat16, d a multiple of 8
__global__ void moe_gather_kernel(const uint4* __restrict__ x, const int* __restrict__ src_token, uint4* __restrict__ xp,
                                  int rows, int d8) {
    ik_pdl_wait();
    IK_AFTER_WAIT(x);
    IK_AFTER_WAIT(src_token);
    ik_pdl_launch_dependents();
    const size_t total = (size_t)rows * d8, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const size_t r = idx / d8;
        const int c = (int)(idx - r * d8), t = src_token[r];
        xp[idx] = t >= 0 ? x[(size_t)t * d8 + c] : make_uint4(0u, 0u, 0u, 0u);
    }
}

// The same with every row multiplied by the weight of its assignment (in float, rounded once): xp[r, :] = x[src_token[r], :] *
// weight[src_assign[r]].
__global__ void moe_gather_scaled_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ src_token,
                                         const int* __restrict__ src_assign, const float* __restrict__ weight,
                                         __nv_bfloat16* __restrict__ xp, int rows, int d) {
    ik_pdl_wait();
    IK_AFTER_WAIT(x);
    IK_AFTER_WAIT(src_token);
    IK_AFTER_WAIT(src_assign);
    IK_AFTER_WAIT(weight);
    ik_pdl_launch_dependents();
    const int d4 = d / 4;
    const size_t total = (size_t)rows * d4, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const size_t r = idx / d4;
        const int c = (int)(idx - r * d4) * 4, t = src_token[r];
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t >= 0) {
            const float w = weight[src_assign[r]];
            v = ik_ld4(x, (size_t)t * d + c);
            v.x *= w; v.y *= w; v.z *= w; v.w *= w;
        }
        ik_st4(xp, r * d + c, v);
    }
}

// ------------------------------------------------------------------------------------------ combine
__global__ void moe_combine_kernel(const float* __restrict__ parts, const float* __restrict__ weight, const int* __restrict__ row_of,
                                   float* __restrict__ y, int T, int top, int d) {
    ik_pdl_wait();
    IK_AFTER_WAIT(parts);
    IK_AFTER_WAIT(weight);
    IK_AFTER_WAIT(row_of);
    ik_pdl_launch_dependents();
    const size_t total = (size_t)T * d, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const size_t t = idx / d;
        const int i = (int)(idx - t * d);
        float acc = 0.f;
        for (int k = 0; k < top; k++) acc = fmaf(weight ? weight[t * top + k] : 1.0f, parts[(size_t)(row_of ? row_of[t * top + k] : t * top + k) * d + i], acc);
        y[idx] = acc;
    }
}

template <int MODE>
int launch_gemm(const void* X, int x_dtype, const void* W, int w_dtype, void* Y, int y_dtype, const int* offsets,
                const int* sorted, const int* tiles, const int* n_tiles, int max_tiles, int top, int N, int K, int ldx,
                int ldy, const float* row_scale, int act, cudaStream_t stream) {
    dim3 grid((N + MOE_BN - 1) / MOE_BN, max_tiles);
#define IK_MOE(TX, TW, TY) \
    IK_RETURN_IF_ERROR(ik_launch(moe_gemm_kernel<TX, TW, TY, MODE>, grid, 256, 0, stream, (const TX*)X, (const TW*)W, (TY*)Y, offsets, sorted, tiles, n_tiles, top, N, K, ldx, ldy, row_scale, act))
    const int code = x_dtype * 4 + w_dtype * 2 + y_dtype;
    switch (code) {
        case 0: IK_MOE(float, float, float); break;
        case 2: IK_MOE(float, __nv_bfloat16, float); break;
        case 6: IK_MOE(__nv_bfloat16, __nv_bfloat16, float); break;
        case 7: IK_MOE(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16); break;
        default: return IK_UNSUPPORTED;
    }
#undef IK_MOE
    IK_LAUNCH_STATUS();
}

}  // namespace

IK_EXPORT int ik_moe_tile_rows() { return MOE_BM; }

IK_EXPORT int ik_moe_route(const float* logits, int* chosen, float* weight, int T, int E, int top, int n_groups, int keep,
                           int renorm, int score, cudaStream_t stream) {
    if (T < 0 || E <= 0 || top <= 0 || top > E) return IK_BAD_ARGUMENT;
    if (n_groups > 1 && (E % n_groups || keep <= 0 || keep > n_groups || top > keep * (E / n_groups))) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    const size_t smem = 4 * (size_t)(E + (n_groups > 1 ? n_groups : 0)) * sizeof(float);
    if (smem > 48 * 1024) return IK_UNSUPPORTED;
    IK_RETURN_IF_ERROR(ik_launch(moe_route_kernel, (T + 3) / 4, 128, smem, stream, logits, chosen, weight, T, E, top, n_groups, keep, renorm, score));
    IK_LAUNCH_STATUS();
}

// x [T, K] (float or bfloat16, rows ldx apart), wr [E, K] float -> chosen, weight [T, top]
IK_EXPORT int ik_moe_router(const void* x, int x_dtype, const float* wr, int* chosen, float* weight, int T, int K, int E, int top,
                            int n_groups, int keep, int renorm, int score, int ldx, cudaStream_t stream) {
    if (T < 0 || E <= 0 || K <= 0 || top <= 0 || top > E || ldx < K) return IK_BAD_ARGUMENT;
    if (n_groups > 1 && (E % n_groups || keep <= 0 || keep > n_groups || top > keep * (E / n_groups))) return IK_BAD_ARGUMENT;
    if (K % 4 || ((uintptr_t)wr % 16)) return IK_UNSUPPORTED;
    if (T == 0) return IK_OK;
    const int ng = n_groups > 1 ? n_groups : 0;
    // few tokens (decode): a block per token, so that the step's tokens spread over the SMs; else eight tokens a block,
    // or four where eight rows of activations would leave room for one block per SM only
    const int tok = T <= 64 ? 1 : K <= 2048 ? 8 : K <= 6144 ? 4 : 1;
    const size_t smem = ((size_t)tok * K + (size_t)tok * (E + ng)) * sizeof(float);
    if (smem > 200 * 1024) return IK_UNSUPPORTED;
#define IK_ROUTER(TOK, TX)                                                                                                 \
    {                                                                                                                      \
        constexpr int THREADS = TOK == 1 ? 1024 : 256;                                                                     \
        auto kern = moe_router_kernel<TOK, THREADS, TX>;                                                                          \
        if (smem > 48 * 1024) {                                                                                            \
            cudaError_t e0 = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
            if (e0 != cudaSuccess) return (int)e0;                                                                         \
        }                                                                                                                  \
        IK_RETURN_IF_ERROR(ik_launch(kern, (T + TOK - 1) / TOK, THREADS, smem, stream, (const TX*)x, wr, chosen, weight, T, K, E, top, \
                                     n_groups, keep, renorm, score, ldx));                                                        \
    }
    if (x_dtype == IK_F32) { if (tok == 1) IK_ROUTER(1, float) else if (tok == 4) IK_ROUTER(4, float) else IK_ROUTER(8, float) }
    else if (x_dtype == IK_BF16) { if (tok == 1) IK_ROUTER(1, __nv_bfloat16) else if (tok == 4) IK_ROUTER(4, __nv_bfloat16) else IK_ROUTER(8, __nv_bfloat16) }
    else return IK_BAD_ARGUMENT;
#undef IK_ROUTER
    IK_LAUNCH_STATUS();
}

IK_EXPORT int ik_moe_sort(const int* chosen, int* offsets, int* sorted, int* tiles, int* n_tiles, int A, int E, int max_tiles,
                          cudaStream_t stream) {
    if (A < 0 || E <= 0 || max_tiles < 0) return IK_BAD_ARGUMENT;
    if ((size_t)2 * E * sizeof(int) > 48 * 1024) return IK_UNSUPPORTED;
    IK_RETURN_IF_ERROR(ik_launch(moe_sort_kernel, 1, 1024, (size_t)2 * E * sizeof(int), stream, chosen, offsets, sorted, tiles, n_tiles, A, E, max_tiles));
    IK_LAUNCH_STATUS();
}

// mode 2: X [T, K] tokens, each row times row_scale[assignment] (rounded to X's type) as it is read, W [E, N, K], Y [A, N] =
// act(product) at sorted places (act 0: relu(x)^2, 1: gelu, tanh form).
// mode 0: X [T, K] tokens, W [E, 2N, K] (gate j, up j in rows 2j, 2j + 1), Y [A, N] = silu(gate) * up at sorted places.  mode 1: X [A, K] at sorted
// places, W [E, N, K], Y [A, N] at the assignments' rows.
IK_EXPORT int ik_moe_gemm(int mode, const void* X, int x_dtype, const void* W, int w_dtype, void* Y, int y_dtype,
                          const int* offsets, const int* sorted, const int* tiles, const int* n_tiles, int max_tiles, int top,
                          int N, int K, int ldx, int ldy, const float* row_scale, int act, cudaStream_t stream) {
    if (max_tiles < 0 || top <= 0 || N <= 0 || K <= 0 || ldx < K || ldy < N || max_tiles > 65535) return IK_BAD_ARGUMENT;
    if (max_tiles == 0) return IK_OK;
    if (mode == 0) return launch_gemm<0>(X, x_dtype, W, w_dtype, Y, y_dtype, offsets, sorted, tiles, n_tiles, max_tiles, top, N, K, ldx, ldy, nullptr, 0, stream);
    if (mode == 1) return launch_gemm<1>(X, x_dtype, W, w_dtype, Y, y_dtype, offsets, sorted, tiles, n_tiles, max_tiles, top, N, K, ldx, ldy, nullptr, 0, stream);
    if (mode == 2 && act >= 0 && act <= 1)
        return launch_gemm<2>(X, x_dtype, W, w_dtype, Y, y_dtype, offsets, sorted, tiles, n_tiles, max_tiles, top, N, K, ldx, ldy, row_scale, act, stream);
    return IK_BAD_ARGUMENT;
}

IK_EXPORT int ik_moe_sort_padded(const int* chosen, int* row_of, int* src_token, int* tile_group, int A, int E, int top, int bn,
                                 int n_tiles, int* src_assign, cudaStream_t stream) {
    if (A < 0 || E <= 0 || top <= 0 || bn <= 0 || n_tiles < 0 || n_tiles < (A / bn + E < A ? A / bn + E : A)) return IK_BAD_ARGUMENT;
    if ((size_t)2 * E * sizeof(int) > 48 * 1024) return IK_UNSUPPORTED;
    IK_RETURN_IF_ERROR(ik_launch(moe_sort_padded_kernel, 1, 1024, (size_t)2 * E * sizeof(int), stream, chosen, row_of, src_token, tile_group, A, E,
                                 top, bn, n_tiles, src_assign));
    IK_LAUNCH_STATUS();
}

IK_EXPORT int ik_moe_gather(const void* x, const int* src_token, void* xp, int rows, int d, cudaStream_t stream) {
    if (rows < 0 || d <= 0 || d % 8 || ((uintptr_t)x % 16) || ((uintptr_t)xp % 16)) return IK_BAD_ARGUMENT;
    if (rows == 0) return IK_OK;
    const size_t total = (size_t)rows * (d / 8), want = (total + 255) / 256, cap = (size_t)ik_sm_count() * 16;
    IK_RETURN_IF_ERROR(ik_launch(moe_gather_kernel, (int)(want < cap ? want : cap), 256, 0, stream, (const uint4*)x, src_token, (uint4*)xp, rows, d / 8));
    IK_LAUNCH_STATUS();
}

IK_EXPORT int ik_moe_gather_scaled(const void* x, const int* src_token, const int* src_assign, const float* weight, void* xp, int rows,
                                   int d, cudaStream_t stream) {
    if (rows < 0 || d <= 0 || d % 8 || ((uintptr_t)x % 16) || ((uintptr_t)xp % 16) || !src_assign || !weight) return IK_BAD_ARGUMENT;
    if (rows == 0) return IK_OK;
    const size_t total = (size_t)rows * (d / 4), want = (total + 255) / 256, cap = (size_t)ik_sm_count() * 16;
    IK_RETURN_IF_ERROR(ik_launch(moe_gather_scaled_kernel, (int)(want < cap ? want : cap), 256, 0, stream, (const __nv_bfloat16*)x, src_token,
                                 src_assign, weight, (__nv_bfloat16*)xp, rows, d));
    IK_LAUNCH_STATUS();
}

// row_of: where assignment a's result lies in `parts` (nullptr: at row a); weight nullptr: every weight is 1
IK_EXPORT int ik_moe_combine(const float* parts, const float* weight, const int* row_of, float* y, int T, int top, int d, cudaStream_t stream) {
    if (T < 0 || top <= 0 || d <= 0) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    const size_t total = (size_t)T * d, want = (total + 255) / 256, cap = (size_t)ik_sm_count() * 16;
    IK_RETURN_IF_ERROR(ik_launch(moe_combine_kernel, (int)(want < cap ? want : cap), 256, 0, stream, parts, weight, row_of, y, T, top, d));
    IK_LAUNCH_STATUS();
}
