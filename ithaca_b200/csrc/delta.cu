// The gated delta rule: a mixer whose state is a matrix per head that is decayed, corrected towards the current value
// along the current key, and read out with the current query.
//
// Per value head h (its query and key come from head h / (H / G) of G query/key heads), with a decay g and a step b per
// token and head:  S <- g S;  u = b (v - S^T k);  S <- S + k u^T;  o = S^T q   (S is dk x dv, zero before the first token).
// Both sums over rows are taken from the state as it was before the token: with A = S_old^T k and B = S_old^T q,
// u = b (v - g A), S_new = g S_old + k u^T and o = g B + (k . q) u.  One pass over a lane's rows and one exchange
// between the lanes of a column per token.
//
// The step's tokens are token-major as everywhere: sequence n brings tokens cu_seqlens[n] .. cu_seqlens[n + 1] - 1 at
// positions kv_lens[n] - count .. kv_lens[n] - 1, its state lies in slot slots[n] as [heads, dv, dk] (the rows of a column
// side by side), kept twice by the parity of the
// position it belongs to (a step reads the copy of parity (first - 1) & 1 and writes that of (last) & 1, so a decode
// step never overwrites what it read and may be run again).  Everything here is float: unit norms, steps, decays
// (formed in double and rounded once: a decay's error is multiplied into the state at every token), states, sums.
#include "common.cuh"

__device__ __forceinline__ void ik_cp_async4(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void ik_cp_async16(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void ik_cp_async_wait_all() { asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory"); }

// ------------------------------------------------------------------ unit vectors, steps and decays
// One block per token.  u [T, ldu] holds q (G heads of dk) from q_off and k from k_off, behind their convolution and
// activation: every head becomes x / sqrt(sum x^2 + unit_eps), q also times q_mult, in place (one warp per head, lanes in
// index order, then the shuffle tree).  p [T, ldp] holds the step's and the decay's projections, one column per head from
// b_off and a_off: bg[t, 0, h] = sigmoid(p_b), bg[t, 1, h] = exp(-exp(A_log[h]) * softplus(p_a + dt_bias[h])).  a_off < 0:
// the decays are formed elsewhere (a decay per key channel) and bg[t, 1, :] is left alone.
__global__ void __launch_bounds__(128)
delta_prepare_kernel(float* __restrict__ u, int ldu, int q_off, int k_off, const float* __restrict__ p, int ldp, int b_off, int a_off,
                     const float* __restrict__ A_log, const float* __restrict__ dt_bias, float* __restrict__ bg, int G, int dk,
                     int H, float q_mult, float unit_eps) {
    ik_pdl_wait();
    IK_AFTER_WAIT(u);
    IK_AFTER_WAIT(p);
    ik_pdl_launch_dependents();
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    for (int head = threadIdx.x >> 5; head < 2 * G; head += 4) {
        float* x = u + (size_t)t * ldu + (head < G ? q_off + head * dk : k_off + (head - G) * dk);
        float ss = 0.f;
        for (int i = lane; i < dk; i += 32) ss = fmaf(x[i], x[i], ss);
        #pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float r = (1.0f / sqrtf(ss + unit_eps)) * (head < G ? q_mult : 1.0f);
        for (int i = lane; i < dk; i += 32) x[i] *= r;
    }
    for (int h = threadIdx.x; h < H; h += 128) {
        const float* row = p + (size_t)t * ldp;
        bg[((size_t)t * 2) * H + h] = 1.0f / (1.0f + expf(-row[b_off + h]));
        if (a_off < 0) continue;
        const double z = (double)row[a_off + h] + (double)dt_bias[h];
        const double sp = z > 30.0 ? z : log1p(exp(z));
        bg[((size_t)t * 2 + 1) * H + h] = (float)exp(-exp((double)A_log[h]) * sp);
    }
}

IK_EXPORT int ik_delta_prepare(float* u, int ldu, int q_off, int k_off, const float* p, int ldp, int b_off, int a_off,
                               const float* A_log, const float* dt_bias, float* bg, int T, int G, int dk, int H, float q_mult,
                               float unit_eps, cudaStream_t stream) {
    if (T < 0 || G <= 0 || dk <= 0 || H <= 0 || !u || !p || (a_off >= 0 && (!A_log || !dt_bias)) || !bg) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    IK_RETURN_IF_ERROR(ik_launch(delta_prepare_kernel, T, 128, 0, stream, u, ldu, q_off, k_off, p, ldp, b_off, a_off, A_log, dt_bias, bg,
                                 G, dk, H, q_mult, unit_eps));
    IK_LAUNCH_STATUS();
}

// ------------------------------------------------------------------ the rule
// A column of the state is a recurrence of its own (u, the update and the read-out of column j use column j only), so the
// work is cut by columns and no block-wide exchange is needed.  L lanes of a warp share one column, each keeping 16 of its
// rows in registers (L = 1, 2, .. 32 for up to 16 L rows), the warp therefore holds 32 / L neighbouring columns, and up to
// eight warps of a block hold neighbouring groups of columns of one head and one sequence.  Lane `part` owns the rows
// 4 f .. 4 f + 3 of the four groups f = part, L + part, 2 L + part, 3 L + part: the lanes of a column then read
// consecutive 16-byte words of q and k from shared memory and of the state from memory.  Rows beyond dk are staged as
// zeros and stay zero in the state.
//
// Tokens come through shared memory in tiles of TT (q and k padded to 16 L rows, the block's values of v, the step, the
// decay and k . q, which a warp forms once per token of a tile for all columns), the next tile on its way (cp.async)
// while one is computed; there are two block barriers per tile and none per token.  Per token a lane forms its rows' share
// of A and B in four running sums each, the shares of a column meet by shuffles between neighbouring lanes, and every lane
// updates its rows.  What is computed for a token depends on its sequence's earlier tokens only, not on where steps or
// tiles begin, and the sums run in the same order for a prompt and for a single token.  The token loop is unrolled by four
// so that a token's loads and the read-out of the one before overlap with the chain S -> A -> u -> S.
template <int L, int R>
__global__ void __launch_bounds__(256)
delta_rule_kernel(const float* __restrict__ u, int ldu, int q_off, int k_off, int v_off, const float* __restrict__ bg,
                  float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ cu_seqlens,
                  const int* __restrict__ kv_lens, float* __restrict__ out, int H, int G, int dk, int dv, int TT, int W, int vec) {
    extern __shared__ __align__(16) float sm[];          // [2][TT][W]: q, k (16 L each), the block's v, step, decay, k . q
    ik_pdl_wait();
    IK_AFTER_WAIT(u);
    IK_AFTER_WAIT(bg);
    IK_AFTER_WAIT(slots);
    IK_AFTER_WAIT(cu_seqlens);
    IK_AFTER_WAIT(kv_lens);
    ik_pdl_launch_dependents();
    constexpr int LR = L * R, CPW = 32 / L, NF = R / 4;
    const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, nthreads = blockDim.x, warp = tid >> 5, lane = tid & 31;
    const int nwarps = nthreads >> 5, CB = nwarps * CPW;
    const int part = lane % L, jj = lane / L;
    const int col0 = blockIdx.z * CB, col = col0 + warp * CPW + jj;
    const bool live = col < dv;
    const int ccol = live ? col : dv - 1;
    const int per_tile = TT * W;
    const int lo = cu_seqlens[b], hi = cu_seqlens[b + 1], end = kv_lens[b], start = end - (hi - lo);
    if (hi <= lo) return;
    const int kvh = h / (H / G);
    const size_t per = (size_t)H * dk * dv;
    const float* st_in = state + ((size_t)slots[b] * 2 + ((start - 1) & 1)) * per + ((size_t)h * dv + ccol) * dk;
    float* st_out = state + ((size_t)slots[b] * 2 + ((end - 1) & 1)) * per + ((size_t)h * dv + ccol) * dk;
    float S[R];
    #pragma unroll
    for (int r = 0; r < R; r++) {
        const int i = ((r >> 2) * L + part) * 4 + (r & 3);
        S[r] = (i < dk && start > 0) ? st_in[i] : 0.f;
    }
    auto stage = [&](int t0, int buf) {                  // a warp brings whole tokens: every warp does the same share
        const int n = min(TT, hi - t0);
        for (int tt = warp; tt < n; tt += nwarps) {
            const float* row = u + (size_t)(t0 + tt) * ldu;
            float* dst = sm + buf * per_tile + tt * W;
            const float* qs = row + q_off + kvh * dk;
            const float* ks = row + k_off + kvh * dk;
            if (vec) {                                   // dk a multiple of 4 and every row of q and k on a 16-byte boundary
                for (int f = lane; f < 2 * (LR / 4); f += 32) {
                    const int g4 = f < LR / 4 ? f : f - LR / 4;
                    const float* src = (f < LR / 4 ? qs : ks) + 4 * g4;
                    if (4 * g4 < dk) ik_cp_async16(dst + 4 * f, src);
                    else *reinterpret_cast<float4*>(dst + 4 * f) = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            } else {
                for (int w = lane; w < 2 * LR; w += 32) {
                    const int i = w < LR ? w : w - LR;
                    if (i < dk) ik_cp_async4(dst + w, (w < LR ? qs : ks) + i);
                    else dst[w] = 0.f;
                }
            }
            for (int w = lane; w < CB + 2; w += 32) {
                if (w < CB) {
                    if (col0 + w < dv) ik_cp_async4(dst + 2 * LR + w, row + v_off + h * dv + col0 + w);
                    else dst[2 * LR + w] = 0.f;
                } else {
                    ik_cp_async4(dst + 2 * LR + w, bg + ((size_t)(t0 + tt) * 2 + (w - CB)) * H + h);
                }
            }
        }
    };
    stage(lo, 0);
    ik_cp_async_wait_all();
    __syncthreads();
    int buf = 0;
    for (int t0 = lo; t0 < hi; t0 += TT, buf ^= 1) {
        if (t0 + TT < hi) stage(t0 + TT, buf ^ 1);
        const int n_here = min(TT, hi - t0);
        for (int tt = warp; tt < n_here; tt += nwarps) {        // k . q of the tile's tokens, lanes in index order, then the tree
            float* x = sm + buf * per_tile + tt * W;
            float c = 0.f;
            for (int i = lane; i < LR; i += 32) c = fmaf(x[i], x[LR + i], c);
            #pragma unroll
            for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
            if (lane == 0) x[2 * LR + CB + 2] = c;
        }
        __syncthreads();
        #pragma unroll 4
        for (int tt = 0; tt < n_here; tt++) {
            const float* x = sm + buf * per_tile + tt * W;
            const float4* q4 = reinterpret_cast<const float4*>(x);
            const float4* k4 = reinterpret_cast<const float4*>(x + LR);
            const float* tail = x + 2 * LR;
            const float v = tail[warp * CPW + jj], beta = tail[CB], g = tail[CB + 1], kq = tail[CB + 2];
            float4 kk[NF];
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, b0 = 0.f, b1 = 0.f, b2 = 0.f, b3 = 0.f;
            #pragma unroll
            for (int f = 0; f < NF; f++) {
                kk[f] = k4[f * L + part];
                const float4 qq = q4[f * L + part];
                a0 = fmaf(S[4 * f], kk[f].x, a0);     b0 = fmaf(S[4 * f], qq.x, b0);
                a1 = fmaf(S[4 * f + 1], kk[f].y, a1); b1 = fmaf(S[4 * f + 1], qq.y, b1);
                a2 = fmaf(S[4 * f + 2], kk[f].z, a2); b2 = fmaf(S[4 * f + 2], qq.z, b2);
                a3 = fmaf(S[4 * f + 3], kk[f].w, a3); b3 = fmaf(S[4 * f + 3], qq.w, b3);
            }
            float A = (a0 + a1) + (a2 + a3), B = (b0 + b1) + (b2 + b3);
            #pragma unroll
            for (int o = 1; o < L; o <<= 1) {
                A += __shfl_xor_sync(0xffffffffu, A, o);
                B += __shfl_xor_sync(0xffffffffu, B, o);
            }
            const float un = beta * (v - g * A);
            #pragma unroll
            for (int f = 0; f < NF; f++) {
                S[4 * f] = fmaf(g, S[4 * f], kk[f].x * un);
                S[4 * f + 1] = fmaf(g, S[4 * f + 1], kk[f].y * un);
                S[4 * f + 2] = fmaf(g, S[4 * f + 2], kk[f].z * un);
                S[4 * f + 3] = fmaf(g, S[4 * f + 3], kk[f].w * un);
            }
            if (part == 0 && live) out[(size_t)(t0 + tt) * H * dv + h * dv + col] = fmaf(g, B, kq * un);
        }
        ik_cp_async_wait_all();
        __syncthreads();
    }
    if (live) {
        #pragma unroll
        for (int r = 0; r < R; r++) {
            const int i = ((r >> 2) * L + part) * 4 + (r & 3);
            if (i < dk) st_out[i] = S[r];
        }
    }
}

template <int L, int R>
static cudaError_t ik_delta_rule_launch(dim3 grid, int threads, size_t smem, cudaStream_t stream, const float* u, int ldu, int q_off, int k_off,
                                        int v_off, const float* bg, float* state, const int* slots, const int* cu_seqlens,
                                        const int* kv_lens, float* out, int H, int G, int dk, int dv, int TT, int W, int vec) {
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        const cudaError_t e = cudaFuncSetAttribute(delta_rule_kernel<L, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        if (e != cudaSuccess) return e;
        raised = true;
    }
    return ik_launch(delta_rule_kernel<L, R>, grid, dim3(threads), smem, stream, u, ldu, q_off, k_off, v_off, bg, state, slots, cu_seqlens,
                     kv_lens, out, H, G, dk, dv, TT, W, vec);
}

IK_EXPORT int ik_delta_rule(const float* u, int ldu, int q_off, int k_off, int v_off, const float* bg, float* state, const int* slots,
                            const int* cu_seqlens, const int* kv_lens, float* out, int T, int B, int H, int G, int dk, int dv,
                            int one_token_each, cudaStream_t stream) {
    if (T < 0 || B < 0 || H <= 0 || G <= 0 || H % G || dk <= 0 || dv <= 0 || !state || !bg) return IK_BAD_ARGUMENT;
    if (T == 0 || B == 0) return IK_OK;
    if (dk > 32 * 16) return IK_UNSUPPORTED;         // 32 lanes of 16 rows
    if (one_token_each && T != B) return IK_BAD_ARGUMENT;
    constexpr int R = 16;                            // rows a lane keeps
    int L = 1;
    while (L * R < dk) L *= 2;
    const int cpw = 32 / L;
    const int nwarps = min(8, (dv + cpw - 1) / cpw), CB = nwarps * cpw, LR = L * R;
    const int W = (2 * LR + CB + 3 + 3) / 4 * 4;
    const int TT = one_token_each ? 1 : (W <= 320 ? 16 : 8);
    const int vec = dk % 4 == 0 && ldu % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 && ((uintptr_t)u & 15) == 0;
    const dim3 grid(B, H, (dv + CB - 1) / CB);
    const size_t smem = (size_t)(2 * TT * W) * sizeof(float);
    if (smem > 160 * 1024) return IK_UNSUPPORTED;
#define IK_DR(LL)                                                                                                                 \
    case LL:                                                                                                                      \
        IK_RETURN_IF_ERROR(ik_delta_rule_launch<LL, R>(grid, 32 * nwarps, smem, stream, u, ldu, q_off, k_off, v_off, bg, state, slots, \
                                                       cu_seqlens, kv_lens, out, H, G, dk, dv, TT, W, vec));                     \
        break
    switch (L) {
        IK_DR(1);
        IK_DR(2);
        IK_DR(4);
        IK_DR(8);
        IK_DR(16);
        IK_DR(32);
    }
#undef IK_DR
    IK_LAUNCH_STATUS();
}

// ------------------------------------------------------------------ RMS norm per head with a gate
// out[t, h*dv + i] = x[t, h, i] * (1 / sqrt(mean_i(x[t, h, :]^2) + eps)) * w[i] * act(p[t, g_off + h*dv + i]), the weight of
// size dv shared by the heads (w_head = 0) or one of size dv per head (w_head = dv: w[h * dv + i]); act 1: silu, 2: sigmoid,
// 0: no gate.  One warp per (token, head).
template <typename TO>
__global__ void __launch_bounds__(256)
head_norm_gate_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ p, int ldp, int g_off,
                      TO* __restrict__ out, int rows, int H, int dv, float eps, int act, int w_head) {
    ik_pdl_wait();
    IK_AFTER_WAIT(x);
    IK_AFTER_WAIT(p);
    ik_pdl_launch_dependents();
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const int t = row / H, h = row - t * H;
    const float* a = x + (size_t)row * dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) ss = fmaf(a[i], a[i], ss);
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float s = 1.0f / sqrtf(ss / (float)dv + eps);
    const float* g = act ? p + (size_t)t * ldp + g_off + h * dv : nullptr;
    for (int i = lane; i < dv; i += 32) {
        float v = a[i] * s * w[h * w_head + i];
        if (act == 1) v *= g[i] / (1.0f + expf(-g[i]));
        else if (act == 2) v *= 1.0f / (1.0f + expf(-g[i]));
        ik_st(out, (size_t)row * dv + i, v);
    }
}

IK_EXPORT int ik_head_norm_gate(const float* x, const float* w, const float* p, int ldp, int g_off, void* out, int out_dtype, int T,
                                int H, int dv, float eps, int act, int w_head, cudaStream_t stream) {
    if (T < 0 || H <= 0 || dv <= 0 || act < 0 || act > 2 || (act && !p) || (w_head != 0 && w_head != dv)) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    const int rows = T * H, blocks = (rows + 7) / 8;
    if (out_dtype == IK_F32)
        IK_RETURN_IF_ERROR(ik_launch(head_norm_gate_kernel<float>, blocks, 256, 0, stream, x, w, p, ldp, g_off, (float*)out, rows, H, dv, eps, act, w_head));
    else if (out_dtype == IK_BF16)
        IK_RETURN_IF_ERROR(ik_launch(head_norm_gate_kernel<__nv_bfloat16>, blocks, 256, 0, stream, x, w, p, ldp, g_off, (__nv_bfloat16*)out, rows, H, dv, eps, act, w_head));
    else return IK_BAD_ARGUMENT;
    IK_LAUNCH_STATUS();
}
