// The gated delta rule: a mixer whose state is a matrix per head that is decayed, corrected towards the current value
// along the current key, and read out with the current query.
//
// Per value head h (its query and key come from head h / (H / G) of G query/key heads), with a decay g and a step b per
// token and head:  S <- g S;  u = b (v - S^T k);  S <- S + k u^T;  o = S^T q   (S is dk x dv, zero before the first token).
// Both sums over rows are taken from the state as it was before the token: with A = S_old^T k and B = S_old^T q,
// u = b (v - g A), S_new = g S_old + k u^T and o = g B + (k . q) u.  One pass over a thread's rows and one exchange
// between the warps of a block per token.
//
// The step's tokens are token-major as everywhere: sequence n brings tokens cu_seqlens[n] .. cu_seqlens[n + 1] - 1 at
// positions kv_lens[n] - count .. kv_lens[n] - 1, its state lies in slot slots[n], kept twice by the parity of the
// position it belongs to (a step reads the copy of parity (first - 1) & 1 and writes that of (last) & 1, so a decode
// step never overwrites what it read and may be run again).  Everything here is float: unit norms, steps, decays
// (formed in double and rounded once: a decay's error is multiplied into the state at every token), states, sums.
#include "common.cuh"

__device__ __forceinline__ void ik_cp_async4(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void ik_cp_async_wait_all() { asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory"); }

// ------------------------------------------------------------------ unit vectors, steps and decays
// One block per token.  u [T, ldu] holds q (G heads of dk) from q_off and k from k_off, behind their convolution and
// activation: every head becomes x / sqrt(sum x^2 + unit_eps), q also times q_mult, in place (one warp per head, lanes in
// index order, then the shuffle tree).  p [T, ldp] holds the step's and the decay's projections, one column per head from
// b_off and a_off: bg[t, 0, h] = sigmoid(p_b), bg[t, 1, h] = exp(-exp(A_log[h]) * softplus(p_a + dt_bias[h])).
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
        const double z = (double)row[a_off + h] + (double)dt_bias[h];
        const double sp = z > 30.0 ? z : log1p(exp(z));
        bg[((size_t)t * 2 + 1) * H + h] = (float)exp(-exp((double)A_log[h]) * sp);
    }
}

IK_EXPORT int ik_delta_prepare(float* u, int ldu, int q_off, int k_off, const float* p, int ldp, int b_off, int a_off,
                               const float* A_log, const float* dt_bias, float* bg, int T, int G, int dk, int H, float q_mult,
                               float unit_eps, cudaStream_t stream) {
    if (T < 0 || G <= 0 || dk <= 0 || H <= 0 || !u || !p || !A_log || !dt_bias || !bg) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    IK_RETURN_IF_ERROR(ik_launch(delta_prepare_kernel, T, 128, 0, stream, u, ldu, q_off, k_off, p, ldp, b_off, a_off, A_log, dt_bias, bg,
                                 G, dk, H, q_mult, unit_eps));
    IK_LAUNCH_STATUS();
}

// ------------------------------------------------------------------ the rule
// A block holds 32 columns of one head's state for one sequence; thread (j, part) keeps rows part*R .. part*R + R - 1 of
// column j in registers, one warp per part.  Tokens come through shared memory in tiles of TT (q, k, the block's 32
// values of v, the step and the decay), the next tile on its way (cp.async) while one is computed.  Per token every
// thread forms its rows' share of A, B and k . q, the shares meet in shared memory (two copies by the token's parity,
// so one barrier a token) and every thread adds them in part order.  What is computed for a token depends on its
// sequence's earlier tokens only, not on where steps or tiles begin.  FULL: dk = parts * RMAX, a multiple of 4: no row
// is guarded and q, k come from shared memory four at a time.
template <int RMAX, bool FULL>
__global__ void __launch_bounds__(512)
delta_rule_kernel(const float* __restrict__ u, int ldu, int q_off, int k_off, int v_off, const float* __restrict__ bg,
                  float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ cu_seqlens,
                  const int* __restrict__ kv_lens, float* __restrict__ out, int H, int G, int dk, int dv, int R, int TT, int W) {
    extern __shared__ __align__(16) float sm[];          // [2][TT][W]: q, k, 32 of v, step, decay;  [2][parts][3][32] shares
    ik_pdl_wait();
    IK_AFTER_WAIT(u);
    IK_AFTER_WAIT(bg);
    IK_AFTER_WAIT(slots);
    IK_AFTER_WAIT(cu_seqlens);
    IK_AFTER_WAIT(kv_lens);
    ik_pdl_launch_dependents();
    const int b = blockIdx.x, h = blockIdx.y, j = threadIdx.x, part = threadIdx.y, parts = blockDim.y;
    const int col0 = blockIdx.z * 32, col = col0 + j;
    const bool live = col < dv;
    const int ccol = live ? col : dv - 1;
    const int tid = part * 32 + j, nthreads = parts * 32, per_tile = TT * W;
    float* shares = sm + 2 * per_tile;
    const int lo = cu_seqlens[b], hi = cu_seqlens[b + 1], end = kv_lens[b], start = end - (hi - lo);
    if (hi <= lo) return;
    const int kvh = h / (H / G);
    const size_t per = (size_t)H * dk * dv;
    const float* st_in = state + ((size_t)slots[b] * 2 + ((start - 1) & 1)) * per + (size_t)h * dk * dv;
    float* st_out = state + ((size_t)slots[b] * 2 + ((end - 1) & 1)) * per + (size_t)h * dk * dv;
    float S[RMAX];
    #pragma unroll
    for (int r = 0; r < RMAX; r++) {
        const int i = part * R + r;
        S[r] = (r < R && i < dk && start > 0) ? st_in[(size_t)i * dv + ccol] : 0.f;
    }
    auto stage = [&](int t0, int buf) {
        const int n = min(TT, hi - t0);
        for (int e = tid; e < n * W; e += nthreads) {
            const int tt = e / W, w = e - tt * W;
            const float* row = u + (size_t)(t0 + tt) * ldu;
            const float* src = nullptr;
            if (w < dk) src = row + q_off + kvh * dk + w;
            else if (w < 2 * dk) src = row + k_off + kvh * dk + (w - dk);
            else if (w < 2 * dk + 32) { if (col0 + w - 2 * dk < dv) src = row + v_off + h * dv + col0 + (w - 2 * dk); }
            else if (w < 2 * dk + 34) src = bg + ((size_t)(t0 + tt) * 2 + (w - 2 * dk - 32)) * H + h;
            float* dst = sm + buf * per_tile + e;
            if (src) ik_cp_async4(dst, src);
            else *dst = 0.f;
        }
    };
    stage(lo, 0);
    ik_cp_async_wait_all();
    __syncthreads();
    int buf = 0;
    for (int t0 = lo; t0 < hi; t0 += TT, buf ^= 1) {
        if (t0 + TT < hi) stage(t0 + TT, buf ^ 1);
        const int n_here = min(TT, hi - t0);
        for (int tt = 0; tt < n_here; tt++) {
            const float* q = sm + buf * per_tile + tt * W + part * R;
            const float* k = q + dk;
            const float* tail = sm + buf * per_tile + tt * W + 2 * dk;
            const float v = tail[j], beta = tail[32], g = tail[33];
            float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f, c0 = 0.f;
            if (FULL) {
                #pragma unroll
                for (int r = 0; r < RMAX; r += 4) {
                    const float4 kk = *reinterpret_cast<const float4*>(k + r), qq = *reinterpret_cast<const float4*>(q + r);
                    a0 = fmaf(S[r], kk.x, a0);     b0 = fmaf(S[r], qq.x, b0);     c0 = fmaf(kk.x, qq.x, c0);
                    a1 = fmaf(S[r + 1], kk.y, a1); b1 = fmaf(S[r + 1], qq.y, b1); c0 = fmaf(kk.y, qq.y, c0);
                    a0 = fmaf(S[r + 2], kk.z, a0); b0 = fmaf(S[r + 2], qq.z, b0); c0 = fmaf(kk.z, qq.z, c0);
                    a1 = fmaf(S[r + 3], kk.w, a1); b1 = fmaf(S[r + 3], qq.w, b1); c0 = fmaf(kk.w, qq.w, c0);
                }
            } else {
                #pragma unroll
                for (int r = 0; r < RMAX; r++) {
                    if (r < R && part * R + r < dk) {
                        if (r & 1) { a1 = fmaf(S[r], k[r], a1); b1 = fmaf(S[r], q[r], b1); }
                        else { a0 = fmaf(S[r], k[r], a0); b0 = fmaf(S[r], q[r], b0); }
                        c0 = fmaf(k[r], q[r], c0);
                    }
                }
            }
            float* mine = shares + ((tt & 1) * parts + part) * 96;
            mine[j] = a0 + a1;
            mine[32 + j] = b0 + b1;
            mine[64 + j] = c0;
            __syncthreads();
            float A = 0.f, B = 0.f, KQ = 0.f;
            for (int pp = 0; pp < parts; pp++) {
                const float* x = shares + ((tt & 1) * parts + pp) * 96;
                A += x[j];
                B += x[32 + j];
                KQ += x[64 + j];
            }
            const float un = beta * (v - g * A);
            if (FULL) {
                #pragma unroll
                for (int r = 0; r < RMAX; r += 4) {
                    const float4 kk = *reinterpret_cast<const float4*>(k + r);
                    S[r] = fmaf(g, S[r], kk.x * un);
                    S[r + 1] = fmaf(g, S[r + 1], kk.y * un);
                    S[r + 2] = fmaf(g, S[r + 2], kk.z * un);
                    S[r + 3] = fmaf(g, S[r + 3], kk.w * un);
                }
            } else {
                #pragma unroll
                for (int r = 0; r < RMAX; r++)
                    if (r < R && part * R + r < dk) S[r] = fmaf(g, S[r], k[r] * un);
            }
            if (part == 0 && live) out[(size_t)(t0 + tt) * H * dv + h * dv + col] = fmaf(g, B, KQ * un);
        }
        ik_cp_async_wait_all();
        __syncthreads();
    }
    if (live) {
        #pragma unroll
        for (int r = 0; r < RMAX; r++) {
            const int i = part * R + r;
            if (r < R && i < dk) st_out[(size_t)i * dv + col] = S[r];
        }
    }
}

IK_EXPORT int ik_delta_rule(const float* u, int ldu, int q_off, int k_off, int v_off, const float* bg, float* state, const int* slots,
                            const int* cu_seqlens, const int* kv_lens, float* out, int T, int B, int H, int G, int dk, int dv,
                            int one_token_each, cudaStream_t stream) {
    if (T < 0 || B < 0 || H <= 0 || G <= 0 || H % G || dk <= 0 || dv <= 0 || !state || !bg) return IK_BAD_ARGUMENT;
    if (T == 0 || B == 0) return IK_OK;
    if (dk > 512) return IK_UNSUPPORTED;
    if (one_token_each && T != B) return IK_BAD_ARGUMENT;
    const int R = dk <= 64 ? 16 : 32;                // rows a thread: two to four warps a block up to 128 rows
    const int parts = (dk + R - 1) / R;
    const int W = (2 * dk + 34 + 3) / 4 * 4;
    const int TT = one_token_each ? 1 : 8;
    const bool full = dk == parts * R && ldu % 4 == 0;
    const dim3 grid(B, H, (dv + 31) / 32), block(32, parts);
    const size_t smem = (size_t)(2 * TT * W + 2 * parts * 96) * sizeof(float);
    if (smem > 160 * 1024) return IK_UNSUPPORTED;
#define IK_DR(RMAX, FULL)                                                                                                        \
    do {                                                                                                                         \
        static bool raised = false;                                                                                              \
        if (smem > 48 * 1024 && !raised) {                                                                                       \
            IK_RETURN_IF_ERROR(cudaFuncSetAttribute(delta_rule_kernel<RMAX, FULL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024)); \
            raised = true;                                                                                                       \
        }                                                                                                                        \
        IK_RETURN_IF_ERROR(ik_launch(delta_rule_kernel<RMAX, FULL>, grid, block, smem, stream, u, ldu, q_off, k_off, v_off, bg, state, slots, \
                                     cu_seqlens, kv_lens, out, H, G, dk, dv, R, TT, W));                                          \
    } while (0)
    if (R == 16 && full) IK_DR(16, true);
    else if (R == 16) IK_DR(16, false);
    else if (full) IK_DR(32, true);
    else IK_DR(32, false);
#undef IK_DR
    IK_LAUNCH_STATUS();
}

// ------------------------------------------------------------------ RMS norm per head with a gate
// out[t, h*dv + i] = x[t, h, i] * (1 / sqrt(mean_i(x[t, h, :]^2) + eps)) * w[i] * act(p[t, g_off + h*dv + i]), the weight of
// size dv shared by the heads; act 1: silu, 2: sigmoid, 0: no gate.  One warp per (token, head).
template <typename TO>
__global__ void __launch_bounds__(256)
head_norm_gate_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ p, int ldp, int g_off,
                      TO* __restrict__ out, int rows, int H, int dv, float eps, int act) {
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
        float v = a[i] * s * w[i];
        if (act == 1) v *= g[i] / (1.0f + expf(-g[i]));
        else if (act == 2) v *= 1.0f / (1.0f + expf(-g[i]));
        ik_st(out, (size_t)row * dv + i, v);
    }
}

IK_EXPORT int ik_head_norm_gate(const float* x, const float* w, const float* p, int ldp, int g_off, void* out, int out_dtype, int T,
                                int H, int dv, float eps, int act, cudaStream_t stream) {
    if (T < 0 || H <= 0 || dv <= 0 || act < 0 || act > 2 || (act && !p)) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    const int rows = T * H, blocks = (rows + 7) / 8;
    if (out_dtype == IK_F32)
        IK_RETURN_IF_ERROR(ik_launch(head_norm_gate_kernel<float>, blocks, 256, 0, stream, x, w, p, ldp, g_off, (float*)out, rows, H, dv, eps, act));
    else if (out_dtype == IK_BF16)
        IK_RETURN_IF_ERROR(ik_launch(head_norm_gate_kernel<__nv_bfloat16>, blocks, 256, 0, stream, x, w, p, ldp, g_off, (__nv_bfloat16*)out, rows, H, dv, eps, act));
    else return IK_BAD_ARGUMENT;
    IK_LAUNCH_STATUS();
}
