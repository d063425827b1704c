// Recurrent mixers whose state is a matrix per head that decays row by row: every key channel has a decay of its own
// per token.  Two rules share one kernel:
//
//   rule 0, the delta rule with a decay per key channel:
//       S <- diag(a) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          (the read-out sees the token's own write)
//   rule 1, token-shift time mixing with a bonus for the current token:
//       o = (S + diag(bonus) k v^T)^T r;   S <- diag(w) S + k v^T                       (the read-out sees the state before the token)
//
// S is dk x dv per head, zero before a sequence's first token, float.  The layout of the work is the delta rule's
// (delta.cu): a column of S is a recurrence of its own, L lanes of a warp share a column and keep 16 of its rows each in
// registers, tokens pass through shared memory in tiles with the next tile on its way, sums run in the same order
// whatever step or tile brings a token.  Rule 0 takes both sums from the decayed state, sd = a * S: A = sd^T k,
// B = sd^T q, u = beta (v - A), S = sd + k u^T, o = B + (k . q) u.  Rule 1: B = S^T r, o = B + (sum_i bonus_i k_i r_i) v,
// S = w * S + k v^T.  The state lies as [2, heads, dv, dk] per slot, the two copies by the parity of the position
// the state belongs to, as for the other recurrences.
//
// Around it: the decays themselves (two forms, float with the accurate exponential and logarithm), and the token shift (every token's input
// mixed with the input one position earlier, which is part of the sequence's state).
#include "common.cuh"

namespace {

__device__ __forceinline__ void rd_cp_async4(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void rd_cp_async16(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void rd_cp_async_wait_all() { asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory"); }

// ------------------------------------------------------------------ decays
// kind 0: out[t, c] = exp(-exp(A_log[c / per_head]) * softplus(x[t, c] + bias[c]));  kind 1: out[t, c] = exp(-exp(x[t, c] + bias[c])).
__global__ void decay_rows_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ bias, const float* __restrict__ A_log,
                                  float* __restrict__ out, size_t total, int C, int per_head, int kind) {
    ik_pdl_wait();
    IK_AFTER_WAIT(x);
    ik_pdl_launch_dependents();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const size_t t = idx / C;
        const int c = (int)(idx - t * C);
        const float z = x[t * ldx + c] + (bias ? bias[c] : 0.f);
        float r;
        if (kind == 0) {
            const float sp = z > 20.0f ? z : log1pf(expf(z));
            r = expf(-expf(A_log[c / per_head]) * sp);
        } else {
            r = expf(-expf(z));
        }
        out[idx] = r;
    }
}

// ------------------------------------------------------------------ token shift
// out[m][t, i] = x[t, i] + (x'[t, i] - x[t, i]) * mu[m, i] for m < n_mix, x' the input one position earlier in the same
// sequence (zeros at position 0): the row before within the step, or what the sequence's ring holds.  The ring keeps the
// input of the last position by that position's parity, [2, d] floats per slot.  Mix m is a matrix [T, d] of its own,
// mix_stride elements after the one before.
template <typename TX>
__global__ void __launch_bounds__(256)
token_shift_kernel(const TX* __restrict__ x, const float* __restrict__ mu, float* __restrict__ ring, const int* __restrict__ slots,
                   const int* __restrict__ cu_seqlens, const int* __restrict__ token_seq, const int* __restrict__ token_pos,
                   TX* __restrict__ out, size_t mix_stride, int d, int n_mix, int inline_ring) {
    ik_pdl_wait();
    IK_AFTER_WAIT(x);
    IK_AFTER_WAIT(slots);
    IK_AFTER_WAIT(cu_seqlens);
    IK_AFTER_WAIT(token_seq);
    IK_AFTER_WAIT(token_pos);
    ik_pdl_launch_dependents();
    const int t = blockIdx.x, i = blockIdx.y * 256 + threadIdx.x;
    if (i >= d) return;
    const int b = token_seq[t], pos = token_pos[t], first = cu_seqlens[b];
    const float cur = ik_ld(x, (size_t)t * d + i);
    float prev = 0.f;
    if (pos > 0) prev = t - 1 >= first ? ik_ld(x, (size_t)(t - 1) * d + i) : ring[((size_t)slots[b] * 2 + ((pos - 1) & 1)) * d + i];
    for (int m = 0; m < n_mix; m++) ik_st(out, m * mix_stride + (size_t)t * d + i, fmaf(prev - cur, mu[(size_t)m * d + i], cur));
    if (inline_ring) ring[((size_t)slots[b] * 2 + (pos & 1)) * d + i] = cur;
}

template <typename TX>
__global__ void __launch_bounds__(256)
token_shift_ring_kernel(const TX* __restrict__ x, float* __restrict__ ring, const int* __restrict__ slots,
                        const int* __restrict__ cu_seqlens, const int* __restrict__ kv_lens, int d) {
    ik_pdl_wait();
    IK_AFTER_WAIT(x);
    IK_AFTER_WAIT(slots);
    IK_AFTER_WAIT(cu_seqlens);
    IK_AFTER_WAIT(kv_lens);
    ik_pdl_launch_dependents();
    const int b = blockIdx.x, i = blockIdx.y * 256 + threadIdx.x;
    const int lo = cu_seqlens[b], hi = cu_seqlens[b + 1];
    if (i >= d || hi <= lo) return;
    const int pos = kv_lens[b] - 1;
    ring[((size_t)slots[b] * 2 + (pos & 1)) * d + i] = ik_ld(x, (size_t)(hi - 1) * d + i);
}

// ------------------------------------------------------------------ the recurrence
// x1 (q or r) and k come from the float matrix u (row stride ldu) at x1_off / k_off + (query/key head) * dk, v at
// v_off + h * dv, the decays from dec [T, H * dk], the steps from beta (row stride ldb, one per head; rule 0), the bonus from bonus [H * dk] (rule 1).
template <int L, int R, int RULE>
__global__ void __launch_bounds__(256, 4)
row_decay_kernel(const float* __restrict__ u, int ldu, int x1_off, int k_off, int v_off, const float* __restrict__ dec,
                 const float* __restrict__ beta, int ldb, const float* __restrict__ bonus, float* __restrict__ state,
                 const int* __restrict__ slots, const int* __restrict__ cu_seqlens, const int* __restrict__ kv_lens,
                 float* __restrict__ out, int H, int G, int dk, int dv, int TT, int W, int vec) {
    extern __shared__ __align__(16) float sm[];          // [2][TT][W]: x1, k, decay (16 L each), the block's v, step, c
    ik_pdl_wait();
    IK_AFTER_WAIT(u);
    IK_AFTER_WAIT(dec);
    IK_AFTER_WAIT(beta);
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
    auto stage = [&](int t0, int buf) {                  // a warp brings whole tokens
        const int n = min(TT, hi - t0);
        for (int tt = warp; tt < n; tt += nwarps) {
            const float* row = u + (size_t)(t0 + tt) * ldu;
            float* dst = sm + buf * per_tile + tt * W;
            const float* s0 = row + x1_off + kvh * dk;
            const float* s1 = row + k_off + kvh * dk;
            const float* s2 = dec + ((size_t)(t0 + tt) * H + h) * dk;
            if (vec) {                                   // dk a multiple of 4 and every source row on a 16-byte boundary
                for (int f = lane; f < 3 * (LR / 4); f += 32) {
                    const int which = f / (LR / 4), g4 = f - which * (LR / 4);
                    const float* src = (which == 0 ? s0 : which == 1 ? s1 : s2) + 4 * g4;
                    if (4 * g4 < dk) rd_cp_async16(dst + 4 * f, src);
                    else *reinterpret_cast<float4*>(dst + 4 * f) = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            } else {
                for (int w = lane; w < 3 * LR; w += 32) {
                    const int which = w / LR, i = w - which * LR;
                    if (i < dk) rd_cp_async4(dst + w, (which == 0 ? s0 : which == 1 ? s1 : s2) + i);
                    else dst[w] = 0.f;
                }
            }
            for (int w = lane; w < CB + 1; w += 32) {
                if (w < CB) {
                    if (col0 + w < dv) rd_cp_async4(dst + 3 * LR + w, row + v_off + h * dv + col0 + w);
                    else dst[3 * LR + w] = 0.f;
                } else if (RULE == 0) {
                    rd_cp_async4(dst + 3 * LR + w, beta + (size_t)(t0 + tt) * ldb + h);
                }
            }
        }
    };
    stage(lo, 0);
    rd_cp_async_wait_all();
    __syncthreads();
    int buf = 0;
    for (int t0 = lo; t0 < hi; t0 += TT, buf ^= 1) {
        if (t0 + TT < hi) stage(t0 + TT, buf ^ 1);
        const int n_here = min(TT, hi - t0);
        for (int tt = warp; tt < n_here; tt += nwarps) {        // c of the tile's tokens, lanes in index order, then the tree
            float* x = sm + buf * per_tile + tt * W;
            float c = 0.f;
            for (int i = lane; i < LR; i += 32) {
                const float kx = x[i] * x[LR + i];
                c = (RULE == 1) ? fmaf(i < dk ? bonus[h * dk + i] : 0.f, kx, c) : c + kx;
            }
            #pragma unroll
            for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
            if (lane == 0) x[3 * LR + CB + 1] = c;
        }
        __syncthreads();
        #pragma unroll 2
        for (int tt = 0; tt < n_here; tt++) {
            const float* x = sm + buf * per_tile + tt * W;
            const float4* x4 = reinterpret_cast<const float4*>(x);
            const float4* k4 = reinterpret_cast<const float4*>(x + LR);
            const float4* d4 = reinterpret_cast<const float4*>(x + 2 * LR);
            const float* tail = x + 3 * LR;
            const float v = tail[warp * CPW + jj], c = tail[CB + 1];
            float4 kk[NF];
            if (RULE == 0) {
                const float step = tail[CB];
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, b0 = 0.f, b1 = 0.f, b2 = 0.f, b3 = 0.f;
                #pragma unroll
                for (int f = 0; f < NF; f++) {
                    kk[f] = k4[f * L + part];
                    const float4 qq = x4[f * L + part], dd = d4[f * L + part];
                    S[4 * f] *= dd.x; S[4 * f + 1] *= dd.y; S[4 * f + 2] *= dd.z; S[4 * f + 3] *= dd.w;
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
                const float un = step * (v - A);
                #pragma unroll
                for (int f = 0; f < NF; f++) {
                    S[4 * f] = fmaf(kk[f].x, un, S[4 * f]);
                    S[4 * f + 1] = fmaf(kk[f].y, un, S[4 * f + 1]);
                    S[4 * f + 2] = fmaf(kk[f].z, un, S[4 * f + 2]);
                    S[4 * f + 3] = fmaf(kk[f].w, un, S[4 * f + 3]);
                }
                if (part == 0 && live) out[(size_t)(t0 + tt) * H * dv + h * dv + col] = fmaf(c, un, B);
            } else {
                float b0 = 0.f, b1 = 0.f, b2 = 0.f, b3 = 0.f;
                #pragma unroll
                for (int f = 0; f < NF; f++) {
                    kk[f] = k4[f * L + part];
                    const float4 rr = x4[f * L + part], dd = d4[f * L + part];
                    b0 = fmaf(S[4 * f], rr.x, b0);
                    b1 = fmaf(S[4 * f + 1], rr.y, b1);
                    b2 = fmaf(S[4 * f + 2], rr.z, b2);
                    b3 = fmaf(S[4 * f + 3], rr.w, b3);
                    S[4 * f] = fmaf(dd.x, S[4 * f], kk[f].x * v);
                    S[4 * f + 1] = fmaf(dd.y, S[4 * f + 1], kk[f].y * v);
                    S[4 * f + 2] = fmaf(dd.z, S[4 * f + 2], kk[f].z * v);
                    S[4 * f + 3] = fmaf(dd.w, S[4 * f + 3], kk[f].w * v);
                }
                float B = (b0 + b1) + (b2 + b3);
                #pragma unroll
                for (int o = 1; o < L; o <<= 1) B += __shfl_xor_sync(0xffffffffu, B, o);
                if (part == 0 && live) out[(size_t)(t0 + tt) * H * dv + h * dv + col] = fmaf(c, v, B);
            }
        }
        rd_cp_async_wait_all();
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

template <int L, int R, int RULE>
cudaError_t row_decay_launch(dim3 grid, int threads, size_t smem, cudaStream_t stream, const float* u, int ldu, int x1_off, int k_off,
                             int v_off, const float* dec, const float* beta, int ldb, const float* bonus, float* state, const int* slots,
                             const int* cu_seqlens, const int* kv_lens, float* out, int H, int G, int dk, int dv, int TT, int W, int vec) {
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        const cudaError_t e = cudaFuncSetAttribute(row_decay_kernel<L, R, RULE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        if (e != cudaSuccess) return e;
        raised = true;
    }
    return ik_launch(row_decay_kernel<L, R, RULE>, grid, dim3(threads), smem, stream, u, ldu, x1_off, k_off, v_off, dec, beta, ldb, bonus, state,
                     slots, cu_seqlens, kv_lens, out, H, G, dk, dv, TT, W, vec);
}

}  // namespace

IK_EXPORT int ik_decay_rows(const float* x, int ldx, const float* bias, const float* A_log, float* out, int T, int C, int per_head,
                            int kind, cudaStream_t stream) {
    if (T < 0 || C <= 0 || ldx < C || kind < 0 || kind > 1 || (kind == 0 && (!A_log || per_head <= 0 || C % per_head))) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    const size_t total = (size_t)T * C, want = (total + 255) / 256, cap = (size_t)ik_sm_count() * 32;
    IK_RETURN_IF_ERROR(ik_launch(decay_rows_kernel, (int)(want < cap ? want : cap), 256, 0, stream, x, ldx, bias, A_log, out, total, C,
                                 per_head > 0 ? per_head : 1, kind));
    IK_LAUNCH_STATUS();
}

IK_EXPORT int ik_token_shift(const void* x, int dtype, const float* mu, float* ring, const int* slots, const int* cu_seqlens,
                             const int* kv_lens, const int* token_seq, const int* token_pos, void* out, unsigned long long mix_stride,
                             int T, int B, int d, int n_mix, int one_token_each, cudaStream_t stream) {
    if (T < 0 || B < 0 || d <= 0 || n_mix <= 0 || !ring || !mu) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    const dim3 grid(T, (d + 255) / 256), grid2(B, (d + 255) / 256);
    const int inl = one_token_each ? 1 : 0;
    if (dtype == IK_F32) {
        IK_RETURN_IF_ERROR(ik_launch(token_shift_kernel<float>, grid, 256, 0, stream, (const float*)x, mu, ring, slots, cu_seqlens, token_seq,
                                     token_pos, (float*)out, (size_t)mix_stride, d, n_mix, inl));
        if (!inl) IK_RETURN_IF_ERROR(ik_launch(token_shift_ring_kernel<float>, grid2, 256, 0, stream, (const float*)x, ring, slots, cu_seqlens, kv_lens, d));
    } else if (dtype == IK_BF16) {
        IK_RETURN_IF_ERROR(ik_launch(token_shift_kernel<__nv_bfloat16>, grid, 256, 0, stream, (const __nv_bfloat16*)x, mu, ring, slots, cu_seqlens,
                                     token_seq, token_pos, (__nv_bfloat16*)out, (size_t)mix_stride, d, n_mix, inl));
        if (!inl) IK_RETURN_IF_ERROR(ik_launch(token_shift_ring_kernel<__nv_bfloat16>, grid2, 256, 0, stream, (const __nv_bfloat16*)x, ring, slots,
                                               cu_seqlens, kv_lens, d));
    } else return IK_BAD_ARGUMENT;
    IK_LAUNCH_STATUS();
}

IK_EXPORT int ik_row_decay(int rule, const float* u, int ldu, int x1_off, int k_off, int v_off, const float* dec, const float* beta,
                           int ldb, const float* bonus, float* state, const int* slots, const int* cu_seqlens, const int* kv_lens, float* out,
                           int T, int B, int H, int G, int dk, int dv, int one_token_each, cudaStream_t stream) {
    if (T < 0 || B < 0 || H <= 0 || G <= 0 || H % G || dk <= 0 || dv <= 0 || !state || !dec || rule < 0 || rule > 1) return IK_BAD_ARGUMENT;
    if ((rule == 0 && !beta) || (rule == 1 && !bonus)) return IK_BAD_ARGUMENT;
    if (T == 0 || B == 0) return IK_OK;
    if (dk > 32 * 16) return IK_UNSUPPORTED;         // 32 lanes of 16 rows
    if (one_token_each && T != B) return IK_BAD_ARGUMENT;
    constexpr int R = 16;                            // rows a lane keeps
    int L = 1;
    while (L * R < dk) L *= 2;
    const int cpw = 32 / L;
    const int nwarps = min(8, (dv + cpw - 1) / cpw), CB = nwarps * cpw, LR = L * R;
    const int W = (3 * LR + CB + 2 + 3) / 4 * 4;
    const int TT = one_token_each ? 1 : (W <= 480 ? 16 : 8);
    const int vec = dk % 4 == 0 && ldu % 4 == 0 && x1_off % 4 == 0 && k_off % 4 == 0 && ((uintptr_t)u & 15) == 0 && ((uintptr_t)dec & 15) == 0;
    const dim3 grid(B, H, (dv + CB - 1) / CB);
    const size_t smem = (size_t)(2 * TT * W) * sizeof(float);
    if (smem > 160 * 1024) return IK_UNSUPPORTED;
#define IK_RD(LL)                                                                                                                    \
    case LL:                                                                                                                         \
        if (rule == 0)                                                                                                               \
            IK_RETURN_IF_ERROR((row_decay_launch<LL, R, 0>(grid, 32 * nwarps, smem, stream, u, ldu, x1_off, k_off, v_off, dec, beta, ldb, bonus, \
                                                           state, slots, cu_seqlens, kv_lens, out, H, G, dk, dv, TT, W, vec)));      \
        else                                                                                                                         \
            IK_RETURN_IF_ERROR((row_decay_launch<LL, R, 1>(grid, 32 * nwarps, smem, stream, u, ldu, x1_off, k_off, v_off, dec, beta, ldb, bonus, \
                                                           state, slots, cu_seqlens, kv_lens, out, H, G, dk, dv, TT, W, vec)));      \
        break
    switch (L) {
        IK_RD(1);
        IK_RD(2);
        IK_RD(4);
        IK_RD(8);
        IK_RD(16);
        IK_RD(32);
    }
#undef IK_RD
    IK_LAUNCH_STATUS();
}
