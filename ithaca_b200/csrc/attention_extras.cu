// What stands around an attention core when the projections come out of one wide product: a norm over a whole
// projection fused with rotation and cache append, a gate per head on the attention's result, and an RMS norm with a
// sigmoid gate on a mixer's result.  Inputs are column ranges of a float matrix `p` with row stride ldp.
#include "common.cuh"

// ------------------------------------------------------------------ norm + rotation + cache append
// One block per token.  q = columns [q_off, q_off + nh*hd), k = [k_off, + nkv*hd), v = [v_off, + nkv*hdv).
// With q_w / k_w: q (and k) is divided by the root mean square of ALL its nh*hd (nkv*hd) values, eps inside the root,
// and multiplied by the weight of that size; with per_head set, every head is divided by the root mean square of its own
// hd values and multiplied by a weight of size hd that all heads share.  Then the leading `rot` dimensions of every q and k head are rotated:
// pairing 0 turns (i, i + rot/2), pairing 1 turns (2i, 2i + 1), by float(pos) * inv_freq[i]; cos and sin are multiplied
// by `magnitude`.  q goes to q_out [T, nh*hd]; k and v into the token's place in the pages
// (pages[page][kv head][position in page][size], page = table[seq * table_stride + pos / page_size]).
// `bias` (or null) is a vector over p's columns that is added to q, k and v as they are read.  With v_norm every value head
// is divided by the root mean square of its own hdv values (eps inside the root, no weight) before it is stored.
template <typename TQ, typename TC>
__global__ void __launch_bounds__(256)
norm_rope_append_kernel(const float* __restrict__ p, int ldp, int q_off, int k_off, int v_off, const float* __restrict__ q_w,
                        const float* __restrict__ k_w, float eps, TQ* __restrict__ q_out, TC* __restrict__ k_pages,
                        TC* __restrict__ v_pages, const int* __restrict__ token_seq, const int* __restrict__ token_pos,
                        const int* __restrict__ table, int table_stride, const float* __restrict__ inv_freq, float magnitude,
                        int nh, int nkv, int hd, int hdv, int rot, int pairing, int page_size, int n_pages, int write_cache,
                        int per_head, const float* __restrict__ bias, int v_norm, int* status) {
    extern __shared__ __align__(16) float cs[];          // [rot/2] cos, [rot/2] sin, [nh + nkv] 1 / rms (per_head), [nkv] 1 / rms of v
    __shared__ float red[32];
    ik_pdl_wait();
    IK_AFTER_WAIT(p);
    IK_AFTER_WAIT(token_seq);
    IK_AFTER_WAIT(token_pos);
    IK_AFTER_WAIT(table);
    ik_pdl_launch_dependents();
    const int t = blockIdx.x, half = rot / 2, pos = token_pos[t];
    const float* row = p + (size_t)t * ldp;
    for (int i = threadIdx.x; i < half; i += 256) {
        const float ang = __fmul_rn((float)pos, inv_freq[i]);
        cs[i] = cosf(ang) * magnitude;
        cs[half + i] = sinf(ang) * magnitude;
    }
    float rq = 1.f, rk = 1.f;
    float* head_r = cs + rot;
    float* v_r = head_r + (per_head ? nh + nkv : 0);
    if (v_norm) {
        for (int head = threadIdx.x >> 5; head < nkv; head += 8) {
            const float* src = row + v_off + head * hdv;
            const float* b = bias ? bias + v_off + head * hdv : nullptr;
            float ss = 0.f;
            for (int i = threadIdx.x & 31; i < hdv; i += 32) { const float v = b ? src[i] + b[i] : src[i]; ss = fmaf(v, v, ss); }
            #pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if ((threadIdx.x & 31) == 0) v_r[head] = 1.0f / sqrtf(ss / (float)hdv + eps);
        }
    }
    if (per_head) {
        // one warp per head, lanes in index order, then the shuffle tree: the sum's order depends on hd alone
        for (int head = threadIdx.x >> 5; head < nh + nkv; head += 8) {
            const bool is_q = head < nh;
            const int col = is_q ? q_off + head * hd : k_off + (head - nh) * hd;
            const float* src = row + col;
            const float* b = bias ? bias + col : nullptr;
            float ss = 0.f;
            if (is_q ? q_w != nullptr : k_w != nullptr) {
                for (int i = threadIdx.x & 31; i < hd; i += 32) { const float v = b ? src[i] + b[i] : src[i]; ss = fmaf(v, v, ss); }
                #pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            }
            if ((threadIdx.x & 31) == 0) head_r[head] = 1.0f / sqrtf(ss / (float)hd + eps);
        }
    } else if (q_w) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < nh * hd; i += 256) { const float v = row[q_off + i] + (bias ? bias[q_off + i] : 0.f); ss = fmaf(v, v, ss); }
        ss = ik_block_sum<256>(ss, red);
        rq = 1.0f / sqrtf(ss / (float)(nh * hd) + eps);
    }
    if (k_w && !per_head) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < nkv * hd; i += 256) { const float v = row[k_off + i] + (bias ? bias[k_off + i] : 0.f); ss = fmaf(v, v, ss); }
        ss = ik_block_sum<256>(ss, red);
        rk = 1.0f / sqrtf(ss / (float)(nkv * hd) + eps);
    }
    size_t page_off = 0;
    bool page_ok = false;
    if (write_cache) {
        const int page = table[(size_t)token_seq[t] * table_stride + pos / page_size];
        page_ok = page >= 0 && page < n_pages;
        if (!page_ok) { if (threadIdx.x == 0) ik_set_status(status, IK_STATUS_WRITE_NO_PAGE); }
        else page_off = (size_t)page * nkv * page_size + (pos % page_size);
    }
    __syncthreads();
    // q heads then k heads: element e of head `head`
    for (int e = threadIdx.x; e < (nh + nkv) * hd; e += 256) {
        const int head = e / hd, i = e - head * hd;
        const bool is_q = head < nh;
        if (!is_q && !page_ok) continue;
        const int col = is_q ? q_off + head * hd : k_off + (head - nh) * hd;
        const float* src = row + col;
        const float* b = bias ? bias + col : nullptr;
        const float* w = is_q ? (q_w ? q_w + (per_head ? 0 : head * hd) : nullptr) : (k_w ? k_w + (per_head ? 0 : (head - nh) * hd) : nullptr);
        const float r = per_head ? head_r[head] : is_q ? rq : rk;
        const float mine = b ? src[i] + b[i] : src[i];
        float val = w ? mine * r * w[i] : mine;
        if (i < rot) {
            int partner, f;
            bool first;
            if (pairing == 0) { first = i < half; partner = first ? i + half : i - half; f = first ? i : i - half; }
            else { first = (i & 1) == 0; partner = first ? i + 1 : i - 1; f = i >> 1; }
            const float theirs = b ? src[partner] + b[partner] : src[partner];
            const float other = w ? theirs * r * w[partner] : theirs;
            const float c = cs[f], s = cs[half + f];
            // (u, v) -> (u c - v s, v c + u s); `first` holds u
            val = first ? __fsub_rn(__fmul_rn(val, c), __fmul_rn(other, s)) : __fadd_rn(__fmul_rn(val, c), __fmul_rn(other, s));
        }
        if (is_q) ik_st(q_out, ((size_t)t * nh + head) * hd + i, val);
        else ik_st(k_pages, (page_off + (size_t)(head - nh) * page_size) * hd + i, val);
    }
    if (page_ok) {
        for (int e = threadIdx.x; e < nkv * hdv; e += 256) {
            const int head = e / hdv, i = e - head * hdv;
            float val = row[v_off + e];
            if (bias) val += bias[v_off + e];
            if (v_norm) val *= v_r[head];
            ik_st(v_pages, (page_off + (size_t)head * page_size) * hdv + i, val);
        }
    }
}

IK_EXPORT int ik_norm_rope_append(const float* p, int ldp, int q_off, int k_off, int v_off, const float* q_w, const float* k_w,
                                  float eps, void* q_out, int q_dtype, void* k_pages, void* v_pages, int cache_dtype,
                                  const int* token_seq, const int* token_pos, const int* table, int table_stride,
                                  const float* inv_freq, float magnitude, int T, int nh, int nkv, int hd, int hdv, int rot,
                                  int pairing, int page_size, int n_pages, int write_cache, int per_head, const float* bias, int v_norm, int* status,
                                  cudaStream_t stream) {
    if (T < 0 || nh <= 0 || nkv <= 0 || hd <= 0 || hdv <= 0 || rot < 0 || rot > hd || (rot & 1) || page_size <= 0)
        return IK_BAD_ARGUMENT;
    if (rot > 0 && !inv_freq) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    const size_t smem = (size_t)(rot + (per_head ? nh + nkv : 0) + (v_norm ? nkv : 0)) * sizeof(float);
#define IK_NRA(TQ, TC)                                                                                                       \
    IK_RETURN_IF_ERROR(ik_launch(norm_rope_append_kernel<TQ, TC>, T, 256, smem, stream, p, ldp, q_off, k_off, v_off, q_w, k_w, eps, \
                                 (TQ*)q_out, (TC*)k_pages, (TC*)v_pages, token_seq, token_pos, table, table_stride, inv_freq,  \
                                 magnitude, nh, nkv, hd, hdv, rot, pairing, page_size, n_pages, write_cache, per_head, bias, v_norm, status))
    if (q_dtype == IK_F32 && cache_dtype == IK_F32) IK_NRA(float, float);
    else if (q_dtype == IK_BF16 && cache_dtype == IK_BF16) IK_NRA(__nv_bfloat16, __nv_bfloat16);
    else return IK_BAD_ARGUMENT;
#undef IK_NRA
    IK_LAUNCH_STATUS();
}

// ------------------------------------------------------------------ a gate per head, or per value
// out[t, h * hdv + j] = att[t, h * hdv + j] * sigmoid(p[t, g_off + h]) * mult (no gate without p); out has row stride ldo.
// wide: the gate has one number per value, p[t, g_off + h * hdv + j].
template <typename TA>
__global__ void head_gate_kernel(const TA* __restrict__ att, const float* __restrict__ p, int ldp, int g_off, TA* __restrict__ out,
                                 int ldo, int H, int hdv, size_t total, float mult, int wide) {
    ik_pdl_wait();
    IK_AFTER_WAIT(att);
    IK_AFTER_WAIT(p);
    ik_pdl_launch_dependents();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const int cols = H * hdv;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const size_t t = idx / cols;
        const int c = (int)(idx - t * cols), h = c / hdv;
        const float g = p ? 1.0f / (1.0f + expf(-p[t * ldp + g_off + (wide ? c : h)])) : 1.0f;
        ik_st(out, t * ldo + c, ik_ld(att, idx) * g * mult);
    }
}

// The same by fours (head sizes and row distances that are multiples of four, aligned pointers): one sigmoid per four values.
template <typename TA>
__global__ void head_gate4_kernel(const TA* __restrict__ att, const float* __restrict__ p, int ldp, int g_off, TA* __restrict__ out,
                                  int ldo, int H, int hdv, size_t total4, float mult, int wide) {
    ik_pdl_wait();
    IK_AFTER_WAIT(att);
    IK_AFTER_WAIT(p);
    ik_pdl_launch_dependents();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const int cols4 = H * hdv / 4;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total4; idx += stride) {
        const size_t t = idx / cols4;
        const int c = (int)(idx - t * cols4) * 4, h = c / hdv;
        float4 v = ik_ld4(att, t * (size_t)(H * hdv) + c);
        if (wide && p) {
            const float* gp = p + t * ldp + g_off + c;
            v.x = v.x * (1.0f / (1.0f + expf(-gp[0]))) * mult; v.y = v.y * (1.0f / (1.0f + expf(-gp[1]))) * mult;
            v.z = v.z * (1.0f / (1.0f + expf(-gp[2]))) * mult; v.w = v.w * (1.0f / (1.0f + expf(-gp[3]))) * mult;
        } else {
            const float g = (p ? 1.0f / (1.0f + expf(-p[t * ldp + g_off + h])) : 1.0f);
            v.x = v.x * g * mult; v.y = v.y * g * mult; v.z = v.z * g * mult; v.w = v.w * g * mult;
        }
        ik_st4(out, t * ldo + c, v);
    }
}

IK_EXPORT int ik_head_gate(const void* att, const float* p, int ldp, int g_off, void* out, int dtype, int ldo, int T, int H,
                           int hdv, float mult, int wide, cudaStream_t stream) {
    if (T < 0 || H <= 0 || hdv <= 0 || ldo < H * hdv) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    const size_t total = (size_t)T * H * hdv;
    if (hdv % 4 == 0 && ldo % 4 == 0 && (uintptr_t)att % 16 == 0 && (uintptr_t)out % 16 == 0 && (dtype == IK_F32 || dtype == IK_BF16)) {
        const size_t total4 = total / 4;
        const int blocks4 = (int)((total4 + 255) / 256 < 65535 * 16 ? (total4 + 255) / 256 : 65535 * 16);
        if (dtype == IK_F32)
            IK_RETURN_IF_ERROR(ik_launch(head_gate4_kernel<float>, blocks4, 256, 0, stream, (const float*)att, p, ldp, g_off, (float*)out, ldo, H, hdv, total4, mult, wide));
        else
            IK_RETURN_IF_ERROR(ik_launch(head_gate4_kernel<__nv_bfloat16>, blocks4, 256, 0, stream, (const __nv_bfloat16*)att, p, ldp, g_off,
                                         (__nv_bfloat16*)out, ldo, H, hdv, total4, mult, wide));
        IK_LAUNCH_STATUS();
    }
    const int blocks = (int)((total + 255) / 256 < 65535 * 16 ? (total + 255) / 256 : 65535 * 16);
    if (dtype == IK_F32)
        IK_RETURN_IF_ERROR(ik_launch(head_gate_kernel<float>, blocks, 256, 0, stream, (const float*)att, p, ldp, g_off, (float*)out, ldo, H, hdv, total, mult, wide));
    else if (dtype == IK_BF16)
        IK_RETURN_IF_ERROR(ik_launch(head_gate_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)att, p, ldp, g_off,
                                     (__nv_bfloat16*)out, ldo, H, hdv, total, mult, wide));
    else return IK_BAD_ARGUMENT;
    IK_LAUNCH_STATUS();
}

// ------------------------------------------------------------------ RMS norm with a sigmoid gate
// out[t, c] = x[t, c] * (1 / sqrt(mean_c(x^2) + eps)) * w[c] * sigmoid(p[t, g_off + c]) * mult; out has row stride ldo.
template <typename TO>
__global__ void __launch_bounds__(256)
gated_rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ p, int ldp, int g_off,
                     TO* __restrict__ out, int ldo, int d, float eps, float mult) {
    ik_pdl_wait();
    IK_AFTER_WAIT(x);
    IK_AFTER_WAIT(p);
    ik_pdl_launch_dependents();
    __shared__ float red[32];
    const float* a = x + (size_t)blockIdx.x * d;
    const float* g = p ? p + (size_t)blockIdx.x * ldp + g_off : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += 256) { const float v = a[i]; ss = fmaf(v, v, ss); }
    ss = ik_block_sum<256>(ss, red);
    const float s = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += 256) {
        float v = a[i] * s * w[i];
        if (g) v *= 1.0f / (1.0f + expf(-g[i]));
        ik_st(out, (size_t)blockIdx.x * ldo + i, v * mult);
    }
}

IK_EXPORT int ik_gated_rmsnorm(const float* x, const float* w, const float* p, int ldp, int g_off, void* out, int out_dtype,
                               int ldo, int rows, int d, float eps, float mult, cudaStream_t stream) {
    if (rows < 0 || d <= 0 || ldo < d) return IK_BAD_ARGUMENT;
    if (rows == 0) return IK_OK;
    if (out_dtype == IK_F32)
        IK_RETURN_IF_ERROR(ik_launch(gated_rmsnorm_kernel<float>, rows, 256, 0, stream, x, w, p, ldp, g_off, (float*)out, ldo, d, eps, mult));
    else if (out_dtype == IK_BF16)
        IK_RETURN_IF_ERROR(ik_launch(gated_rmsnorm_kernel<__nv_bfloat16>, rows, 256, 0, stream, x, w, p, ldp, g_off, (__nv_bfloat16*)out, ldo, d, eps, mult));
    else return IK_BAD_ARGUMENT;
    IK_LAUNCH_STATUS();
}
