// Latent attention: what stands between the projections and the attention core when keys and values are kept as one
// low-rank latent per token.
//
// A token's cache row is [c | r]: the latent c (rank values, RMS-normed with a weight) and one turning key part r (dr
// values, turned by the token's position) that all heads share.  A head's plain key would be Wuk c and its value Wuv c;
// neither is ever formed for cached tokens.  The score q_plain . (Wuk c) equals (Wuk^T q_plain) . c, so the query is
// carried into the latent's space once per token and head (a batch of small products, one per head) and attention runs
// over the rows themselves with ONE key/value head of size rank + dr whose values are the leading rank columns of its
// keys; the head's result, a weighted sum of latents, is brought to value space by Wuv afterwards (again one small
// product per head).  A layer that shares another layer's latents runs the same steps without writing rows.
//
// latent_prepare: one block per token.  From the float projections p (row stride ldp): the plain part of every query
// head goes to q_plain [T, H, dk] (the operand of the products with Wuk^T); the turning part, turned in pairs
// (2i, 2i + 1) by float(pos) * inv_freq[i], goes to columns rank .. rank + dr of q_full [T, H, rank + dr]; and, when the
// layer writes rows, c = rmsnorm(p[c_off : c_off + rank]) * c_w and the turned p[c_off + rank : + dr] go into the
// token's place in the pages (pages[page][0][position in page][rank + dr]).
#include "common.cuh"

template <typename TQ, typename TC>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const float* __restrict__ p, int ldp, int q_off, int c_off, const float* __restrict__ c_w, float eps,
                      TQ* __restrict__ q_plain, TQ* __restrict__ q_full, TC* __restrict__ k_pages, const int* __restrict__ token_seq,
                      const int* __restrict__ token_pos, const int* __restrict__ table, int table_stride,
                      const float* __restrict__ inv_freq, int H, int dk, int dr, int rank, int page_size, int n_pages,
                      int write_cache, int* status) {
    extern __shared__ __align__(16) float cs[];          // [dr/2] cos, [dr/2] sin
    __shared__ float red[32];
    ik_pdl_wait();
    IK_AFTER_WAIT(p);
    IK_AFTER_WAIT(token_seq);
    IK_AFTER_WAIT(token_pos);
    IK_AFTER_WAIT(table);
    ik_pdl_launch_dependents();
    const int t = blockIdx.x, half = dr / 2, pos = token_pos[t], hd = rank + dr;
    const float* row = p + (size_t)t * ldp;
    for (int i = threadIdx.x; i < half; i += 256) {
        const float ang = __fmul_rn((float)pos, inv_freq[i]);
        cs[i] = cosf(ang);
        cs[half + i] = sinf(ang);
    }
    float rc = 1.f;
    size_t page_off = 0;
    bool page_ok = false;
    if (write_cache) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < rank; i += 256) { const float v = row[c_off + i]; ss = fmaf(v, v, ss); }
        ss = ik_block_sum<256>(ss, red);
        rc = 1.0f / sqrtf(ss / (float)rank + eps);
        const int page = table[(size_t)token_seq[t] * table_stride + pos / page_size];
        page_ok = page >= 0 && page < n_pages;
        if (!page_ok) { if (threadIdx.x == 0) ik_set_status(status, IK_STATUS_WRITE_NO_PAGE); }
        else page_off = (size_t)page * page_size + (pos % page_size);
    }
    __syncthreads();
    const int per = dk + dr;
    for (int e = threadIdx.x; e < H * per; e += 256) {
        const int head = e / per, i = e - head * per;
        const float val = row[q_off + e];
        if (i < dk) { ik_st(q_plain, ((size_t)t * H + head) * dk + i, val); continue; }
        const int ii = i - dk, f = ii >> 1;
        const bool first = (ii & 1) == 0;
        const float other = row[q_off + (first ? e + 1 : e - 1)];
        const float c = cs[f], s = cs[half + f];
        // (u, v) -> (u c - v s, v c + u s); `first` holds u
        const float turned = first ? __fsub_rn(__fmul_rn(val, c), __fmul_rn(other, s)) : __fadd_rn(__fmul_rn(val, c), __fmul_rn(other, s));
        ik_st(q_full, ((size_t)t * H + head) * hd + rank + ii, turned);
    }
    if (!page_ok) return;
    TC* dst = k_pages + page_off * hd;
    for (int i = threadIdx.x; i < rank; i += 256) ik_st(dst, i, row[c_off + i] * rc * c_w[i]);
    for (int ii = threadIdx.x; ii < dr; ii += 256) {
        const int f = ii >> 1;
        const bool first = (ii & 1) == 0;
        const float val = row[c_off + rank + ii], other = row[c_off + rank + (first ? ii + 1 : ii - 1)];
        const float c = cs[f], s = cs[half + f];
        ik_st(dst, rank + ii, first ? __fsub_rn(__fmul_rn(val, c), __fmul_rn(other, s)) : __fadd_rn(__fmul_rn(val, c), __fmul_rn(other, s)));
    }
}

IK_EXPORT int ik_latent_prepare(const float* p, int ldp, int q_off, int c_off, const float* c_w, float eps, void* q_plain, void* q_full,
                                int q_dtype, void* k_pages, int cache_dtype, const int* token_seq, const int* token_pos,
                                const int* table, int table_stride, const float* inv_freq, int T, int H, int dk, int dr, int rank,
                                int page_size, int n_pages, int write_cache, int* status, cudaStream_t stream) {
    // H = 0: the queries are made elsewhere (behind a latent of their own) and only the row is written; dr = 0: no turning part
    if (T < 0 || H < 0 || (H > 0 && (dk <= 0 || !q_plain || (dr > 0 && !q_full))) || dr < 0 || (dr & 1) || rank <= 0 || page_size <= 0 ||
        (dr > 0 && !inv_freq))
        return IK_BAD_ARGUMENT;
    if (write_cache && (!c_w || !k_pages)) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    const size_t smem = (size_t)dr * sizeof(float);
#define IK_LP(TQ, TC)                                                                                                            \
    IK_RETURN_IF_ERROR(ik_launch(latent_prepare_kernel<TQ, TC>, T, 256, smem, stream, p, ldp, q_off, c_off, c_w, eps, (TQ*)q_plain,   \
                                 (TQ*)q_full, (TC*)k_pages, token_seq, token_pos, table, table_stride, inv_freq, H, dk, dr, rank,  \
                                 page_size, n_pages, write_cache, status))
    if (q_dtype == IK_F32 && cache_dtype == IK_F32) IK_LP(float, float);
    else if (q_dtype == IK_BF16 && cache_dtype == IK_BF16) IK_LP(__nv_bfloat16, __nv_bfloat16);
    else return IK_BAD_ARGUMENT;
#undef IK_LP
    IK_LAUNCH_STATUS();
}
