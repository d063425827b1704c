// Attention over a paged bfloat16 cache whose key rows carry their own values: a row of IK_HD numbers is the key, its
// leading IK_HDV numbers are the value (a latent that serves as both).  Compiled once per (IK_HD, IK_HDV).
//
// All query heads of a key/value group read the same rows, so the heads ARE the rows of the tensor-core tile: a block
// owns up to 32 (token, head) rows of one sequence and one key/value head, tokens_per_block consecutive tokens times
// heads_per_block heads, and walks the pages its rows can see (64 keys each).  Every key row is read once for all of
// them, for the scores and for the values.
//
// Eight warps form two row groups of 16 rows and four column groups.  For a page, warp (rg, cg) computes the scores of
// its 16 rows against the page's keys 16 cg .. 16 cg + 15 over all IK_HD dimensions (mma.sync m16n8k16, float
// accumulators), the row maxima are joined across the four warps through shared memory, the weights exp2(s - m) go to
// shared memory as bfloat16, and the warp then adds P V for its quarter of the IK_HDV value columns, reading the same
// shared key rows transposed.  Scores, maximum, sum and the rescaling are float, in base 2.  Pages are loaded with
// cp.async into two buffers, the next page while this one is used.
//
// Prefill and decode use the same kernel.  With n_splits > 1 the pages of a block's range are cut into n_splits runs
// of chunk_pages; each block writes an unnormalised partial (maximum, sum, output) and a second kernel merges them in
// order.  Keys beyond a row's position or outside its window are masked by position.  Options: a window, and a sink (one
// more key of score 0 without a value).
#include <math.h>
#define IK_FAMILY 4
#include "common.cuh"

#if !defined(IK_HD) || !defined(IK_HDV)
#error "compile with -DIK_HD=<key row size> -DIK_HDV=<leading columns that are the value>"
#endif

namespace {

typedef __nv_bfloat16 bf16;
constexpr int HD = IK_HD, HDV = IK_HDV, PAGE = 64;
constexpr int RG = 2, CG = 4, BM = 16 * RG, NW = RG * CG, THREADS = 32 * NW;
constexpr int VC = HDV / CG;               // value columns of a warp
constexpr int LD = HD + 8;                 // padded rows: consecutive rows fall into different banks
constexpr int LDP = PAGE + 8;
static_assert(HD % 16 == 0 && HDV % (16 * CG) == 0 && HDV <= HD && HDV >= 16 * CG, "sizes");
constexpr size_t SMEM = (size_t)(BM * LD + 2 * PAGE * LD + BM * LDP) * sizeof(bf16) + (size_t)RG * CG * 16 * sizeof(float);

__device__ __forceinline__ void cp16(void* smem, const void* gmem, bool valid) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" :: "r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n"); }
__device__ __forceinline__ void cp_wait_all() { asm volatile("cp.async.wait_group 0;\n"); }
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const void* p) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], const void* p) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// q [T, nh, HD]; k_pages [n_pages, nkv, PAGE, HD]; out [T, nh, HDV] (n_splits == 1) or part_o [T * nh, n_splits, HDV]
// and part_ml [T * nh, n_splits, 2].  grid: (token blocks * n_splits, nkv * head blocks, sequences).
__global__ void __launch_bounds__(THREADS, 1)
attn_latent_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages, bf16* __restrict__ out,
                   float* __restrict__ part_o, float* __restrict__ part_ml, const int* __restrict__ cu_seqlens,
                   const int* __restrict__ kv_lens, const int* __restrict__ table, int table_stride, int nh, int nkv,
                   int heads_per_block, int tokens_per_block, float scale_log2e, int window, int sink, int n_pages,
                   int chunk_pages, int n_splits, int* status) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    ik_pdl_wait();
    ik_pdl_launch_dependents();
    bf16* Qs = (bf16*)smem_raw;                  // [BM][LD]
    bf16* Ks = Qs + BM * LD;                     // [2][PAGE][LD]
    bf16* Ps = Ks + 2 * PAGE * LD;               // [BM][LDP]
    float* red = (float*)(Ps + BM * LDP);        // [RG][CG][16]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int rg = warp / CG, cg = warp % CG;
    const int b = blockIdx.z;
    const int tok0 = cu_seqlens[b], n_new = cu_seqlens[b + 1] - tok0, kv_len = kv_lens[b];
    const int tb = blockIdx.x / n_splits, split = blockIdx.x % n_splits;
    const int t_lo = tb * tokens_per_block;
    if (t_lo >= n_new) return;
    const int ntok = min(tokens_per_block, n_new - t_lo);
    const int group = nh / nkv, hblocks = (group + heads_per_block - 1) / heads_per_block;
    const int kvh = blockIdx.y / hblocks, hb = blockIdx.y % hblocks;
    const int h0 = kvh * group + hb * heads_per_block, nhead = min(heads_per_block, group - hb * heads_per_block);
    const int pos_lo = kv_len - n_new + t_lo, pos_hi = pos_lo + ntok - 1;
    const int j_first = (window > 0 && pos_lo + 1 > window) ? pos_lo + 1 - window : 0;
    const int p_first = j_first / PAGE + split * chunk_pages;
    const int p_last = min(pos_hi / PAGE, p_first + chunk_pages - 1);
    const int n_iter = p_last - p_first + 1;                         // may be <= 0 for a late split

    // this thread's two rows of its row group
    int row_tok[2], row_head[2], row_pos[2];
    bool row_ok[2];
    #pragma unroll
    for (int e = 0; e < 2; e++) {
        const int r = rg * 16 + g + 8 * e, tk = r / heads_per_block, hh = r - tk * heads_per_block;
        row_ok[e] = tk < ntok && hh < nhead;
        row_tok[e] = tok0 + t_lo + tk;
        row_head[e] = h0 + hh;
        row_pos[e] = pos_lo + tk;
    }
    const bool group_used = rg * 16 < ntok * heads_per_block;        // warp-uniform: the row group has rows at all

    auto load_page = [&](int p, int buf) {
        const int page = table[(size_t)b * table_stride + p];
        const bool ok = page >= 0 && page < n_pages;
        if (!ok && tid == 0) ik_set_status(status, IK_STATUS_READ_NO_PAGE);
        const bf16* src = k_pages + ((size_t)(ok ? page : 0) * nkv + kvh) * PAGE * HD;
        bf16* dst = Ks + (size_t)buf * PAGE * LD;
        constexpr int CH = HD / 8;
        for (int c = tid; c < PAGE * CH; c += THREADS) {
            const int r = c / CH, x = c - r * CH;
            cp16(dst + r * LD + x * 8, src + (size_t)r * HD + x * 8, ok);
        }
    };

    if (n_iter > 0) {
        constexpr int CH = HD / 8;
        for (int c = tid; c < BM * CH; c += THREADS) {
            const int r = c / CH, x = c - r * CH, tk = r / heads_per_block, hh = r - tk * heads_per_block;
            const bool ok = tk < ntok && hh < nhead;
            const bf16* src = q + ((size_t)(tok0 + t_lo + (ok ? tk : 0)) * nh + h0 + (ok ? hh : 0)) * HD + x * 8;
            cp16(Qs + r * LD + x * 8, src, ok);
        }
        load_page(p_first, 0);
        cp_commit();
    }

    float o[VC / 8][4];
    #pragma unroll
    for (int n = 0; n < VC / 8; n++)
        #pragma unroll
        for (int e = 0; e < 4; e++) o[n][e] = 0.f;
    // the sink opens the running softmax of the first split: maximum 0, and its weight 1 in one thread's part of the sum
    const bool with_sink = sink && split == 0;
    float m_i[2] = {with_sink ? 0.f : -INFINITY, with_sink ? 0.f : -INFINITY};
    float l_i[2] = {(with_sink && cg == 0 && t == 0) ? 1.f : 0.f, (with_sink && cg == 0 && t == 0) ? 1.f : 0.f};

    for (int i = 0; i < n_iter; i++) {
        const int p = p_first + i, buf = i & 1;
        cp_wait_all();
        __syncthreads();
        if (i + 1 < n_iter) { load_page(p + 1, buf ^ 1); cp_commit(); }
        const bf16* Kb = Ks + (size_t)buf * PAGE * LD;

        float s[2][4];
        #pragma unroll
        for (int n = 0; n < 2; n++)
            #pragma unroll
            for (int e = 0; e < 4; e++) s[n][e] = 0.f;
        if (group_used) {
            const bf16* qa = Qs + (rg * 16 + (lane & 15)) * LD + (lane >> 4) * 8;
            const bf16* kb = Kb + (cg * 16 + (lane >> 4) * 8 + (lane & 7)) * LD + ((lane >> 3) & 1) * 8;
            #pragma unroll 4
            for (int kk = 0; kk < HD / 16; kk++) {
                uint32_t a[4], bk[4];
                ldsm4(a, qa + kk * 16);
                ldsm4(bk, kb + kk * 16);
                mma(s[0], a, bk[0], bk[1]);
                mma(s[1], a, bk[2], bk[3]);
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
        #pragma unroll
        for (int n = 0; n < 2; n++)
            #pragma unroll
            for (int e = 0; e < 4; e++) {
                const int r = e >> 1, j = p * PAGE + cg * 16 + n * 8 + 2 * t + (e & 1);
                const bool vis = row_ok[r] && j <= row_pos[r] && (window <= 0 || j > row_pos[r] - window);
                s[n][e] = vis ? s[n][e] * scale_log2e : -INFINITY;
                mx[r] = fmaxf(mx[r], s[n][e]);
            }
        #pragma unroll
        for (int r = 0; r < 2; r++) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        }
        if (t == 0) {
            red[(rg * CG + cg) * 16 + g] = mx[0];
            red[(rg * CG + cg) * 16 + g + 8] = mx[1];
        }
        __syncthreads();
        float alpha[2];
        #pragma unroll
        for (int r = 0; r < 2; r++) {
            float m_new = m_i[r];
            #pragma unroll
            for (int c = 0; c < CG; c++) m_new = fmaxf(m_new, red[(rg * CG + c) * 16 + g + 8 * r]);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            alpha[r] = exp2f(m_i[r] - m_use);                       // 0 while nothing was seen (m_i = -inf)
            m_i[r] = m_new;
            float sum = 0.f;
            #pragma unroll
            for (int n = 0; n < 2; n++) {
                const float p0 = exp2f(s[n][2 * r] - m_use), p1 = exp2f(s[n][2 * r + 1] - m_use);
                sum += p0 + p1;
                *reinterpret_cast<uint32_t*>(Ps + (rg * 16 + g + 8 * r) * LDP + cg * 16 + n * 8 + 2 * t) = pack_bf16(p0, p1);
            }
            l_i[r] = l_i[r] * alpha[r] + sum;
        }
        __syncthreads();
        if (group_used) {
            #pragma unroll
            for (int n = 0; n < VC / 8; n++) {
                o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
                o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
            }
            const bf16* pa = Ps + (rg * 16 + (lane & 15)) * LDP + (lane >> 4) * 8;
            const bf16* vb = Kb + (((lane >> 3) & 1) * 8 + (lane & 7)) * LD + cg * VC + (lane >> 4) * 8;
            #pragma unroll
            for (int ks = 0; ks < PAGE / 16; ks++) {
                uint32_t a[4];
                ldsm4(a, pa + ks * 16);
                #pragma unroll
                for (int np = 0; np < VC / 16; np++) {
                    uint32_t bv[4];
                    ldsm4t(bv, vb + (size_t)ks * 16 * LD + np * 16);
                    mma(o[2 * np], a, bv[0], bv[1]);
                    mma(o[2 * np + 1], a, bv[2], bv[3]);
                }
            }
        }
    }

    // the sum of a row: over the four threads of a quad, then over the four column groups
    #pragma unroll
    for (int r = 0; r < 2; r++) {
        l_i[r] += __shfl_xor_sync(0xffffffffu, l_i[r], 1);
        l_i[r] += __shfl_xor_sync(0xffffffffu, l_i[r], 2);
    }
    __syncthreads();
    if (t == 0) {
        red[(rg * CG + cg) * 16 + g] = l_i[0];
        red[(rg * CG + cg) * 16 + g + 8] = l_i[1];
    }
    __syncthreads();
    #pragma unroll
    for (int r = 0; r < 2; r++) {
        if (!row_ok[r]) continue;
        float l = 0.f;
        #pragma unroll
        for (int c = 0; c < CG; c++) l += red[(rg * CG + c) * 16 + g + 8 * r];
        const size_t grow = (size_t)row_tok[r] * nh + row_head[r];
        if (n_splits == 1) {
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            bf16* dst = out + grow * HDV + cg * VC + 2 * t;
            #pragma unroll
            for (int n = 0; n < VC / 8; n++)
                *reinterpret_cast<uint32_t*>(dst + n * 8) = pack_bf16(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
        } else {
            float* dst = part_o + (grow * n_splits + split) * HDV + cg * VC + 2 * t;
            #pragma unroll
            for (int n = 0; n < VC / 8; n++)
                *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][2 * r], o[n][2 * r + 1]);
            if (cg == 0 && t == 0) {
                part_ml[(grow * n_splits + split) * 2] = m_i[r];
                part_ml[(grow * n_splits + split) * 2 + 1] = l;
            }
        }
    }
}

// One block per (token, head) row: merges the partials of the row's splits in order and writes the normalised output.
// A split that saw nothing has maximum -inf and sum 0.  The sink is already inside the first split's maximum and sum.
__global__ void attn_latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         bf16* __restrict__ out, int n_splits) {
    ik_pdl_wait();
    ik_pdl_launch_dependents();
    const size_t row = blockIdx.x;
    float mm = -INFINITY;
    for (int s = 0; s < n_splits; s++) mm = fmaxf(mm, part_ml[(row * n_splits + s) * 2]);
    const float m_use = mm == -INFINITY ? 0.f : mm;
    float ll = 0.f;
    for (int s = 0; s < n_splits; s++) ll += part_ml[(row * n_splits + s) * 2 + 1] * exp2f(part_ml[(row * n_splits + s) * 2] - m_use);
    const float inv = ll > 0.f ? 1.0f / ll : 0.f;
    for (int x = threadIdx.x; x < HDV; x += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; s++) {
            const float m_s = part_ml[(row * n_splits + s) * 2];
            if (m_s != -INFINITY) acc += part_o[(row * n_splits + s) * HDV + x] * exp2f(m_s - m_use);
        }
        out[row * HDV + x] = __float2bfloat16_rn(acc * inv);
    }
}

}  // namespace

IK_EXPORT int ik_attn_latent_rows() { return BM; }

// T: rows of q (all tokens of the step).  n_splits * chunk_pages must cover the pages any block's rows can see.
IK_EXPORT int ik_attn_latent(const void* q, const void* k_pages, void* out, float* part_o, float* part_ml,
                             const int* cu_seqlens, const int* kv_lens, const int* table, int table_stride, int T, int B,
                             int max_new, int nh, int nkv, float scale, int window, int sink, int page_size, int n_pages,
                             int chunk_pages, int n_splits, int* status, cudaStream_t stream) {
    if (B <= 0 || max_new <= 0 || nh <= 0 || nkv <= 0 || nh % nkv || page_size != PAGE || chunk_pages <= 0 || n_splits <= 0 ||
        B > 65535 || (n_splits > 1 && (!part_o || !part_ml)))
        return IK_BAD_ARGUMENT;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_latent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int group = nh / nkv;
    const int hpb = group < BM ? group : BM, tpb = BM / hpb, hblocks = (group + hpb - 1) / hpb;
    if ((long long)nkv * hblocks > 65535) return IK_BAD_ARGUMENT;
    dim3 grid((unsigned)((max_new + tpb - 1) / tpb) * n_splits, nkv * hblocks, B);
    IK_RETURN_IF_ERROR(ik_launch(attn_latent_kernel, grid, THREADS, SMEM, stream, (const bf16*)q, (const bf16*)k_pages, (bf16*)out,
                                 part_o, part_ml, cu_seqlens, kv_lens, table, table_stride, nh, nkv, hpb, tpb,
                                 scale * 1.4426950408889634f, window, sink, n_pages, chunk_pages, n_splits, status));
    if (n_splits > 1)
        IK_RETURN_IF_ERROR(ik_launch_family(IK_FAMILY_ATTENTION_MERGE, attn_latent_merge_kernel, dim3((unsigned)T * nh), 128, 0, stream,
                                            (const float*)part_o, (const float*)part_ml, (bf16*)out, n_splits));
    IK_LAUNCH_STATUS();
}
