// Several residual streams per token ("hyper-connections"), and norms that join the results of side-by-side branches.
//
// The streams lie token-major: xs [T, n, d] float, stream s of token t at (t * n + s) * d.  A sublayer reads one
// combination of them, u = sum_s a[s] x_s, through an RMS norm; its result y then goes into all streams at once:
// x_k' = sum_s M[s, k] x_s + b[k] y  (M indexed [from, to]).  Every sum runs over s in ascending order, so a token's
// streams depend on its own earlier values alone.
//
//   hyper_start   every stream a copy of x [T, d].
//   hyper_read    out[r, :] = rmsnorm(sum_s a[s] xs[row r, s, :]) * w, in the output type; `rows_in` picks rows (the final
//                 norm on the wanted rows only), a == nullptr means all ones (the plain sum of the streams).
//   hyper_write   the update above, in place, and with a_next / w_next the read of the NEXT sublayer from the new streams
//                 in the same pass over the token (its operand never waits for another kernel).
//   branch_norm_sum  out[t, :] (+)= sum_b c_b * rmsnorm(y_b[t, :] + bias_b) * w_b over up to four branches.
//   rmsnorm_range    an RMS norm with a weight over a column range of a wider float matrix.
#include "common.cuh"

namespace {

constexpr int HY_MAX = 16;           // most streams (a block of 256 threads brings the 16 x 16 matrix in one go)

__global__ void hyper_start_kernel(const float* __restrict__ x, float* __restrict__ xs, size_t total, int n, int d) {
    ik_pdl_wait();
    IK_AFTER_WAIT(x);
    ik_pdl_launch_dependents();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const size_t t = idx / d;
        const int i = (int)(idx - t * d);
        const float v = x[idx];
        for (int s = 0; s < n; s++) xs[(t * n + s) * d + i] = v;
    }
}

// N: the number of streams, fixed at compile time so that the sums over streams are straight-line code.
template <typename TO, int N>
__global__ void __launch_bounds__(256)
hyper_read_kernel(const float* __restrict__ xs, const int* __restrict__ rows_in, const float* __restrict__ a,
                  const float* __restrict__ w, TO* __restrict__ out, int d, float eps) {
    constexpr int n = N;
    ik_pdl_wait();
    IK_AFTER_WAIT(xs);
    IK_AFTER_WAIT(rows_in);
    ik_pdl_launch_dependents();
    __shared__ float red[32];
    const int r = blockIdx.x;
    const size_t t = rows_in ? (size_t)rows_in[r] : (size_t)r;
    const float* row = xs + t * n * d;
    float as[N];
    #pragma unroll
    for (int s = 0; s < N; s++) as[s] = a ? a[s] : 1.0f;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += 256) {
        float u = 0.f;
        #pragma unroll
        for (int s = 0; s < N; s++) u = fmaf(as[s], row[(size_t)s * d + i], u);
        ss = fmaf(u, u, ss);
    }
    ss = ik_block_sum<256>(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += 256) {
        float u = 0.f;
        #pragma unroll
        for (int s = 0; s < N; s++) u = fmaf(as[s], row[(size_t)s * d + i], u);
        ik_st(out, (size_t)r * d + i, u * inv * w[i]);
    }
}

template <typename TO, int N>
__global__ void __launch_bounds__(256)
hyper_write_kernel(float* __restrict__ xs, const float* __restrict__ y, const float* __restrict__ M, const float* __restrict__ b,
                   const float* __restrict__ a_next, const float* __restrict__ w_next, TO* __restrict__ out, int d, float eps) {
    constexpr int n = N;
    ik_pdl_wait();
    IK_AFTER_WAIT(xs);
    IK_AFTER_WAIT(y);
    ik_pdl_launch_dependents();
    __shared__ float red[32];
    __shared__ float Ms[HY_MAX * HY_MAX], bs[HY_MAX], an[HY_MAX];
    if (threadIdx.x < n * n) Ms[threadIdx.x] = M[threadIdx.x];
    if (threadIdx.x < n) { bs[threadIdx.x] = b[threadIdx.x]; an[threadIdx.x] = a_next ? a_next[threadIdx.x] : 0.f; }
    __syncthreads();
    const size_t t = blockIdx.x;
    float* row = xs + t * n * d;
    const float* yr = y + t * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += 256) {
        float old[N];
        #pragma unroll
        for (int s = 0; s < N; s++) old[s] = row[(size_t)s * d + i];
        const float yv = yr[i];
        float u = 0.f;
        #pragma unroll
        for (int k = 0; k < N; k++) {
            float v = 0.f;
            #pragma unroll
            for (int s = 0; s < N; s++) v = fmaf(Ms[s * n + k], old[s], v);
            v = fmaf(bs[k], yv, v);
            row[(size_t)k * d + i] = v;
            u = fmaf(an[k], v, u);
        }
        ss = fmaf(u, u, ss);
    }
    if (!a_next) return;
    ss = ik_block_sum<256>(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += 256) {          // a thread reads back what it wrote itself
        float u = 0.f;
        #pragma unroll
        for (int k = 0; k < N; k++) u = fmaf(an[k], row[(size_t)k * d + i], u);
        ik_st(out, t * d + i, u * inv * w_next[i]);
    }
}

struct BranchSet {
    const float* y[4];
    const float* bias[4];
    const float* w[4];
    float c[4];
    int n;
};

__global__ void __launch_bounds__(256)
branch_norm_sum_kernel(BranchSet bset, float* __restrict__ out, int d, float eps, int accumulate) {
    ik_pdl_wait();
    ik_pdl_launch_dependents();
    __shared__ float red[32];
    const size_t t = blockIdx.x;
    float inv[4];
    for (int b = 0; b < bset.n; b++) {
        const float* yr = bset.y[b] + t * d;
        const float* bias = bset.bias[b];
        float ss = 0.f;
        for (int i = threadIdx.x; i < d; i += 256) { const float v = bias ? yr[i] + bias[i] : yr[i]; ss = fmaf(v, v, ss); }
        ss = ik_block_sum<256>(ss, red);
        inv[b] = 1.0f / sqrtf(ss / (float)d + eps);
    }
    for (int i = threadIdx.x; i < d; i += 256) {
        float acc = 0.f;
        for (int b = 0; b < bset.n; b++) {
            const float v = bset.bias[b] ? bset.y[b][t * d + i] + bset.bias[b][i] : bset.y[b][t * d + i];
            acc = fmaf(bset.c[b], v * inv[b] * bset.w[b][i], acc);
        }
        out[t * d + i] = accumulate ? out[t * d + i] + acc : acc;
    }
}

template <typename TO>
__global__ void __launch_bounds__(256)
rmsnorm_range_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ w, TO* __restrict__ out, int d, float eps) {
    ik_pdl_wait();
    IK_AFTER_WAIT(x);
    ik_pdl_launch_dependents();
    __shared__ float red[32];
    const float* a = x + (size_t)blockIdx.x * ldx;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += 256) ss = fmaf(a[i], a[i], ss);
    ss = ik_block_sum<256>(ss, red);
    const float s = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += 256) ik_st(out, (size_t)blockIdx.x * d + i, a[i] * s * w[i]);
}

__global__ void add_rows_kernel(float* __restrict__ y, const float* __restrict__ v, size_t total, int d) {
    ik_pdl_wait();
    IK_AFTER_WAIT(y);
    ik_pdl_launch_dependents();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) y[idx] += v[idx % d];
}

}  // namespace

// y[t, :] += v for every row
IK_EXPORT int ik_add_rows(float* y, const float* v, int T, int d, cudaStream_t stream) {
    if (T < 0 || d <= 0 || !v) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    const size_t total = (size_t)T * d, want = (total + 255) / 256, cap = (size_t)ik_sm_count() * 16;
    IK_RETURN_IF_ERROR(ik_launch(add_rows_kernel, (int)(want < cap ? want : cap), 256, 0, stream, y, v, total, d));
    IK_LAUNCH_STATUS();
}

IK_EXPORT int ik_hyper_start(const float* x, float* xs, int T, int n, int d, cudaStream_t stream) {
    if (T < 0 || n <= 0 || d <= 0) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    const size_t total = (size_t)T * d, want = (total + 255) / 256, cap = (size_t)ik_sm_count() * 16;
    IK_RETURN_IF_ERROR(ik_launch(hyper_start_kernel, (int)(want < cap ? want : cap), 256, 0, stream, x, xs, total, n, d));
    IK_LAUNCH_STATUS();
}

IK_EXPORT int ik_hyper_read(const float* xs, const int* rows_in, const float* a, const float* w, void* out, int out_dtype, int rows,
                            int n, int d, float eps, cudaStream_t stream) {
    if (rows < 0 || n <= 0 || n > HY_MAX || d <= 0 || !w) return IK_BAD_ARGUMENT;
    if (rows == 0) return IK_OK;
    if (out_dtype != IK_F32 && out_dtype != IK_BF16) return IK_BAD_ARGUMENT;
#define IK_HR(NN)                                                                                                                   \
    case NN:                                                                                                                        \
        if (out_dtype == IK_F32)                                                                                                    \
            IK_RETURN_IF_ERROR(ik_launch(hyper_read_kernel<float, NN>, rows, 256, 0, stream, xs, rows_in, a, w, (float*)out, d, eps)); \
        else                                                                                                                        \
            IK_RETURN_IF_ERROR(ik_launch(hyper_read_kernel<__nv_bfloat16, NN>, rows, 256, 0, stream, xs, rows_in, a, w,             \
                                         (__nv_bfloat16*)out, d, eps));                                                             \
        break
    switch (n) {
        IK_HR(1); IK_HR(2); IK_HR(3); IK_HR(4); IK_HR(5); IK_HR(6); IK_HR(7); IK_HR(8);
        IK_HR(9); IK_HR(10); IK_HR(11); IK_HR(12); IK_HR(13); IK_HR(14); IK_HR(15); IK_HR(16);
    }
#undef IK_HR
    IK_LAUNCH_STATUS();
}

IK_EXPORT int ik_hyper_write(float* xs, const float* y, const float* M, const float* b, const float* a_next, const float* w_next,
                             void* out, int out_dtype, int T, int n, int d, float eps, cudaStream_t stream) {
    if (T < 0 || n <= 0 || n > HY_MAX || d <= 0 || !M || !b || (a_next && (!w_next || !out))) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    if (out_dtype != IK_F32 && out_dtype != IK_BF16) return IK_BAD_ARGUMENT;
#define IK_HW(NN)                                                                                                                   \
    case NN:                                                                                                                        \
        if (out_dtype == IK_F32)                                                                                                    \
            IK_RETURN_IF_ERROR(ik_launch(hyper_write_kernel<float, NN>, T, 256, 0, stream, xs, y, M, b, a_next, w_next, (float*)out, d, eps)); \
        else                                                                                                                        \
            IK_RETURN_IF_ERROR(ik_launch(hyper_write_kernel<__nv_bfloat16, NN>, T, 256, 0, stream, xs, y, M, b, a_next, w_next,     \
                                         (__nv_bfloat16*)out, d, eps));                                                             \
        break
    switch (n) {
        IK_HW(1); IK_HW(2); IK_HW(3); IK_HW(4); IK_HW(5); IK_HW(6); IK_HW(7); IK_HW(8);
        IK_HW(9); IK_HW(10); IK_HW(11); IK_HW(12); IK_HW(13); IK_HW(14); IK_HW(15); IK_HW(16);
    }
#undef IK_HW
    IK_LAUNCH_STATUS();
}

// y, bias, w: arrays of n pointers (bias entries may be null); c: n constants
IK_EXPORT int ik_branch_norm_sum(const float* const* y, const float* const* bias, const float* const* w, const float* c, int n,
                                 float* out, int T, int d, float eps, int accumulate, cudaStream_t stream) {
    if (T < 0 || n <= 0 || n > 4 || d <= 0 || !out) return IK_BAD_ARGUMENT;
    if (T == 0) return IK_OK;
    BranchSet bset;
    bset.n = n;
    for (int b = 0; b < 4; b++) {
        bset.y[b] = b < n ? y[b] : nullptr;
        bset.bias[b] = b < n ? bias[b] : nullptr;
        bset.w[b] = b < n ? w[b] : nullptr;
        bset.c[b] = b < n ? c[b] : 0.f;
        if (b < n && (!bset.y[b] || !bset.w[b])) return IK_BAD_ARGUMENT;
    }
    IK_RETURN_IF_ERROR(ik_launch(branch_norm_sum_kernel, T, 256, 0, stream, bset, out, d, eps, accumulate));
    IK_LAUNCH_STATUS();
}

IK_EXPORT int ik_rmsnorm_range(const float* x, int ldx, const float* w, void* out, int out_dtype, int rows, int d, float eps,
                               cudaStream_t stream) {
    if (rows < 0 || d <= 0 || ldx < d || !w) return IK_BAD_ARGUMENT;
    if (rows == 0) return IK_OK;
    if (out_dtype == IK_F32) IK_RETURN_IF_ERROR(ik_launch(rmsnorm_range_kernel<float>, rows, 256, 0, stream, x, ldx, w, (float*)out, d, eps));
    else if (out_dtype == IK_BF16)
        IK_RETURN_IF_ERROR(ik_launch(rmsnorm_range_kernel<__nv_bfloat16>, rows, 256, 0, stream, x, ldx, w, (__nv_bfloat16*)out, d, eps));
    else return IK_BAD_ARGUMENT;
    IK_LAUNCH_STATUS();
}
