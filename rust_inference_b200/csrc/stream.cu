// Work on the float32 hidden stream that needs no statistics of a row, and the sums of normalised branches.
//
//   dyt_norm        y = tanh(alpha x) w + b  (a norm without mean or variance: every element by itself), optionally
//                   on gathered rows, into the run dtype
//   stream_update   the end of a sublayer whose result is normalised before it joins the stream, in one pass:
//                       r = stream + post(branch + branch_bias)          post: tanh(alpha x) w + b, or the identity
//                       history[index + 1] = r;  r = sum_j depth_w[j] history[j]   (a weighted sum over the results of
//                                                                                   all layers so far and the embedding)
//                       stream = r;  next_out = next(r)                  next: tanh(alpha x) w + b, into the run dtype
//                   every stage optional; the branch buffer is left zeroed for its next user
//   normed_sum      out (+)= sum_m scale_m * rmsnorm(x_m + bias_m) * w_m over up to four branch buffers (the members of a
//                   mixer made of several mixers, each normalised over the model width before they are added);
//                   the buffers are left zeroed
//   xielu           act(z) = a_p z^2 + z/2 for z > 0, a_n (e^z - 1 - z) + z/2 otherwise, a_p = softplus(p),
//                   a_n = 1/2 + softplus(q), p and q read from device memory
//   add_row_bias    x[t, :] += bias
//
// All arithmetic is float32 with accurate tanhf / expf / expm1f.  Data an earlier kernel of the step wrote is read
// after `wait_for_previous_kernels()` through plain pointers.
#include "common.cuh"

using namespace ri;

namespace {

__device__ __forceinline__ float softplus_f32(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <typename T>
__global__ void dyt_norm_kernel(const float* x, const float* __restrict__ w, const float* __restrict__ b,
                                const float* __restrict__ alpha, const int* rows, T* __restrict__ out, int n_rows, int n) {
    let_next_kernel_start();
    const float a = alpha[0];
    wait_for_previous_kernels();
    const size_t total = (size_t)n_rows * n;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int r = (int)(i / n), c = (int)(i % n);
        const int src = rows != nullptr ? rows[r] : r;
        out[i] = from_f32<T>(fmaf(tanhf(a * x[(size_t)src * n + c]), w[c], b[c]));
    }
}

struct StreamUpdate {
    float* stream;
    float* branch;                 // null: nothing joins the stream
    const float* branch_bias;      // null: none
    const float* post_w;           // null: the branch joins as it is
    const float* post_b;
    const float* post_alpha;
    float* history;                // null: no sum over depth; else [depth_index + 2 or more][n_tokens * n]
    const float* depth_w;          // [depth_index + 2]
    int depth_index;
    int store_result;              // whether history[depth_index + 1] is written (a later layer reads it)
    const float* next_w;           // null: no norm of the new stream
    const float* next_b;
    const float* next_alpha;
    void* next_out;
    int n_tokens, n;
};

template <typename T>
__global__ void __launch_bounds__(256) stream_update_kernel(StreamUpdate p) {
    let_next_kernel_start();
    const float pa = p.post_w != nullptr ? p.post_alpha[0] : 0.f;
    const float na = p.next_w != nullptr ? p.next_alpha[0] : 0.f;
    wait_for_previous_kernels();
    const size_t total = (size_t)p.n_tokens * p.n;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % p.n);
        float r = p.stream[i];
        if (p.branch != nullptr) {
            float v = p.branch[i];
            p.branch[i] = 0.f;
            if (p.branch_bias != nullptr) v += p.branch_bias[c];
            r += p.post_w != nullptr ? fmaf(tanhf(pa * v), p.post_w[c], p.post_b[c]) : v;
        }
        if (p.history != nullptr) {
            const int last = p.depth_index + 1;
            if (p.store_result) p.history[(size_t)last * total + i] = r;
            float acc = 0.f;
            for (int j = 0; j < last; ++j) acc = fmaf(p.depth_w[j], p.history[(size_t)j * total + i], acc);
            r = fmaf(p.depth_w[last], r, acc);
        }
        p.stream[i] = r;
        if (p.next_w != nullptr)
            reinterpret_cast<T*>(p.next_out)[i] = from_f32<T>(fmaf(tanhf(na * r), p.next_w[c], p.next_b[c]));
    }
}

constexpr int MAX_MEMBERS = 4;
struct NormedSum {
    float* x[MAX_MEMBERS];
    const float* bias[MAX_MEMBERS];
    const float* w[MAX_MEMBERS];
    float scale[MAX_MEMBERS];
    int members;
};

// A block per row; the row of every member is read twice (sum of squares, then the weighted values): it stays in L1.
__global__ void __launch_bounds__(256) normed_sum_kernel(NormedSum p, float* out, int n, float eps, int accumulate) {
    __shared__ float scratch[33];
    let_next_kernel_start();
    wait_for_previous_kernels();
    const size_t row = (size_t)blockIdx.x * n;
    float inv[MAX_MEMBERS];
    for (int m = 0; m < p.members; ++m) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < n; c += blockDim.x) {
            const float v = p.x[m][row + c] + (p.bias[m] != nullptr ? p.bias[m][c] : 0.f);
            ss = fmaf(v, v, ss);
        }
        ss = block_sum(ss, scratch);
        inv[m] = p.scale[m] / sqrtf(ss / (float)n + eps);
    }
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
        float acc = accumulate ? out[row + c] : 0.f;
        for (int m = 0; m < p.members; ++m) {
            const float v = p.x[m][row + c] + (p.bias[m] != nullptr ? p.bias[m][c] : 0.f);
            p.x[m][row + c] = 0.f;
            acc = fmaf(v * inv[m], p.w[m][c], acc);
        }
        out[row + c] = acc;
    }
}

template <typename T>
__global__ void xielu_kernel(const T* x, T* out, const float* __restrict__ pq, size_t total) {
    let_next_kernel_start();
    const ActForm form = load_act_form(pq);
    wait_for_previous_kernels();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f32<T>(act_f32(to_f32<T>(x[i]), form));
}

__global__ void add_row_bias_kernel(float* x, const float* __restrict__ bias, int n, size_t total) {
    let_next_kernel_start();
    wait_for_previous_kernels();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        x[i] += bias[i % n];
}

inline int blocks_for(size_t total, int threads) {
    const size_t b = (total + threads - 1) / threads;
    return (int)(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

}  // namespace

RI_API int ri_dyt_norm(const float* x, const float* w, const float* b, const float* alpha, const int* rows, void* out,
                       int out_dtype, int n_rows, int n, cudaStream_t stream) {
    if (n_rows <= 0 || n <= 0) return 0;
    const size_t total = (size_t)n_rows * n;
    cudaError_t e;
    if (out_dtype == RI_F32)
        e = launch_dependent(dyt_norm_kernel<float>, blocks_for(total, 256), 256, 0, stream, x, w, b, alpha, rows, (float*)out, n_rows, n);
    else if (out_dtype == RI_BF16)
        e = launch_dependent(dyt_norm_kernel<__nv_bfloat16>, blocks_for(total, 256), 256, 0, stream, x, w, b, alpha, rows,
                             (__nv_bfloat16*)out, n_rows, n);
    else
        return fail("dyt_norm: unknown dtype %d", out_dtype);
    return check_launch(e, "dyt_norm");
}

RI_API int ri_stream_update(float* stream_x, float* branch, const float* branch_bias, const float* post_w, const float* post_b,
                            const float* post_alpha, float* history, const float* depth_w, int depth_index, int store_result,
                            const float* next_w, const float* next_b, const float* next_alpha, void* next_out, int next_dtype,
                            int n_tokens, int n, cudaStream_t stream) {
    if (n_tokens <= 0 || n <= 0) return 0;
    if (history != nullptr && (depth_w == nullptr || depth_index < 0)) return fail("stream_update: a sum over depth needs its weights");
    if (post_w != nullptr && (post_b == nullptr || post_alpha == nullptr)) return fail("stream_update: the norm of the branch is incomplete");
    if (next_w != nullptr && (next_b == nullptr || next_alpha == nullptr || next_out == nullptr)) return fail("stream_update: the norm of the new stream is incomplete");
    StreamUpdate p{stream_x, branch, branch_bias, post_w, post_b, post_alpha, history, depth_w, depth_index, store_result,
                   next_w, next_b, next_alpha, next_out, n_tokens, n};
    const size_t total = (size_t)n_tokens * n;
    cudaError_t e;
    if (next_w == nullptr || next_dtype == RI_F32)
        e = launch_dependent(stream_update_kernel<float>, blocks_for(total, 256), 256, 0, stream, p);
    else if (next_dtype == RI_BF16)
        e = launch_dependent(stream_update_kernel<__nv_bfloat16>, blocks_for(total, 256), 256, 0, stream, p);
    else
        return fail("stream_update: unknown dtype %d", next_dtype);
    return check_launch(e, "stream_update");
}

RI_API int ri_normed_sum(float* const* xs, const float* const* biases, const float* const* ws, const float* scales, int members,
                         float* out, int n_tokens, int n, float eps, int accumulate, cudaStream_t stream) {
    if (n_tokens <= 0 || n <= 0) return 0;
    if (members < 1 || members > MAX_MEMBERS) return fail("normed_sum: %d members, at most %d", members, MAX_MEMBERS);
    NormedSum p{};
    p.members = members;
    for (int m = 0; m < members; ++m) {
        p.x[m] = xs[m];
        p.bias[m] = biases[m];
        p.w[m] = ws[m];
        p.scale[m] = scales[m];
    }
    cudaError_t e = launch_dependent(normed_sum_kernel, n_tokens, 256, 0, stream, p, out, n, eps, accumulate);
    return check_launch(e, "normed_sum");
}

RI_API int ri_xielu(const void* x, void* out, int dtype, const float* pq, long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    cudaError_t e;
    if (dtype == RI_F32)
        e = launch_dependent(xielu_kernel<float>, blocks_for((size_t)total, 256), 256, 0, stream, (const float*)x, (float*)out, pq, (size_t)total);
    else if (dtype == RI_BF16)
        e = launch_dependent(xielu_kernel<__nv_bfloat16>, blocks_for((size_t)total, 256), 256, 0, stream, (const __nv_bfloat16*)x,
                             (__nv_bfloat16*)out, pq, (size_t)total);
    else
        return fail("xielu: unknown dtype %d", dtype);
    return check_launch(e, "xielu");
}

RI_API int ri_add_row_bias(float* x, const float* bias, int n_rows, int n, cudaStream_t stream) {
    if (n_rows <= 0 || n <= 0) return 0;
    const size_t total = (size_t)n_rows * n;
    cudaError_t e = launch_dependent(add_row_bias_kernel, blocks_for(total, 256), 256, 0, stream, x, bias, n, total);
    return check_launch(e, "add_row_bias");
}

RI_DEFINE_LAST_ERROR()
