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
#include <initializer_list>

using namespace ri;

namespace {

__device__ __forceinline__ float softplus_f32(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// V consecutive floats of a row as one access (V = 4: 16 bytes; rows and pointers must allow it) or one by one.
template <int V> struct Pack { float v[V]; };
template <int V> __device__ __forceinline__ Pack<V> load_pack(const float* p) {
    Pack<V> r;
    if constexpr (V == 4) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w;
    } else {
#pragma unroll
        for (int k = 0; k < V; ++k) r.v[k] = p[k];
    }
    return r;
}
template <int V> __device__ __forceinline__ Pack<V> zero_pack() {
    Pack<V> r;
#pragma unroll
    for (int k = 0; k < V; ++k) r.v[k] = 0.f;
    return r;
}
template <int V> __device__ __forceinline__ void store_pack(float* p, const Pack<V>& r) {
    if constexpr (V == 4) {
        *reinterpret_cast<float4*>(p) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
    } else {
#pragma unroll
        for (int k = 0; k < V; ++k) p[k] = r.v[k];
    }
}
template <int V> __device__ __forceinline__ void store_pack(__nv_bfloat16* p, const Pack<V>& r) {
    if constexpr (V == 4) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(r.v[0], r.v[1]), hi = __floats2bfloat162_rn(r.v[2], r.v[3]);
        uint2 u;
        u.x = *reinterpret_cast<const uint32_t*>(&lo);
        u.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = u;
    } else {
#pragma unroll
        for (int k = 0; k < V; ++k) p[k] = __float2bfloat16_rn(r.v[k]);
    }
}

// A thread owns V columns and walks down the rows (blockIdx.y, then in steps of gridDim.y): the vectors of its columns
// are read once, and no index is ever divided.
template <typename T, int V>
__global__ void __launch_bounds__(128) dyt_norm_kernel(const float* x, const float* __restrict__ w, const float* __restrict__ b,
                                const float* __restrict__ alpha, const int* rows, T* __restrict__ out, int n_rows, int n) {
    let_next_kernel_start();
    const float a = alpha[0];
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    const bool mine = c < n;
    const Pack<V> wv = mine ? load_pack<V>(w + c) : zero_pack<V>(), bv = mine ? load_pack<V>(b + c) : zero_pack<V>();
    wait_for_previous_kernels();
    if (!mine) return;
    for (int r = blockIdx.y; r < n_rows; r += gridDim.y) {
        const int src = rows != nullptr ? rows[r] : r;
        Pack<V> v = load_pack<V>(x + (size_t)src * n + c);
#pragma unroll
        for (int k = 0; k < V; ++k) v.v[k] = fmaf(tanhf(a * v.v[k]), wv.v[k], bv.v[k]);
        store_pack<V>(out + (size_t)r * n + c, v);
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

template <typename T, int V>
__global__ void __launch_bounds__(128) stream_update_kernel(StreamUpdate p) {
    let_next_kernel_start();
    const float pa = p.post_w != nullptr ? p.post_alpha[0] : 0.f;
    const float na = p.next_w != nullptr ? p.next_alpha[0] : 0.f;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    const bool mine = c < p.n;
    const bool post = p.post_w != nullptr && mine, next = p.next_w != nullptr && mine;
    const Pack<V> bias = (p.branch_bias != nullptr && mine) ? load_pack<V>(p.branch_bias + c) : zero_pack<V>();
    const Pack<V> pw = post ? load_pack<V>(p.post_w + c) : zero_pack<V>(), pb = post ? load_pack<V>(p.post_b + c) : zero_pack<V>();
    const Pack<V> nw = next ? load_pack<V>(p.next_w + c) : zero_pack<V>(), nb = next ? load_pack<V>(p.next_b + c) : zero_pack<V>();
    wait_for_previous_kernels();
    if (!mine) return;
    const size_t total = (size_t)p.n_tokens * p.n;
    const int last = p.depth_index + 1;
    for (int row = blockIdx.y; row < p.n_tokens; row += gridDim.y) {
        const size_t i = (size_t)row * p.n + c;
        Pack<V> r = load_pack<V>(p.stream + i);
        if (p.branch != nullptr) {
            const Pack<V> v = load_pack<V>(p.branch + i);
            store_pack<V>(p.branch + i, zero_pack<V>());
#pragma unroll
            for (int k = 0; k < V; ++k) {
                const float x = v.v[k] + bias.v[k];
                r.v[k] += p.post_w != nullptr ? fmaf(tanhf(pa * x), pw.v[k], pb.v[k]) : x;
            }
        }
        if (p.history != nullptr) {
            if (p.store_result) store_pack<V>(p.history + (size_t)last * total + i, r);
            Pack<V> acc = zero_pack<V>();
            for (int j = 0; j < last; ++j) {
                const float wj = p.depth_w[j];
                const Pack<V> hj = load_pack<V>(p.history + (size_t)j * total + i);
#pragma unroll
                for (int k = 0; k < V; ++k) acc.v[k] = fmaf(wj, hj.v[k], acc.v[k]);
            }
            const float wl = p.depth_w[last];
#pragma unroll
            for (int k = 0; k < V; ++k) r.v[k] = fmaf(wl, r.v[k], acc.v[k]);
        }
        store_pack<V>(p.stream + i, r);
        if (p.next_w != nullptr) {
#pragma unroll
            for (int k = 0; k < V; ++k) r.v[k] = fmaf(tanhf(na * r.v[k]), nw.v[k], nb.v[k]);
            store_pack<V>(reinterpret_cast<T*>(p.next_out) + i, r);
        }
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
// V = 4: 16-byte accesses where the rows and pointers allow them.
template <int V>
__global__ void __launch_bounds__(256) normed_sum_kernel(NormedSum p, float* out, int n, float eps, int accumulate) {
    __shared__ float scratch[33];
    let_next_kernel_start();
    wait_for_previous_kernels();
    const size_t row = (size_t)blockIdx.x * n;
    float inv[MAX_MEMBERS];
    for (int m = 0; m < p.members; ++m) {
        float ss = 0.f;
        for (int c = threadIdx.x * V; c < n; c += blockDim.x * V) {
            const Pack<V> x = load_pack<V>(p.x[m] + row + c);
            const Pack<V> bv = p.bias[m] != nullptr ? load_pack<V>(p.bias[m] + c) : zero_pack<V>();
#pragma unroll
            for (int k = 0; k < V; ++k) {
                const float v = x.v[k] + bv.v[k];
                ss = fmaf(v, v, ss);
            }
        }
        ss = block_sum(ss, scratch);
        inv[m] = p.scale[m] / sqrtf(ss / (float)n + eps);
    }
    for (int c = threadIdx.x * V; c < n; c += blockDim.x * V) {
        Pack<V> acc = accumulate ? load_pack<V>(out + row + c) : zero_pack<V>();
        for (int m = 0; m < p.members; ++m) {
            const Pack<V> x = load_pack<V>(p.x[m] + row + c);
            const Pack<V> bv = p.bias[m] != nullptr ? load_pack<V>(p.bias[m] + c) : zero_pack<V>();
            const Pack<V> wv = load_pack<V>(p.w[m] + c);
            store_pack<V>(p.x[m] + row + c, zero_pack<V>());
#pragma unroll
            for (int k = 0; k < V; ++k) acc.v[k] = fmaf((x.v[k] + bv.v[k]) * inv[m], wv.v[k], acc.v[k]);
        }
        store_pack<V>(out + row + c, acc);
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

// Whether every pointer given lies on a 16-byte boundary (null counts) and rows of n floats keep it.
inline bool rows_of_16_bytes(int n, std::initializer_list<const void*> ptrs) {
    if (n % 4) return false;
    for (const void* q : ptrs)
        if (reinterpret_cast<uintptr_t>(q) & 15) return false;
    return true;
}

// The grid of a kernel whose threads own V columns and walk down the rows.
inline dim3 column_grid(int n_rows, int n, int v, int threads) {
    const int gx = (n / v + threads - 1) / threads;
    int gy = 148 * 8 / gx;
    gy = gy < 1 ? 1 : (gy > n_rows ? n_rows : gy);
    return dim3(gx, gy);
}

inline int blocks_for(size_t total, int threads) {
    const size_t b = (total + threads - 1) / threads;
    return (int)(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

}  // namespace

RI_API int ri_dyt_norm(const float* x, const float* w, const float* b, const float* alpha, const int* rows, void* out,
                       int out_dtype, int n_rows, int n, cudaStream_t stream) {
    if (n_rows <= 0 || n <= 0) return 0;
    const bool vec = rows_of_16_bytes(n, {x, w, b, out});
    const dim3 grid = column_grid(n_rows, n, vec ? 4 : 1, 128);
    cudaError_t e;
    if (out_dtype == RI_F32)
        e = vec ? launch_dependent(dyt_norm_kernel<float, 4>, grid, 128, 0, stream, x, w, b, alpha, rows, (float*)out, n_rows, n)
                : launch_dependent(dyt_norm_kernel<float, 1>, grid, 128, 0, stream, x, w, b, alpha, rows, (float*)out, n_rows, n);
    else if (out_dtype == RI_BF16)
        e = vec ? launch_dependent(dyt_norm_kernel<__nv_bfloat16, 4>, grid, 128, 0, stream, x, w, b, alpha, rows, (__nv_bfloat16*)out, n_rows, n)
                : launch_dependent(dyt_norm_kernel<__nv_bfloat16, 1>, grid, 128, 0, stream, x, w, b, alpha, rows, (__nv_bfloat16*)out, n_rows, n);
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
    const bool vec = rows_of_16_bytes(n, {stream_x, branch, branch_bias, post_w, post_b, history, next_w, next_b, next_out});
    const dim3 grid = column_grid(n_tokens, n, vec ? 4 : 1, 128);
    cudaError_t e;
    if (next_w == nullptr || next_dtype == RI_F32)
        e = vec ? launch_dependent(stream_update_kernel<float, 4>, grid, 128, 0, stream, p)
                : launch_dependent(stream_update_kernel<float, 1>, grid, 128, 0, stream, p);
    else if (next_dtype == RI_BF16)
        e = vec ? launch_dependent(stream_update_kernel<__nv_bfloat16, 4>, grid, 128, 0, stream, p)
                : launch_dependent(stream_update_kernel<__nv_bfloat16, 1>, grid, 128, 0, stream, p);
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
    bool vec = rows_of_16_bytes(n, {out});
    for (int m = 0; m < members; ++m) vec = vec && rows_of_16_bytes(n, {xs[m], biases[m], ws[m]});
    cudaError_t e = vec ? launch_dependent(normed_sum_kernel<4>, n_tokens, 256, 0, stream, p, out, n, eps, accumulate)
                        : launch_dependent(normed_sum_kernel<1>, n_tokens, 256, 0, stream, p, out, n, eps, accumulate);
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
