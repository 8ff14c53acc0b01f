// Routed experts (a mixture of small gated feed-forward layers), on the device from the router to
// the sum, so a step needs nothing from the host:
//
//   route     per token: s = sigmoid(W_router h) in float32 and c = s + correction, which ranks the
//             experts; expert e belongs to group e / (experts / groups); a group ranks by its top-2
//             sum of c, and only the `keep` highest groups remain candidates (the rest leave the
//             ranking, whatever the sign of their c); the `top` candidates with the highest c are
//             taken, with weights s / (sum of the taken s + 1e-20).
//             Optionally one more number per token: sigmoid(w_gate . h), the gate of a shared expert.
//             Another form (`form` bit 0): s = softmax(W_router h) over all experts instead of the sigmoid; and
//             (bit 1) the weights are the taken s as they are, not divided by their sum.
//   arrange   the (token, choice) pairs listed expert by expert, cut into tiles of rows that belong
//             to one expert
//   experts   the grouped contractions on the FFMA pipe with float32 accumulation, any sizes:
//             act[p] = silu(Wg[e] h) * (Wu[e] h) and y[p] = Wd[e] act[p] for pair p of expert e
//   combine   residual[t] += scale * (sum_c weight[t, c] * y[t * top + c] (+ gate[t] * shared[t])), in a fixed order;
//             a chosen id at or beyond the number of experts with tensors is an expert that hands its input
//             through: its y is the token's input row itself
//
// Every kernel here runs behind others of the same step and may come onto the SMs before they have
// finished (programmatic dependent launch): what an earlier kernel of the step wrote is read after
// `wait_for_previous_kernels()` through plain pointers, never `const __restrict__` ones, whose loads the
// compiler may move ahead of the wait.
//
// A pair is p = token * top + choice; its rows of act and y sit at p, so the order of the lists
// decides only which block works on which rows.  The tensor-core form of the contractions
// (`moe_tcgen05.cu`) wants an expert's rows consecutive instead: `gather` copies the activations
// into the order of the list, act and y stay in that order, and `combine` finds pair p's row through
// `place`.
#include "common.cuh"

using namespace ri;

namespace {

__device__ __forceinline__ float sigmoid_f32(float x) {
    if (x >= 0.f) return 1.f / (1.f + expf(-x));
    const float e = expf(x);
    return e / (1.f + e);
}

// (value, index) maximum over a warp; ties go to the lower index.
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}

constexpr int ROUTE_WARPS = 32;
constexpr int ROUTE_TOKENS = 8;           // most tokens a block routes: the router's rows are read once for all of them

template <typename T> __device__ __forceinline__ void load4_f32(const T* p, float* o);
template <> __device__ __forceinline__ void load4_f32<float>(const float* p, float* o) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
}
template <> __device__ __forceinline__ void load4_f32<__nv_bfloat16>(const __nv_bfloat16* p, float* o) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
}

// A block routes `per_block` tokens (1..ROUTE_TOKENS).  First its warps share out the router's rows (and
// the shared expert's gate row): a row is read once and multiplied with every token of the block, four
// values at a time with as many independent sums as tokens.  Then warp k makes token k's choice.
// Shared memory per token: score[E], choice[E], group score[G].
// A step of few tokens (one per block) may cut the router's rows over gridDim.y blocks per token, so that more SMs than
// tokens read them: every block leaves its rows' sums in `split_sums` ([tokens, experts + 1], float32) and takes a ticket
// from the token's counter in `split_count` (int32, zero before and after the kernel); the block that draws the last
// ticket reads all sums back and makes the token's choice.
template <typename T, bool VEC, int TOK>
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(const T* x, const float* __restrict__ router, const float* __restrict__ correction,
                 const float* __restrict__ gate_w, int* __restrict__ ids, float* __restrict__ weights,
                 float* __restrict__ gate_out, int n_tokens, int width, int experts, int top, int groups, int keep,
                 int per_block, int form, float* split_sums, int* split_count) {
    extern __shared__ float smem[];
    __shared__ int last_ticket;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int stride = 2 * experts + groups;
    let_next_kernel_start();
    wait_for_previous_kernels();
    const int tok0 = blockIdx.x * per_block;
    const int n_here = min(per_block, n_tokens - tok0);

    const int n_rows = experts + (gate_w != nullptr ? 1 : 0);
    const bool split = gridDim.y > 1;                 // only with one token per block
    const int rows_each = (n_rows + (int)gridDim.y - 1) / (int)gridDim.y;
    const int row_lo = split ? (int)blockIdx.y * rows_each : 0, row_hi = split ? min(n_rows, row_lo + rows_each) : n_rows;
    // what a row's sum becomes: the score (or, for the softmax, the logit) and the choice score; the gate's sigmoid
    auto place = [&](int k, int e, float a) {
        const float s = sigmoid_f32(a);
        if (e < experts) {
            smem[k * stride + e] = (form & 1) ? a : s;           // softmax: the logit, turned into a score below
            smem[k * stride + experts + e] = s + correction[e];
        } else {
            gate_out[tok0 + k] = s;
        }
    };
    for (int e = row_lo + warp; e < row_hi; e += ROUTE_WARPS) {
        const float* w = e < experts ? router + (size_t)e * width : gate_w;
        float acc[TOK];
#pragma unroll
        for (int k = 0; k < TOK; ++k) acc[k] = 0.f;
        if (VEC) {
#pragma unroll (TOK == 1 ? 8 : 4)
            for (int d = lane * 4; d < width; d += 128) {
                const float4 w4 = *reinterpret_cast<const float4*>(w + d);
#pragma unroll
                for (int k = 0; k < TOK; ++k)
                    if (TOK == 1 || k < n_here) {
                        float xv[4];
                        load4_f32<T>(x + (size_t)(tok0 + k) * width + d, xv);
                        acc[k] = fmaf(xv[0], w4.x, fmaf(xv[1], w4.y, fmaf(xv[2], w4.z, fmaf(xv[3], w4.w, acc[k]))));
                    }
            }
        } else {
            for (int d = lane; d < width; d += 32) {
                const float wv = w[d];
#pragma unroll
                for (int k = 0; k < TOK; ++k)
                    if (TOK == 1 || k < n_here) acc[k] = fmaf(to_f32<T>(x[(size_t)(tok0 + k) * width + d]), wv, acc[k]);
            }
        }
#pragma unroll
        for (int k = 0; k < TOK; ++k) {
            if (k >= n_here) break;
            const float a = warp_sum(acc[k]);
            if (lane == 0) {
                if (split) split_sums[(size_t)(tok0 + k) * (experts + 1) + e] = a;
                else place(k, e, a);
            }
        }
    }
    if (split) {
        __threadfence();                               // this block's sums are visible before its ticket is
        __syncthreads();
        if (threadIdx.x == 0) last_ticket = atomicAdd(&split_count[tok0], 1);
        __syncthreads();
        if (last_ticket != (int)gridDim.y - 1) return;
        __threadfence();
        for (int e = threadIdx.x; e < n_rows; e += blockDim.x) place(0, e, __ldcg(split_sums + (size_t)tok0 * (experts + 1) + e));
        if (threadIdx.x == 0) split_count[tok0] = 0;   // zero again for the next launch
    }
    __syncthreads();
    if (warp >= n_here) return;
    const int t = tok0 + warp;
    float* score = smem + (size_t)warp * stride;
    float* choice = score + experts;
    float* gscore = choice + experts;
    if (form & 1) {
        // softmax over all experts, in float32: the maximum, the exponentials' sum, the scores
        float mx = -INFINITY;
        for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, score[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < experts; e += 32) sum += expf(score[e] - mx);
        sum = warp_sum(sum);
        for (int e = lane; e < experts; e += 32) {
            const float s = expf(score[e] - mx) / sum;
            score[e] = s;
            choice[e] = s + correction[e];
        }
        __syncwarp();
    }

    // groups: top-2 sum of c per group; all but the `keep` highest leave the ranking
    const int size = experts / groups;
    if (keep < groups) {
        for (int g = lane; g < groups; g += 32) {
            float a = -INFINITY, b = -INFINITY;
            for (int k = 0; k < size; ++k) {
                const float c = choice[g * size + k];
                if (c > a) { b = a; a = c; } else if (c > b) { b = c; }
            }
            gscore[g] = size > 1 ? a + b : a;
        }
        __syncwarp();
        // `keep` rounds of taking the best remaining group; a taken group is marked with +inf
        for (int round = 0; round < keep; ++round) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            for (int g = lane; g < groups; g += 32) {
                const float v = gscore[g];
                if (v != INFINITY && (v > bv || (v == bv && g < bi))) { bv = v; bi = g; }
            }
            warp_argmax(bv, bi);
            if (lane == 0 && bi < groups) gscore[bi] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < experts; e += 32)
            if (gscore[e / size] != INFINITY) choice[e] = -INFINITY;
        __syncwarp();
    }

    // `top` rounds of taking the best remaining expert
    float sum = 0.f;
    for (int c = 0; c < top; ++c) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float v = choice[e];              // NaN: taken already; -inf: shut out with its group
            if (v > bv || (v == bv && v != -INFINITY && e < bi)) { bv = v; bi = e; }
        }
        warp_argmax(bv, bi);
        if (bi >= experts) bi = 0;
        const float s = score[bi];
        sum += s;
        if (lane == 0) {
            ids[(size_t)t * top + c] = bi;
            weights[(size_t)t * top + c] = s;
            choice[bi] = NAN;                    // taken
        }
        __syncwarp();
    }
    if (form & 2) return;                        // the weights are the scores as they are
    const float inv = 1.0f / (sum + 1e-20f);
    for (int c = lane; c < top; c += 32) weights[(size_t)t * top + c] *= inv;
}

// ---- arrange ---------------------------------------------------------------------------------
// One block.  offsets[e]..offsets[e+1] index `order`, which lists the pairs of expert e; tiles[2k],
// tiles[2k+1] = (expert, first index into `order`) of tile k, each tile holding at most `tile_rows`
// pairs of one expert; n_tiles[0] their number; place[p] (optional) the index of pair p in `order`.
__global__ void __launch_bounds__(1024)
moe_arrange_kernel(const int* ids, int n_pairs, int experts, int tile_rows, int* __restrict__ offsets,
                   int* order, int* __restrict__ tiles, int* __restrict__ n_tiles, int* __restrict__ place,
                   const uint4* x, uint4* __restrict__ xs, int top, int vecs) {
    extern __shared__ int sh[];
    int* count = sh;                 // [experts]
    int* start = sh + experts;       // [experts + 1]
    int* fill = start + experts + 1; // [experts]
    let_next_kernel_start();
    wait_for_previous_kernels();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) { count[e] = 0; fill[e] = 0; }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0, nt = 0;
        for (int e = 0; e < experts; ++e) {
            start[e] = acc;
            for (int r0 = 0; r0 < count[e]; r0 += tile_rows) {
                tiles[2 * nt] = e;
                tiles[2 * nt + 1] = acc + r0;
                ++nt;
            }
            acc += count[e];
        }
        start[experts] = acc;
        n_tiles[0] = nt;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= experts; e += blockDim.x) offsets[e] = start[e];
    // a pair's place among its expert's pairs is whatever the atomics hand out: every pair owns its rows
    // of the results, so the order changes no number
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < experts) {
            const int at = start[e] + atomicAdd(&fill[e], 1);
            order[at] = p;
            if (place != nullptr) place[p] = at;
        }
    }
    if (xs != nullptr) {
        // a step of few pairs: the activations go into the lists' order here, without a kernel of their own
        __syncthreads();
        const int listed = start[experts];       // pairs whose id names no expert of the lists are in none of them
        for (int i = threadIdx.x; i < listed * vecs; i += blockDim.x) {
            const int r = i / vecs, c = i % vecs;
            xs[i] = x[(size_t)(order[r] / top) * vecs + c];
        }
    }
}

// xs[i, :] = x[order[i] / top, :]: the activations in the order of the list, 16 bytes at a time
// (width a multiple of 8 bf16).
__global__ void moe_gather_kernel(const uint4* x, uint4* __restrict__ xs, const int* order,
                                  int n_pairs, int top, int vecs, const int* listed) {
    let_next_kernel_start();
    wait_for_previous_kernels();
    // listed: the number of pairs in the lists (the last of the arrange kernel's offsets), where some pairs are in none
    const size_t total = (size_t)(listed != nullptr ? min(n_pairs, *listed) : n_pairs) * vecs;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int r = (int)(i / vecs), c = (int)(i % vecs);
        xs[i] = x[(size_t)(order[r] / top) * vecs + c];
    }
}

// ---- the grouped contractions ------------------------------------------------------------------
constexpr int GM = 32, GN = 64, GK = 16, G_THREADS = 256;      // a tile of 32 pairs x 64 features; thread: 2 x 4

// gate_form (GATE only): the five constants of another gate than SiLU (`GateForm`), or null.
// GATE: act[p, n] = silu(sum_k Wg[e][n, k] x[p / top, k]) * (sum_k Wu[e][n, k] x[p / top, k])   (T out)
// else: y[p, n]   = sum_k Wd[e][n, k] act[p, k]                                                  (float out)
template <typename T, bool GATE>
__global__ void __launch_bounds__(G_THREADS)
moe_grouped_kernel(const T* X, const T* __restrict__ W, const T* __restrict__ W2, void* __restrict__ out_,
                   const int* offsets, const int* order, const int* tiles, const int* n_tiles, int top, int N, int K,
                   const float* __restrict__ gate_form) {
    const GateForm gf = load_gate_form(GATE ? gate_form : nullptr);
    __shared__ float Xs[GK][GM + 1];
    __shared__ float Ws[GK][GN + 1];
    __shared__ float W2s[GATE ? GK : 1][GATE ? GN + 1 : 1];
    __shared__ int rows[GM];
    let_next_kernel_start();
    wait_for_previous_kernels();
    if ((int)blockIdx.x >= *reinterpret_cast<const volatile int*>(n_tiles)) return;
    const int e = tiles[2 * blockIdx.x], first = tiles[2 * blockIdx.x + 1];
    const int n_rows = min(GM, offsets[e + 1] - first);
    const int n0 = blockIdx.y * GN;
    const int tid = threadIdx.x;
    if (tid < GM) rows[tid] = tid < n_rows ? order[first + tid] : -1;
    __syncthreads();
    const T* We = W + (size_t)e * N * K;
    const T* W2e = GATE ? W2 + (size_t)e * N * K : nullptr;
    const int tm = (tid / 16) * 2, tn = (tid % 16) * 4;
    float acc[2][4] = {}, acc2[2][4] = {};
    for (int k0 = 0; k0 < K; k0 += GK) {
        // X tile: GM x GK
        for (int i = tid; i < GM * GK; i += G_THREADS) {
            const int m = i / GK, k = i % GK;
            const int p = rows[m];
            float v = 0.f;
            if (p >= 0 && k0 + k < K) v = to_f32<T>(X[(size_t)(GATE ? p / top : p) * K + k0 + k]);
            Xs[k][m] = v;
        }
        for (int i = tid; i < GN * GK; i += G_THREADS) {
            const int n = i / GK, k = i % GK;
            const bool in = n0 + n < N && k0 + k < K;
            Ws[k][n] = in ? to_f32<T>(We[(size_t)(n0 + n) * K + k0 + k]) : 0.f;
            if (GATE) W2s[k][n] = in ? to_f32<T>(W2e[(size_t)(n0 + n) * K + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GK; ++k) {
            float xv[2], wv[4], w2v[4];
#pragma unroll
            for (int a = 0; a < 2; ++a) xv[a] = Xs[k][tm + a];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                wv[b] = Ws[k][tn + b];
                if (GATE) w2v[b] = W2s[k][tn + b];
            }
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    acc[a][b] = fmaf(xv[a], wv[b], acc[a][b]);
                    if (GATE) acc2[a][b] = fmaf(xv[a], w2v[b], acc2[a][b]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int a = 0; a < 2; ++a) {
        const int p = rows[tm + a];
        if (p < 0) continue;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int n = n0 + tn + b;
            if (n >= N) continue;
            if (GATE)
                reinterpret_cast<T*>(out_)[(size_t)p * N + n] = from_f32<T>(gated_f32(acc[a][b], acc2[a][b], gf));
            else
                reinterpret_cast<float*>(out_)[(size_t)p * N + n] = acc[a][b];
        }
    }
}

// ids / x / n_real (optional): a chosen id >= n_real hands the token's input row x[t] through instead of a row of y.
template <typename T>
__global__ void moe_combine_kernel(float* residual, const float* y, const float* weights, const float* shared_y,
                                   const float* gate, const int* place, int n_tokens, int width, int top,
                                   const int* ids, const T* x, int n_real, float scale) {
    let_next_kernel_start();
    wait_for_previous_kernels();
    const size_t total = (size_t)n_tokens * width;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / width), d = (int)(i % width);
        float acc = 0.f;
        for (int c = 0; c < top; ++c) {
            const size_t p = (size_t)t * top + c;
            if (ids != nullptr && ids[p] >= n_real) {
                acc = fmaf(weights[p], to_f32<T>(x[i]), acc);
                continue;
            }
            acc = fmaf(weights[p], y[(place != nullptr ? (size_t)place[p] : p) * width + d], acc);
        }
        if (shared_y != nullptr) acc = gate != nullptr ? fmaf(gate[t], shared_y[i], acc) : acc + shared_y[i];
        residual[i] += scale == 1.f ? acc : scale * acc;
    }
}

}  // namespace

// form: bit 0 softmax scores instead of sigmoid ones, bit 1 weights not divided by their sum.
// split > 1 (steps of up to ROUTE_SPLIT_TOKENS tokens): the router's rows are cut over that many blocks per token;
// split_sums: float32 [n_tokens, experts + 1] scratch, split_count: int32 [n_tokens], zero before the call and after it.
RI_API int ri_moe_route(const void* x, int dtype, const float* router, const float* correction, const float* gate_w,
                        int* ids, float* weights, float* gate_out, int n_tokens, int width, int experts, int top,
                        int groups, int keep, int form, int split, float* split_sums, int* split_count,
                        cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (experts <= 0 || top <= 0 || top > experts) return fail("moe_route: top %d of %d experts", top, experts);
    if (groups <= 0 || experts % groups || keep <= 0 || keep > groups)
        return fail("moe_route: %d experts in %d groups, %d kept", experts, groups, keep);
    if ((long long)keep * (experts / groups) < top)
        return fail("moe_route: %d groups of %d experts cannot give %d choices", keep, experts / groups, top);
    // few tokens: one per block, so that the router's rows are shared out over more SMs
    const int per_block = n_tokens >= 148 * ROUTE_TOKENS ? ROUTE_TOKENS : (n_tokens >= 2 * 148 ? 2 : 1);
    if (split > 1 && (per_block != 1 || split_sums == nullptr || split_count == nullptr || split > 65535))
        return fail("moe_route: rows cut over %d blocks need one token per block and their scratch", split);
    const size_t smem = (size_t)per_block * (2 * experts + groups) * sizeof(float);
    if (smem > 48 * 1024) return fail("moe_route: %d experts exceed the router kernel's shared memory", experts);
    const dim3 blocks((n_tokens + per_block - 1) / per_block, split > 1 ? split : 1);
    const bool vec = width % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)router % 16 == 0 &&
                     (gate_w == nullptr || (uintptr_t)gate_w % 16 == 0);
    cudaError_t e;
#define RI_ROUTE_N(T, V, N) launch_dependent(moe_route_kernel<T, V, N>, blocks, ROUTE_WARPS * 32, smem, stream, (const T*)x, \
                                             router, correction, gate_w, ids, weights, gate_out, n_tokens, width, experts, top,   \
                                             groups, keep, per_block, form, split_sums, split_count)
#define RI_ROUTE(T, V) (per_block == 1 ? RI_ROUTE_N(T, V, 1) : per_block == 2 ? RI_ROUTE_N(T, V, 2) : RI_ROUTE_N(T, V, ROUTE_TOKENS))
    if (dtype == RI_F32) e = vec ? RI_ROUTE(float, true) : RI_ROUTE(float, false);
    else if (dtype == RI_BF16) e = vec ? RI_ROUTE(__nv_bfloat16, true) : RI_ROUTE(__nv_bfloat16, false);
    else return fail("moe_route: unknown dtype %d", dtype);
#undef RI_ROUTE_N
#undef RI_ROUTE
    return check_launch(e, "moe_route");
}

RI_API int ri_moe_tile_rows() { return GM; }

// x, xs (optional, bf16 rows of `width` values, a multiple of 8): also xs[i] = x[order[i] / top], for steps of few pairs.
RI_API int ri_moe_arrange(const int* ids, int n_pairs, int experts, int tile_rows, int* offsets, int* order, int* tiles,
                          int* n_tiles, int* place, const void* x, void* xs, int top, int width, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (tile_rows <= 0) return fail("moe_arrange: tile of %d rows", tile_rows);
    const size_t smem = (size_t)(3 * experts + 1) * sizeof(int);
    if (smem > 48 * 1024) return fail("moe_arrange: %d experts exceed the kernel's shared memory", experts);
    if (xs != nullptr && (x == nullptr || top <= 0 || width % 8 || (uintptr_t)x % 16 || (uintptr_t)xs % 16))
        return fail("moe_arrange: rows of %d bf16 cannot be gathered 16 bytes at a time", width);
    cudaError_t e = launch_dependent(moe_arrange_kernel, 1, 1024, smem, stream, ids, n_pairs, experts, tile_rows, offsets,
                                     order, tiles, n_tiles, place, (const uint4*)x, (uint4*)xs, top, width / 8);
    return check_launch(e, "moe_arrange");
}

RI_API int ri_moe_gather(const void* x, void* xs, const int* order, int n_pairs, int top, int width, const int* listed,
                         cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (width % 8 || (uintptr_t)x % 16 || (uintptr_t)xs % 16) return fail("moe_gather: rows of %d bf16 are not 16-byte runs", width);
    const size_t total = (size_t)n_pairs * (width / 8);
    const int blocks = (int)((total + 255) / 256 < 8192 ? (total + 255) / 256 : 8192);
    cudaError_t e = launch_dependent(moe_gather_kernel, blocks, 256, 0, stream, (const uint4*)x, (uint4*)xs, order, n_pairs,
                                     top, width / 8, listed);
    return check_launch(e, "moe_gather");
}

// gate != 0: x [tokens, K], w / w2 [experts, N, K] -> out<dtype> [pairs, N]; else x [pairs, K], w -> out<float> [pairs, N]
RI_API int ri_moe_grouped_simt(const void* x, const void* w, const void* w2, void* out, int dtype, int gate,
                               const int* offsets, const int* order, const int* tiles, const int* n_tiles, int n_pairs,
                               int experts, int top, int N, int K, const float* gate_form, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    const int max_tiles = (n_pairs + GM - 1) / GM + experts;
    dim3 grid(max_tiles, (N + GN - 1) / GN);
    if (grid.y > 65535) return fail("moe_grouped: %d features exceed the grid limit", N);
    cudaError_t e;
#define RI_GROUPED(T, G) launch_dependent(moe_grouped_kernel<T, G>, grid, G_THREADS, 0, stream, (const T*)x, (const T*)w, \
                                          (const T*)w2, out, offsets, order, tiles, n_tiles, top, N, K, gate_form)
    if (dtype == RI_F32) e = gate ? RI_GROUPED(float, true) : RI_GROUPED(float, false);
    else if (dtype == RI_BF16) e = gate ? RI_GROUPED(__nv_bfloat16, true) : RI_GROUPED(__nv_bfloat16, false);
    else return fail("moe_grouped: unknown dtype %d", dtype);
#undef RI_GROUPED
    return check_launch(e, "moe_grouped");
}

// ids, x (dtype x_dtype), n_real: all null / 0, or the chosen ids [tokens, top], the experts' input [tokens, width] and
// the number of experts with tensors (a chosen id at or beyond it hands x through).  gate may be null with shared_y
// (the shared result is added as it is).  scale: a factor on everything that is added.
RI_API int ri_moe_combine(float* residual, const float* y, const float* weights, const float* shared_y, const float* gate,
                          const int* place, int n_tokens, int width, int top, const int* ids, const void* x, int x_dtype,
                          int n_real, float scale, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if ((ids == nullptr) != (x == nullptr)) return fail("moe_combine: ids and the experts' input go together");
    const size_t total = (size_t)n_tokens * width;
    const int blocks = (int)((total + 255) / 256 < 8192 ? (total + 255) / 256 : 8192);
    cudaError_t e;
    if (x == nullptr || x_dtype == RI_F32)
        e = launch_dependent(moe_combine_kernel<float>, blocks, 256, 0, stream, residual, y, weights, shared_y, gate, place,
                             n_tokens, width, top, ids, (const float*)x, n_real, scale);
    else if (x_dtype == RI_BF16)
        e = launch_dependent(moe_combine_kernel<__nv_bfloat16>, blocks, 256, 0, stream, residual, y, weights, shared_y, gate,
                             place, n_tokens, width, top, ids, (const __nv_bfloat16*)x, n_real, scale);
    else
        return fail("moe_combine: unknown dtype %d", x_dtype);
    return check_launch(e, "moe_combine");
}

RI_DEFINE_LAST_ERROR()
