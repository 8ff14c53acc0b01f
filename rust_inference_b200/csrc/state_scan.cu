// Recurrent mixers with a matrix state per head and ONE decay per head and token: the selective state space
// (scalar decay, the form its authors call state-space duality) and the gated delta rule.  Per head, with the state
// S [dim, vdim] in float32, the decay a_t, a key k_t [dim], a query q_t [dim], a value v_t [vdim] and a step s_t:
//
//     state space    S <- a S + k (s v)^T                      o = S^T q + skip * v
//     delta rule     S <- a S;  u = s (v - S^T k);  S <- S + k u^T      o = S^T q
//
// (state space: k = B, q = C, v = x, s = dt, a = exp(-exp(A_log) dt);  delta rule: s = beta, a = exp(-exp(A_log)
// softplus(.)); the read-out sees the token's own write.)  Heads share keys and queries in groups.  The state lives in
// a per-slot area of the cache, starts at zero when a slot is handed out and is carried from step to step; so do the
// last taps - 1 inputs of the short causal convolutions that come before the recurrence.  A prompt may therefore be
// cut anywhere, and a decode step is the same kernels with one token per sequence.
//
// Four kernels, all reading the step's arrays on the device (graph-safe), everything float32:
//   prepare     per token: the short convolution (+ bias) and silu over a range of the projection's columns; unit
//               vectors x / sqrt(sum x^2 + 1e-6) for the first heads of that range (the first of them times a factor);
//               the decay and the step of every head
//   conv_state  per (sequence, channel): the convolution's carried inputs move on by the step's tokens
//   scan        per (sequence, head, tile of value columns): the recurrence over the sequence's new tokens in
//               order; the state is read first and written last
//   finish      per (token, group of channels): RMS norm over the group and a silu gate, before or after the norm
//
// What an earlier kernel of the step wrote is read after `wait_for_previous_kernels()` through plain pointers.
#include "common.cuh"

using namespace ri;

namespace {

__device__ __forceinline__ float softplus_f32(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f32(float x) {
    if (x >= 0.f) return 1.f / (1.f + expf(-x));
    const float e = expf(x);
    return e / (1.f + e);
}

struct Prepare {
    const float* z;            // [tokens, ld] the projection's results
    int ld;
    int conv_col, conv_ch;     // the convolved columns of z
    const float* taps;         // [conv_ch, k_taps], the last column is the current token's
    const float* conv_bias;    // null: none
    int k_taps;
    float* conv_state;         // [slots, k_taps - 1, conv_ch]: the inputs before the step, oldest first
    int unit_heads, unit_dim;  // the first unit_heads * unit_dim convolved channels are made unit vectors per head
    int scaled_heads;          // the first of those heads are also multiplied by unit_scale
    float unit_scale;
    int heads;                 // heads with a decay
    int decay_col;             // column of z with the decay's raw step, per head
    int step_col;              // >= 0: column of z whose sigmoid is the step (delta rule); < 0: the step is softplus(raw + bias)
    const float* a_log;        // [heads]
    const float* dt_bias;      // [heads]
    float* out;                // [tokens, out_ld] = [convolved channels | decay per head | step per head]
    int out_ld;
    const int* cu_seqlens;
    const int* token_seq;
    const int* seq_slot;
    int tile_ch;               // convolved channels per block: a multiple of unit_dim where there are unit vectors
};

// A block per (token, tile of p.tile_ch convolved channels); tiles hold whole heads of the unit vectors.  The first
// tile's block also writes the heads' decays and steps.
__global__ void __launch_bounds__(256) scan_prepare_kernel(Prepare p) {
    extern __shared__ float ch[];                 // [tile_ch]
    const int t = blockIdx.x;
    const int c0 = blockIdx.y * p.tile_ch, c1 = min(p.conv_ch, c0 + p.tile_ch);
    let_next_kernel_start();
    wait_for_previous_kernels();
    const int b = p.token_seq[t];
    const int i = t - p.cu_seqlens[b];            // place among the sequence's new tokens
    int slot = p.seq_slot[b];
    if (!RI_BLOCK_IN_LIMIT(slot, RI_LIMIT_SLOTS, RI_CHECK_SLOT)) slot = 0;
    const int K = p.k_taps;
    const float* carried = p.conv_state + (size_t)slot * (K - 1) * p.conv_ch;
    for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
        float acc = p.conv_bias != nullptr ? p.conv_bias[c] : 0.f;
        for (int k = 0; k < K; ++k) {             // the input k tokens back
            const int src = i - k;
            const float x = src >= 0 ? p.z[(size_t)(t - k) * p.ld + p.conv_col + c]
                                     : carried[(size_t)(K - 1 + src) * p.conv_ch + c];
            acc = fmaf(p.taps[(size_t)c * K + (K - 1 - k)], x, acc);
        }
        ch[c - c0] = silu_f32(acc);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    if (p.unit_heads > 0 && c0 < p.unit_heads * p.unit_dim) {
        const int h0 = c0 / p.unit_dim, h1 = min(p.unit_heads, c1 / p.unit_dim);     // tiles are multiples of unit_dim there
        for (int h = h0 + warp; h < h1; h += warps) {
            float* v = ch + (h - h0) * p.unit_dim;
            float ss = 0.f;
            for (int d = lane; d < p.unit_dim; d += 32) ss = fmaf(v[d], v[d], ss);
            ss = warp_sum(ss);
            const float f = (h < p.scaled_heads ? p.unit_scale : 1.f) / sqrtf(ss + 1e-6f);
            for (int d = lane; d < p.unit_dim; d += 32) v[d] *= f;
        }
        __syncthreads();
    }
    float* out = p.out + (size_t)t * p.out_ld;
    for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) out[c] = ch[c - c0];
    if (blockIdx.y == 0)
        for (int h = threadIdx.x; h < p.heads; h += blockDim.x) {
            const float dt = softplus_f32(p.z[(size_t)t * p.ld + p.decay_col + h] + p.dt_bias[h]);
            out[p.conv_ch + h] = expf(-expf(p.a_log[h]) * dt);
            out[p.conv_ch + p.heads + h] = p.step_col >= 0 ? sigmoid_f32(p.z[(size_t)t * p.ld + p.step_col + h]) : dt;
        }
}

__global__ void conv_state_kernel(const float* z, int ld, int conv_col, int conv_ch, int k_taps, float* conv_state,
                                  const int* cu_seqlens, const int* seq_slot) {
    let_next_kernel_start();
    wait_for_previous_kernels();
    const int b = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= conv_ch) return;
    const int t0 = cu_seqlens[b], n = cu_seqlens[b + 1] - t0;
    const int slot = seq_slot[b];
    if (n <= 0 || !RI_IN_LIMIT(slot, RI_LIMIT_SLOTS, RI_CHECK_SLOT)) return;
    float* carried = conv_state + (size_t)slot * (k_taps - 1) * conv_ch;
    for (int s = 0; s < k_taps - 1; ++s) {        // ascending: an entry is read before a later round overwrites it
        const int src = n - (k_taps - 1) + s;
        carried[(size_t)s * conv_ch + c] = src >= 0 ? z[(size_t)(t0 + src) * ld + conv_col + c]
                                                    : carried[(size_t)(s + n) * conv_ch + c];
    }
}

// Threads of a warp: lane = column_in_warp * R + r.  Thread (r, j) keeps ROWS consecutive rows (r * ROWS ...) of
// column j of the state in registers; sums over the rows are finished by log2(R) shuffles inside the warp.  The
// tokens' keys, queries, values, decays and steps come through shared memory in tiles, a key's and a query's row
// slices padded so that the eight slices' 16-byte reads fall into different banks.  There are two tiles: while the
// recurrence runs over one, asynchronous copies (16 bytes each where every column offset and the row length are
// multiples of four floats, 4 bytes each otherwise) fill the other, so the global loads' latency stays off the
// sequential path.
constexpr int R = 8;
constexpr int SCAN_WARPS = 4;
constexpr int COLS = SCAN_WARPS * 32 / R;        // value columns per block
constexpr int SCAN_THREADS = SCAN_WARPS * 32;

__device__ __forceinline__ void copy_async4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct Scan {
    const float* u;            // [tokens, ld]: the prepared rows
    int ld;
    int q_col, k_col, v_col, decay_col, step_col;
    const float* skip;         // [heads] or null: o += skip * v
    float* state;              // [slots, heads, dim, vdim]
    float* o;                  // [tokens, heads * vdim]
    const int* cu_seqlens;
    const int* seq_slot;
    int heads, groups, dim, vdim, tile_t;
    int vec;                   // 1: rows, columns and sizes allow 16-byte copies
    int piece, max_pieces;     // passes over pieces: tokens per piece, most pieces of a sequence
    float* piece_state;        // [seqs, max_pieces, heads, dim, vdim]: a piece's end state from zero, then its start state
    float* piece_decay;        // [seqs, max_pieces, heads]: the product of a piece's decays
};

// How a launch of the scan treats its tokens.  WHOLE: a block runs over all new tokens of its sequence from the slot's
// state and writes the state back.  For long runs of the state space, whose update is linear in the state with a scalar
// factor, three launches work on pieces of a sequence side by side: LOCAL scans every piece from zero (no read-out) and
// keeps its end state and the product of its decays; a carry kernel walks the pieces of a sequence per state element,
// start(p + 1) = decays(p) * start(p) + end(p), leaving every piece's start state and the sequence's final state in the
// slot; FINAL scans every piece again from its start state and writes the read-outs.
enum { WHOLE = 0, LOCAL = 1, FINAL = 2 };

template <int ROWS, bool DELTA, int MODE>
__global__ void __launch_bounds__(SCAN_THREADS) state_scan_kernel(Scan p) {
    constexpr int SLICE = ROWS + 4;
    constexpr int TOKEN = 2 * R * SLICE + COLS + 4;       // k, q, the block's values, decay and step
    extern __shared__ __align__(16) float tile[];          // two tiles of tile_t tokens
    const int b = MODE == WHOLE ? blockIdx.x : blockIdx.x / p.max_pieces, h = blockIdx.y, j0 = blockIdx.z * COLS;
    const int pc = MODE == WHOLE ? 0 : blockIdx.x % p.max_pieces;
    const int r = threadIdx.x % R, jj = threadIdx.x / R;
    const int j = j0 + jj, i0 = r * ROWS;
    const bool live = j < p.vdim;
    for (int i = threadIdx.x; i < 2 * p.tile_t * TOKEN; i += SCAN_THREADS) tile[i] = 0.f;
    const float skip = p.skip != nullptr ? p.skip[h] : 0.f;
    let_next_kernel_start();
    wait_for_previous_kernels();
    const int t0 = p.cu_seqlens[b] + (MODE == WHOLE ? 0 : pc * p.piece);
    const int t1 = MODE == WHOLE ? p.cu_seqlens[b + 1] : min(p.cu_seqlens[b + 1], t0 + p.piece);
    const int slot = p.seq_slot[b];
    if (t0 >= t1 || !RI_BLOCK_IN_LIMIT(slot, RI_LIMIT_SLOTS, RI_CHECK_SLOT)) return;
    float* S = MODE == WHOLE ? p.state + (((size_t)slot * p.heads + h) * p.dim) * p.vdim
                             : p.piece_state + ((((size_t)b * p.max_pieces + pc) * p.heads + h) * p.dim) * p.vdim;
    float s[ROWS];
#pragma unroll
    for (int k = 0; k < ROWS; ++k) s[k] = (MODE != LOCAL && live && i0 + k < p.dim) ? S[(size_t)(i0 + k) * p.vdim + j] : 0.f;
    float decays = 1.f;
    const int g = h / (p.heads / p.groups);
    const int q_off = p.q_col + g * p.dim, k_off = p.k_col + g * p.dim, v_off = p.v_col + h * p.vdim + j0;
    const int cols = min(COLS, p.vdim - j0);
    const int o_ld = p.heads * p.vdim;
    __syncthreads();                                      // the zeros are in place

    // the copies of the tokens tb .. tb + n_tok - 1 into one of the two tiles; every thread commits one group
    auto fetch = [&](float* dst, int tb, int n_tok) {
        if (p.vec) {
            const int dq = p.dim >> 2, cq = cols >> 2, per = 2 * dq + cq;
            for (int tok = 0; tok < n_tok; ++tok) {
                const float* row = p.u + (size_t)(tb + tok) * p.ld;
                float* base = dst + tok * TOKEN;
                for (int it = threadIdx.x; it < per; it += SCAN_THREADS) {
                    if (it < dq) copy_async16(base + (4 * it / ROWS) * SLICE + 4 * it % ROWS, row + k_off + 4 * it);
                    else if (it < 2 * dq) copy_async16(base + R * SLICE + (4 * (it - dq) / ROWS) * SLICE + 4 * (it - dq) % ROWS, row + q_off + 4 * (it - dq));
                    else copy_async16(base + 2 * R * SLICE + 4 * (it - 2 * dq), row + v_off + 4 * (it - 2 * dq));
                }
            }
        } else {
            const int per = 2 * p.dim + cols;
            for (int tok = 0; tok < n_tok; ++tok) {
                const float* row = p.u + (size_t)(tb + tok) * p.ld;
                float* base = dst + tok * TOKEN;
                for (int it = threadIdx.x; it < per; it += SCAN_THREADS) {
                    if (it < p.dim) copy_async4(base + (it / ROWS) * SLICE + it % ROWS, row + k_off + it);
                    else if (it < 2 * p.dim) copy_async4(base + R * SLICE + ((it - p.dim) / ROWS) * SLICE + (it - p.dim) % ROWS, row + q_off + it - p.dim);
                    else copy_async4(base + 2 * R * SLICE + it - 2 * p.dim, row + v_off + it - 2 * p.dim);
                }
            }
        }
        for (int tok = threadIdx.x; tok < 2 * n_tok; tok += SCAN_THREADS) {      // decay and step of every token
            const int tk = tok >> 1, which = tok & 1;
            copy_async4(dst + tk * TOKEN + 2 * R * SLICE + COLS + which,
                        p.u + (size_t)(tb + tk) * p.ld + (which ? p.step_col : p.decay_col) + h);
        }
        copy_async_commit();
    };

    const int tile_floats = p.tile_t * TOKEN;
    fetch(tile, t0, min(p.tile_t, t1 - t0));
    int buf = 0;
    for (int tb = t0; tb < t1; tb += p.tile_t, buf ^= 1) {
        const int n_tok = min(p.tile_t, t1 - tb);
        const int nb = tb + p.tile_t;
        if (nb < t1) {                                    // the next tile is on its way while this one is used
            fetch(tile + (buf ^ 1) * tile_floats, nb, min(p.tile_t, t1 - nb));
            copy_async_wait<1>();
        } else {
            copy_async_wait<0>();
        }
        __syncthreads();
        const float* cur = tile + buf * tile_floats;
        // unrolled: only the state's update chains the tokens, so the loads and the read-out's sums of one token overlap
        // the next token's update
#pragma unroll(DELTA ? 2 : 4)
        for (int tok = 0; tok < n_tok; ++tok) {
            const float* base = cur + tok * TOKEN;
            const float4* k4 = reinterpret_cast<const float4*>(base + r * SLICE);
            const float4* q4 = reinterpret_cast<const float4*>(base + R * SLICE + r * SLICE);
            const float v = base[2 * R * SLICE + jj];
            const float a = base[2 * R * SLICE + COLS], step = base[2 * R * SLICE + COLS + 1];
            float kk[ROWS], qq[ROWS];
#pragma unroll
            for (int k = 0; k < ROWS / 4; ++k) {
                const float4 kv = k4[k], qv = q4[k];
                kk[4 * k] = kv.x; kk[4 * k + 1] = kv.y; kk[4 * k + 2] = kv.z; kk[4 * k + 3] = kv.w;
                qq[4 * k] = qv.x; qq[4 * k + 1] = qv.y; qq[4 * k + 2] = qv.z; qq[4 * k + 3] = qv.w;
            }
            float write = step * v;
            if (MODE == LOCAL) decays *= a;
            if (DELTA) {
                float d0 = 0.f, d1 = 0.f;
#pragma unroll
                for (int k = 0; k < ROWS; k += 2) {
                    s[k] *= a;
                    s[k + 1] *= a;
                    d0 = fmaf(s[k], kk[k], d0);
                    d1 = fmaf(s[k + 1], kk[k + 1], d1);
                }
                float dot = d0 + d1;
#pragma unroll
                for (int o = R / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                write = step * (v - dot);
            }
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int k = 0; k < ROWS; k += 2) {
                s[k] = DELTA ? fmaf(kk[k], write, s[k]) : fmaf(a, s[k], kk[k] * write);
                s[k + 1] = DELTA ? fmaf(kk[k + 1], write, s[k + 1]) : fmaf(a, s[k + 1], kk[k + 1] * write);
                a0 = fmaf(s[k], qq[k], a0);
                a1 = fmaf(s[k + 1], qq[k + 1], a1);
            }
            float acc = a0 + a1;
#pragma unroll
            for (int o = R / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (MODE != LOCAL && live && r == 0) p.o[(size_t)(tb + tok) * o_ld + h * p.vdim + j] = fmaf(skip, v, acc);
        }
        __syncthreads();                                  // this tile may be overwritten by the fetch after next
    }
    if (MODE == FINAL) return;                            // the carry kernel left the final state in the slot
#pragma unroll
    for (int k = 0; k < ROWS; ++k)
        if (live && i0 + k < p.dim) S[(size_t)(i0 + k) * p.vdim + j] = s[k];
    if (MODE == LOCAL && blockIdx.z == 0 && threadIdx.x == 0) p.piece_decay[((size_t)b * p.max_pieces + pc) * p.heads + h] = decays;
}

// Per (sequence, head, state element): the pieces' start states from their end states and decay products; the
// sequence's final state goes to the slot.
__global__ void __launch_bounds__(256) scan_carry_kernel(float* state, float* piece_state, const float* piece_decay,
                                                         const int* cu_seqlens, const int* seq_slot, int heads, int per_head,
                                                         int piece, int max_pieces) {
    let_next_kernel_start();
    wait_for_previous_kernels();
    const int b = blockIdx.z, h = blockIdx.y;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    const int n = cu_seqlens[b + 1] - cu_seqlens[b];
    const int slot = seq_slot[b];
    if (e >= per_head || n <= 0 || !RI_IN_LIMIT(slot, RI_LIMIT_SLOTS, RI_CHECK_SLOT)) return;
    const int pieces = (n + piece - 1) / piece;
    float* dst = state + ((size_t)slot * heads + h) * per_head + e;
    float s = *dst;
    for (int pc = 0; pc < pieces; ++pc) {
        float* ps = piece_state + (((size_t)b * max_pieces + pc) * heads + h) * per_head + e;
        const float local = *ps;
        *ps = s;
        s = fmaf(piece_decay[((size_t)b * max_pieces + pc) * heads + h], s, local);
    }
    *dst = s;
}

// One warp per (token, group of `gs` channels): with gate_first the channels are multiplied by silu(gate) and then
// normalised, otherwise normalised and then multiplied; the weight of channel c of a token's row is w[c % w_len].
template <typename T>
__global__ void gated_group_norm_kernel(const float* x, int x_ld, const float* gate, int gate_ld, int gate_col,
                                        const float* __restrict__ w, int w_len, T* __restrict__ out, int n_tokens, int groups,
                                        int gs, int gate_first, float eps, float out_scale) {
    let_next_kernel_start();
    wait_for_previous_kernels();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n_tokens * groups) return;
    const int t = warp / groups, g = warp % groups;
    const float* src = x + (size_t)t * x_ld + g * gs;
    const float* gt = gate + (size_t)t * gate_ld + gate_col + g * gs;
    float ss = 0.f;
    for (int d = lane; d < gs; d += 32) {
        const float v = gate_first ? src[d] * silu_f32(gt[d]) : src[d];
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float inv = out_scale / sqrtf(ss / (float)gs + eps);
    T* dst = out + ((size_t)t * groups + g) * gs;
    for (int d = lane; d < gs; d += 32) {
        const float sg = silu_f32(gt[d]);
        const float v = gate_first ? src[d] * sg : src[d];
        const float y = v * inv * w[(g * gs + d) % w_len];
        dst[d] = from_f32<T>(gate_first ? y : y * sg);
    }
}

// The same with a block per (token, group), for groups of many channels.
template <typename T>
__global__ void __launch_bounds__(256) gated_group_norm_block_kernel(const float* x, int x_ld, const float* gate, int gate_ld, int gate_col,
                                        const float* __restrict__ w, int w_len, T* __restrict__ out, int groups,
                                        int gs, int gate_first, float eps, float out_scale) {
    __shared__ float scratch[33];
    let_next_kernel_start();
    wait_for_previous_kernels();
    const int t = blockIdx.x / groups, g = blockIdx.x % groups;
    const float* src = x + (size_t)t * x_ld + g * gs;
    const float* gt = gate + (size_t)t * gate_ld + gate_col + g * gs;
    float ss = 0.f;
    for (int d = threadIdx.x; d < gs; d += blockDim.x) {
        const float v = gate_first ? src[d] * silu_f32(gt[d]) : src[d];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = out_scale / sqrtf(ss / (float)gs + eps);
    T* dst = out + ((size_t)t * groups + g) * gs;
    for (int d = threadIdx.x; d < gs; d += blockDim.x) {
        const float sg = silu_f32(gt[d]);
        const float v = gate_first ? src[d] * sg : src[d];
        const float y = v * inv * w[(g * gs + d) % w_len];
        dst[d] = from_f32<T>(gate_first ? y : y * sg);
    }
}

constexpr int SCAN_SMEM_LIMIT = 44 * 1024;

template <int ROWS>
int launch_scan(bool delta, dim3 grid, cudaStream_t stream, Scan p, int longest, int n_seqs) {
    const int token_bytes = (2 * R * (ROWS + 4) + COLS + 4) * (int)sizeof(float);
    int tile_t = SCAN_SMEM_LIMIT / (2 * token_bytes);     // two tiles
    if (tile_t > 16) tile_t = 16;
    if (longest > 0 && tile_t > longest) tile_t = longest;
    if (tile_t < 1) tile_t = 1;
    p.tile_t = tile_t;
    const size_t smem = (size_t)2 * tile_t * token_bytes;
    cudaError_t e;
    if (delta) {
        e = launch_dependent(state_scan_kernel<ROWS, true, WHOLE>, grid, SCAN_THREADS, smem, stream, p);
    } else if (p.piece <= 0) {
        e = launch_dependent(state_scan_kernel<ROWS, false, WHOLE>, grid, SCAN_THREADS, smem, stream, p);
    } else {
        const dim3 pieces(grid.x * p.max_pieces, grid.y, grid.z);
        e = launch_dependent(state_scan_kernel<ROWS, false, LOCAL>, pieces, SCAN_THREADS, smem, stream, p);
        if (check_launch(e, "state_scan (pieces from zero)")) return 1;
        const int per_head = p.dim * p.vdim;
        e = launch_dependent(scan_carry_kernel, dim3((per_head + 255) / 256, p.heads, n_seqs), 256, 0, stream, p.state, p.piece_state,
                             (const float*)p.piece_decay, p.cu_seqlens, p.seq_slot, p.heads, per_head, p.piece, p.max_pieces);
        if (check_launch(e, "state_scan (carry)")) return 1;
        e = launch_dependent(state_scan_kernel<ROWS, false, FINAL>, pieces, SCAN_THREADS, smem, stream, p);
    }
    return check_launch(e, "state_scan");
}

}  // namespace

RI_API int ri_scan_prepare(const float* z, int ld, int conv_col, int conv_ch, const float* taps, const float* conv_bias,
                           int k_taps, float* conv_state, int unit_heads, int unit_dim, int scaled_heads, float unit_scale,
                           int heads, int decay_col, int step_col, const float* a_log, const float* dt_bias, float* out,
                           int out_ld, const int* cu_seqlens, const int* token_seq, const int* seq_slot, int n_tokens,
                           int n_seqs, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (k_taps < 1 || conv_ch < 1) return fail("scan_prepare: a convolution of %d taps over %d channels", k_taps, conv_ch);
    if (conv_col < 0 || conv_col + conv_ch > ld || decay_col + heads > ld || step_col + heads > ld)
        return fail("scan_prepare: columns beyond the projection's %d", ld);
    if (unit_heads * unit_dim > conv_ch || scaled_heads > unit_heads) return fail("scan_prepare: unit vectors beyond the convolved channels");
    if (out_ld < conv_ch + 2 * heads) return fail("scan_prepare: output rows of %d values are too short", out_ld);
    // tiles of about 512 channels; where heads are made unit vectors a tile holds whole heads (a head wider than that
    // is a tile of its own)
    int tile_ch = 512;
    if (unit_heads > 0 && unit_dim > 0) tile_ch = unit_dim * ((512 + unit_dim - 1) / unit_dim);
    if (tile_ch > conv_ch) tile_ch = conv_ch;
    const size_t smem = (size_t)tile_ch * sizeof(float);
    if (smem > 200 * 1024) return fail("scan_prepare: heads of %d channels do not fit shared memory", unit_dim);
    static PerDeviceOnce once;
    if (smem > 48 * 1024)
        if (int rc = raise_dynamic_smem(scan_prepare_kernel, 200 * 1024, once, "scan_prepare")) return rc;
    const int tiles = (conv_ch + tile_ch - 1) / tile_ch;
    if (tiles > 65535) return fail("scan_prepare: %d tiles of channels exceed the grid limit", tiles);
    Prepare p{z, ld, conv_col, conv_ch, taps, conv_bias, k_taps, conv_state, unit_heads, unit_dim, scaled_heads, unit_scale,
              heads, decay_col, step_col, a_log, dt_bias, out, out_ld, cu_seqlens, token_seq, seq_slot, tile_ch};
    cudaError_t e = launch_dependent(scan_prepare_kernel, dim3(n_tokens, tiles), 256, smem, stream, p);
    if (check_launch(e, "scan_prepare")) return 1;
    if (k_taps > 1) {
        dim3 grid((conv_ch + 127) / 128, n_seqs);
        e = launch_dependent(conv_state_kernel, grid, 128, 0, stream, z, ld, conv_col, conv_ch, k_taps, conv_state, cu_seqlens, seq_slot);
        if (check_launch(e, "scan_prepare (carried inputs)")) return 1;
    }
    return 0;
}

// u: float32 [n_tokens, ld] with the columns of queries and keys ([groups, dim] each), values ([heads, vdim]), decays and
// steps ([heads] each).  state: float32 [slots, heads, dim, vdim].  o: float32 [n_tokens, heads * vdim].
// delta != 0: the gated delta rule; else the state space (with skip [heads] or null).  longest_run: the most new tokens
// any sequence brings (0: unknown), which sizes the scan's shared memory.  piece > 0 (state space only): the three passes
// over pieces of that many tokens, with scratch piece_state [n_seqs, max_pieces, heads, dim, vdim] and piece_decay
// [n_seqs, max_pieces, heads]; max_pieces * piece covers the longest run.
RI_API int ri_state_scan(const float* u, int ld, int q_col, int k_col, int v_col, int decay_col, int step_col, const float* skip,
                         float* state, float* o, const int* cu_seqlens, const int* seq_slot, int n_seqs, int heads, int groups,
                         int dim, int vdim, int delta, int longest_run, int piece, int max_pieces, float* piece_state,
                         float* piece_decay, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (groups <= 0 || heads % groups) return fail("state_scan: %d heads are not a multiple of %d groups", heads, groups);
    if (heads > 65535) return fail("state_scan: %d heads exceed the grid limit", heads);
    if (dim > 32 * R) return fail("state_scan: a state of %d rows exceeds %d", dim, 32 * R);
    int rows = (dim + R - 1) / R;
    rows = rows <= 4 ? 4 : rows <= 8 ? 8 : rows <= 16 ? 16 : 32;
    const int vec = ((ld | q_col | k_col | v_col | dim | vdim) % 4 == 0 && (reinterpret_cast<uintptr_t>(u) & 15) == 0) ? 1 : 0;
    if (piece > 0) {
        if (delta) return fail("state_scan: the delta rule's update is not a scalar times the state: no pieces");
        if (max_pieces < 1 || piece_state == nullptr || piece_decay == nullptr) return fail("state_scan: pieces need their scratch");
        if ((long long)n_seqs * max_pieces > 0x7fffffffLL || n_seqs > 65535) return fail("state_scan: %d sequences of %d pieces exceed the grid limit", n_seqs, max_pieces);
        if (longest_run <= 0 || longest_run > piece) longest_run = piece;
    }
    Scan p{u, ld, q_col, k_col, v_col, decay_col, step_col, skip, state, o, cu_seqlens, seq_slot, heads, groups, dim, vdim, 1, vec,
           piece > 0 ? piece : 0, piece > 0 ? max_pieces : 1, piece_state, piece_decay};
    dim3 grid(n_seqs, heads, (vdim + COLS - 1) / COLS);
    if (rows == 4) return launch_scan<4>(delta != 0, grid, stream, p, longest_run, n_seqs);
    if (rows == 8) return launch_scan<8>(delta != 0, grid, stream, p, longest_run, n_seqs);
    if (rows == 16) return launch_scan<16>(delta != 0, grid, stream, p, longest_run, n_seqs);
    return launch_scan<32>(delta != 0, grid, stream, p, longest_run, n_seqs);
}

RI_API int ri_gated_group_norm(const float* x, int x_ld, const float* gate, int gate_ld, int gate_col, const float* w, int w_len,
                               void* out, int dtype, int n_tokens, int groups, int gs, int gate_first, float eps, float out_scale,
                               cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (groups <= 0 || gs <= 0 || w_len <= 0) return fail("gated_group_norm: %d groups of %d channels, %d weights", groups, gs, w_len);
    const long long warps = (long long)n_tokens * groups;
    const int blocks = (int)((warps * 32 + 255) / 256);
    const bool wide = gs >= 512 && warps <= 0x7fffffffLL;          // a block per group instead of a warp
    cudaError_t e;
    if (dtype == RI_F32)
        e = wide ? launch_dependent(gated_group_norm_block_kernel<float>, (int)warps, 256, 0, stream, x, x_ld, gate, gate_ld, gate_col,
                                    w, w_len, (float*)out, groups, gs, gate_first, eps, out_scale)
                 : launch_dependent(gated_group_norm_kernel<float>, blocks, 256, 0, stream, x, x_ld, gate, gate_ld, gate_col, w, w_len,
                                    (float*)out, n_tokens, groups, gs, gate_first, eps, out_scale);
    else if (dtype == RI_BF16)
        e = wide ? launch_dependent(gated_group_norm_block_kernel<__nv_bfloat16>, (int)warps, 256, 0, stream, x, x_ld, gate, gate_ld,
                                    gate_col, w, w_len, (__nv_bfloat16*)out, groups, gs, gate_first, eps, out_scale)
                 : launch_dependent(gated_group_norm_kernel<__nv_bfloat16>, blocks, 256, 0, stream, x, x_ld, gate, gate_ld, gate_col, w,
                                    w_len, (__nv_bfloat16*)out, n_tokens, groups, gs, gate_first, eps, out_scale);
    else
        return fail("gated_group_norm: unknown dtype %d", dtype);
    return check_launch(e, "gated_group_norm");
}

RI_DEFINE_LAST_ERROR()
