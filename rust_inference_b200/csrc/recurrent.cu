// A gated linear recurrence with a matrix state per head (the HGRN2 form of linear attention):
//
//     S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T          S: [dim, vdim] per head, float32
//     o_t = S_t^T q_t
//
// with q = silu(zq), f = low + (1 - low) * sigmoid(zf + bias): the write weight 1 - f is tied to the forget
// gate and takes a key's place.  The keyed form (gated linear attention) has a key of its own,
//
//     S_t = diag(f_t) S_(t-1) + k_t v_t^T,      f = sigmoid(W2 (W1 h) + b)^(1/tau),  q = (Wq h) dim^(-1/2),
//
// its decay from a low-rank map, and a gate silu(g) on the normed result.  The state lives in a per-slot area of the cache, starts at zero when a
// slot is handed out and is carried from step to step, so a prompt may be cut anywhere and a decode
// step is the same kernels with one token per sequence.  Everything here is float32: gates,
// sigmoid, the state, the per-head RMS norm that follows.
//
// Three kernels, all reading the step's arrays on the device (graph-safe):
//   prepare  zq <- silu(zq), zf <- low + (1 - low) sigmoid(zf + bias), in place, every token at once
//            (long runs only: the one-pass scan of a decode step or a short portion does it in its tile)
//   scan     per (sequence, head, tile of value columns): the recurrence over the sequence's new
//            tokens in order; the state is read first and written last.  Long runs of new tokens are
//            cut into pieces that are scanned side by side (see below), all in float32
//   norm     per (token, head): o / sqrt(mean(o^2) + eps) * w * out_scale -> the run dtype
//
// The projections z = [zq | zf | v] arrive as one float32 matrix [tokens, ld].  What an earlier kernel of the
// step wrote is read after `wait_for_previous_kernels()` through plain pointers (a `const __restrict__` load
// may be moved ahead of the wait).
#include "common.cuh"

using namespace ri;

namespace {

__device__ __forceinline__ float sigmoid_f32(float x) {
    if (x >= 0.f) return 1.f / (1.f + expf(-x));
    const float e = expf(x);
    return e / (1.f + e);
}

__global__ void recurrence_prepare_kernel(float* __restrict__ z, int ld, const float* __restrict__ bias,
                                          const float* __restrict__ low, int n_tokens, int qdim) {
    let_next_kernel_start();
    wait_for_previous_kernels();
    const size_t total = (size_t)n_tokens * qdim;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / qdim), c = (int)(i % qdim);
        float* row = z + (size_t)t * ld;
        row[c] = silu_f32(row[c]);
        const float l = low[c];
        row[qdim + c] = l + (1.f - l) * sigmoid_f32(row[qdim + c] + bias[c]);
    }
}

// Threads of a warp: lane = column_in_warp * R + r.  Thread (r, j) keeps ROWS consecutive rows
// (r * ROWS ...) of columns j and j + 32 of the state in registers (its gates and query values, read once
// per token from shared memory, serve both columns: the scan is bound by those reads); the sum over rows of S[i, j] q[i] is finished by
// log2(R) shuffles inside the warp.  The tokens' q, f and v come through shared memory in tiles of up to 64
// tokens, fetched by all threads at once with cp.async (a token's gates are shared by the block's columns),
// so the loop over a tile's tokens touches no global memory but its one store of o.
//
// A long run of new tokens is cut into pieces of `piece` tokens that run side by side (three passes):
//   LOCAL   every piece from a zero state: its end state and the product of its gates go to scratch
//   (carry) per state element, piece after piece: scratch <- the state the piece starts from,
//           running <- gates' product * running + the piece's end state; the slot's state at the end
//   FINAL   every piece again, from its true start state: writes o
// A short run (one piece per sequence: decode steps, small portions) is one pass, WHOLE: from the
// slot's state, writing o and the slot's state.
constexpr int R = 8;                 // row slices per column
constexpr int CPT = 2;               // value columns per thread: a thread's gates serve both
constexpr int COLS = 32 * CPT;       // value columns per block
constexpr int SCAN_THREADS = R * 32;
enum ScanMode { WHOLE = 0, LOCAL = 1, FINAL = 2 };

// Shared memory of the scan: tiles of up to `tile_t` tokens, per token f and q as [R][ROWS + 4] (a slice of
// ROWS channels per row slice, padded so that the eight slices' 16-byte reads fall into different banks;
// channels beyond `dim` stay zero) and the block's COLS values of v.
template <int ROWS, bool KEYED = false>
struct ScanTile {
    static constexpr int SLICE = ROWS + 4;
    static constexpr int V_AT = (KEYED ? 3 : 2) * R * SLICE;    // f, q (, k), then the values
    static constexpr int TOKEN = V_AT + COLS;                   // floats per token
};

__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Where a token's numbers are: q, v (and k: KEYED) in the rows of z at the columns q_col, v_col, k_col (+ the head's
// offset), the gates f in the rows of fz (which may be z itself) at f_col.
struct ScanCols { int q_col, f_col, v_col, k_col, f_ld; };

// The keyed form's decays and query scale for the one-pass scan, which forms them in its tile (no kernel of their own
// for a step's few tokens): decay = sigmoid(bias + w2 a)^(1/tau) with a = the `rank` values at a_col of a token's row
// of z, and q times q_scale.  w2 == nullptr: the gates come from memory as they are.
struct KeyedPrep { const float* w2; const float* bias; int rank, a_col; float inv_tau, q_scale; };

template <int ROWS, bool VEC, int mode, bool KEYED>
__global__ void __launch_bounds__(SCAN_THREADS)
recurrence_scan_kernel(const float* z, int ld, const float* fz, ScanCols at, float* __restrict__ o_raw, float* state,
                       float* piece_state, float* piece_gates, const int* __restrict__ cu_seqlens,
                       const int* __restrict__ seq_slot, int heads, int dim, int vdim, int piece, int max_pieces,
                       int tile_t, const float* __restrict__ prep_bias, const float* __restrict__ prep_low, KeyedPrep keyed) {
    using Tile = ScanTile<ROWS, KEYED>;
    const bool forms_decays = KEYED && mode == WHOLE && keyed.w2 != nullptr;
    extern __shared__ __align__(16) float tile[];
    const int b = blockIdx.x / max_pieces, c = blockIdx.x % max_pieces, h = blockIdx.y;
    const int r = threadIdx.x % R, jj = threadIdx.x / R;
    const int j0 = blockIdx.z * COLS;                            // the thread's columns: j0 + jj + 32 c
    const int i0 = r * ROWS;
    for (int i = threadIdx.x; i < tile_t * Tile::TOKEN; i += SCAN_THREADS) tile[i] = 0.f;
    let_next_kernel_start();
    wait_for_previous_kernels();
    const int t0 = cu_seqlens[b] + c * piece;
    const int seq_end = cu_seqlens[b + 1];
    if (t0 >= seq_end) return;                                   // uniform over the block
    const int t1 = (mode == WHOLE) ? seq_end : min(seq_end, t0 + piece);
    float* S = nullptr;
    if (mode == WHOLE) {
        const int slot = seq_slot[b];
        if (!RI_BLOCK_IN_LIMIT(slot, RI_LIMIT_SLOTS, RI_CHECK_SLOT)) return;
        S = state + (((size_t)slot * heads + h) * dim) * vdim;
    } else {
        S = piece_state + (((size_t)blockIdx.x * heads + h) * dim) * vdim;
    }
    bool live[CPT];
    float s[CPT][ROWS], g[ROWS];
#pragma unroll
    for (int cc = 0; cc < CPT; ++cc) {
        const int j = j0 + jj + 32 * cc;
        live[cc] = j < vdim;
#pragma unroll
        for (int k = 0; k < ROWS; ++k)
            s[cc][k] = (mode != LOCAL && live[cc] && i0 + k < dim) ? S[(size_t)(i0 + k) * vdim + j] : 0.f;
    }
#pragma unroll
    for (int k = 0; k < ROWS; ++k) g[k] = 1.f;
    const int q_off = at.q_col + h * dim, f_off = at.f_col + h * dim, v_off = at.v_col + h * vdim + j0;
    const int k_off = at.k_col + h * dim, f_ld = at.f_ld;
    const int cols = min(COLS, vdim - j0);
    const int o_ld = heads * vdim;
    __syncthreads();                                              // the zeros are in place

    for (int tb = t0; tb < t1; tb += tile_t) {
        const int n_tok = min(tile_t, t1 - tb);
        // ---- the tile's q, f and v into shared memory, all threads, everything in flight at once ----
        if (VEC) {
            const int dq = dim / 4, parts = KEYED ? 3 : 2;
            const int per = parts * dq + cols / 4;                // 16-byte items per token: f, q (, k), v
            for (int idx = threadIdx.x; idx < n_tok * per; idx += SCAN_THREADS) {
                const int tok = idx / per, it = idx % per;
                const float* row = z + (size_t)(tb + tok) * ld;
                float* base = tile + tok * Tile::TOKEN;
                if (it < dq) {
                    const int ch = 4 * it;
                    if (!forms_decays)
                        cp_async16(base + (ch / ROWS) * Tile::SLICE + ch % ROWS, fz + (size_t)(tb + tok) * f_ld + f_off + ch);
                } else if (it < 2 * dq) {
                    const int ch = 4 * (it - dq);
                    if (mode != LOCAL)                            // a piece's end state needs no q
                        cp_async16(base + R * Tile::SLICE + (ch / ROWS) * Tile::SLICE + ch % ROWS, row + q_off + ch);
                } else if (KEYED && it < 3 * dq) {
                    const int ch = 4 * (it - 2 * dq);
                    cp_async16(base + 2 * R * Tile::SLICE + (ch / ROWS) * Tile::SLICE + ch % ROWS, row + k_off + ch);
                } else {
                    const int cc = 4 * (it - parts * dq);
                    cp_async16(base + Tile::V_AT + cc, row + v_off + cc);
                }
            }
            cp_async_wait_all();
        } else {
            const int parts = KEYED ? 3 : 2;
            const int per = parts * dim + cols;
            for (int idx = threadIdx.x; idx < n_tok * per; idx += SCAN_THREADS) {
                const int tok = idx / per, it = idx % per;
                const float* row = z + (size_t)(tb + tok) * ld;
                float* base = tile + tok * Tile::TOKEN;
                if (it < dim) {
                    if (!forms_decays) base[(it / ROWS) * Tile::SLICE + it % ROWS] = fz[(size_t)(tb + tok) * f_ld + f_off + it];
                } else if (it < 2 * dim) base[R * Tile::SLICE + ((it - dim) / ROWS) * Tile::SLICE + (it - dim) % ROWS] = row[q_off + it - dim];
                else if (KEYED && it < 3 * dim)
                    base[2 * R * Tile::SLICE + ((it - 2 * dim) / ROWS) * Tile::SLICE + (it - 2 * dim) % ROWS] = row[k_off + it - 2 * dim];
                else base[Tile::V_AT + it - parts * dim] = row[v_off + it - parts * dim];
            }
        }
        __syncthreads();
        if (forms_decays) {
            // the keyed form's decays of this head's channels and the queries' scale, in the tile
            for (int idx = threadIdx.x; idx < n_tok * dim; idx += SCAN_THREADS) {
                const int tok = idx / dim, ch = idx % dim;
                const float* a = z + (size_t)(tb + tok) * ld + keyed.a_col;
                const float* w = keyed.w2 + (size_t)(h * dim + ch) * keyed.rank;
                float acc = keyed.bias[h * dim + ch];
                for (int rr = 0; rr < keyed.rank; ++rr) acc = fmaf(w[rr], a[rr], acc);
                const float log_sig = fminf(acc, 0.f) - log1pf(expf(-fabsf(acc)));
                float* base = tile + tok * Tile::TOKEN + (ch / ROWS) * Tile::SLICE + ch % ROWS;
                base[0] = expf(log_sig * keyed.inv_tau);
                base[R * Tile::SLICE] *= keyed.q_scale;
            }
            __syncthreads();
        }
        if (!KEYED && mode == WHOLE && prep_bias != nullptr) {
            // the one-pass form applies the activations itself (no kernel of its own for a step's few tokens):
            // f <- low + (1 - low) sigmoid(f + bias), q <- silu(q), in the tile
            for (int idx = threadIdx.x; idx < n_tok * 2 * dim; idx += SCAN_THREADS) {
                const int tok = idx / (2 * dim), it = idx % (2 * dim);
                const int ch = it < dim ? it : it - dim;
                float* at = tile + tok * Tile::TOKEN + (it < dim ? 0 : R * Tile::SLICE) + (ch / ROWS) * Tile::SLICE + ch % ROWS;
                if (it < dim) {
                    const float l = prep_low[h * dim + ch];
                    *at = l + (1.f - l) * sigmoid_f32(*at + prep_bias[h * dim + ch]);
                } else {
                    *at = silu_f32(*at);
                }
            }
            __syncthreads();
        }
        // ---- the recurrence over the tile, out of shared memory ----
        for (int tok = 0; tok < n_tok; ++tok) {
            const float* base = tile + tok * Tile::TOKEN;
            const float4* f4 = reinterpret_cast<const float4*>(base + r * Tile::SLICE);
            const float4* q4 = reinterpret_cast<const float4*>(base + R * Tile::SLICE + r * Tile::SLICE);
            const float4* k4 = reinterpret_cast<const float4*>(base + 2 * R * Tile::SLICE + r * Tile::SLICE);   // KEYED only
            float v[CPT], acc0[CPT], acc1[CPT];
#pragma unroll
            for (int cc = 0; cc < CPT; ++cc) {
                v[cc] = base[Tile::V_AT + jj + 32 * cc];             // columns beyond vdim: zero, never stored
                acc0[cc] = acc1[cc] = 0.f;
            }
#pragma unroll
            for (int k4i = 0; k4i < ROWS / 4; ++k4i) {
                const float4 fv = f4[k4i], qv = mode != LOCAL ? q4[k4i] : make_float4(0.f, 0.f, 0.f, 0.f);
                const float4 kv = KEYED ? k4[k4i] : make_float4(0.f, 0.f, 0.f, 0.f);
                const float ff[4] = {fv.x, fv.y, fv.z, fv.w}, qq[4] = {qv.x, qv.y, qv.z, qv.w}, kk[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int k = 4 * k4i + u;
                    if (mode == LOCAL) g[k] *= ff[u];
#pragma unroll
                    for (int cc = 0; cc < CPT; ++cc) {
                        // f s + (1 - f) v, or with a key f s + k v; channels beyond dim: f = 0, q = 0, k = 0
                        s[cc][k] = KEYED ? fmaf(ff[u], s[cc][k], kk[u] * v[cc])
                                         : fmaf(ff[u], s[cc][k], fmaf(-ff[u], v[cc], v[cc]));
                        if (mode != LOCAL) {
                            if (u & 1) acc1[cc] = fmaf(s[cc][k], qq[u], acc1[cc]); else acc0[cc] = fmaf(s[cc][k], qq[u], acc0[cc]);
                        }
                    }
                }
            }
            if (mode != LOCAL) {
#pragma unroll
                for (int cc = 0; cc < CPT; ++cc) {
                    float acc = acc0[cc] + acc1[cc];
#pragma unroll
                    for (int o = R / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                    if (live[cc] && r == 0) o_raw[(size_t)(tb + tok) * o_ld + h * vdim + j0 + jj + 32 * cc] = acc;
                }
            }
        }
        __syncthreads();                                          // the tile may be overwritten
    }
    if (mode != FINAL) {
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc)
#pragma unroll
            for (int k = 0; k < ROWS; ++k)
                if (live[cc] && i0 + k < dim) S[(size_t)(i0 + k) * vdim + j0 + jj + 32 * cc] = s[cc][k];
    }
    if (mode == LOCAL && blockIdx.z == 0 && jj == 0) {
        float* G = piece_gates + ((size_t)blockIdx.x * heads + h) * dim;
#pragma unroll
        for (int k = 0; k < ROWS; ++k)
            if (i0 + k < dim) G[i0 + k] = g[k];
    }
}

// Per state element, piece after piece: the state each piece starts from, and the slot's state at the end.
__global__ void recurrence_carry_kernel(float* state, float* piece_state,
                                        const float* piece_gates, const int* __restrict__ cu_seqlens,
                                        const int* __restrict__ seq_slot, int heads, int dim, int vdim, int piece,
                                        int max_pieces) {
    let_next_kernel_start();
    wait_for_previous_kernels();
    const int b = blockIdx.y;
    const size_t per_seq = (size_t)heads * dim * vdim;
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= per_seq) return;
    const int n_new = cu_seqlens[b + 1] - cu_seqlens[b];
    const int pieces = (n_new + piece - 1) / piece;
    const int slot = seq_slot[b];
    if (!RI_IN_LIMIT(slot, RI_LIMIT_SLOTS, RI_CHECK_SLOT)) return;
    const size_t row = e / vdim;                                  // head * dim + channel
    float running = state[(size_t)slot * per_seq + e];
    for (int c = 0; c < pieces; ++c) {
        const size_t at = (size_t)(b * max_pieces + c);
        const float local = piece_state[at * per_seq + e];
        piece_state[at * per_seq + e] = running;
        running = fmaf(piece_gates[at * heads * dim + row], running, local);
    }
    state[(size_t)slot * per_seq + e] = running;
}

// One warp per (token, head): RMS norm over the head's vdim values with one weight shared by heads; with `gate`
// (float32 rows of gate_ld values, the head's at gate_col + h * vdim) the result is also times silu(gate).
template <typename T>
__global__ void headwise_rmsnorm_kernel(const float* x, int ld, int col0, const float* __restrict__ w,
                                        T* __restrict__ out, int out_ld, int n_tokens, int heads, int vdim,
                                        float eps, float out_scale, const float* gate, int gate_ld, int gate_col) {
    let_next_kernel_start();
    wait_for_previous_kernels();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n_tokens * heads) return;
    const int t = warp / heads, h = warp % heads;
    const float* src = x + (size_t)t * ld + col0 + h * vdim;
    float ss = 0.f;
    for (int d = lane; d < vdim; d += 32) ss = fmaf(src[d], src[d], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
    T* dst = out + (size_t)t * out_ld + h * vdim;
    if (gate != nullptr) {
        const float* g = gate + (size_t)t * gate_ld + gate_col + h * vdim;
        for (int d = lane; d < vdim; d += 32) dst[d] = from_f32<T>(src[d] * inv * w[d] * silu_f32(g[d]) * out_scale);
    } else {
        for (int d = lane; d < vdim; d += 32) dst[d] = from_f32<T>(src[d] * inv * w[d] * out_scale);
    }
}

// The keyed form's decays and queries, every token at once.  A block takes PREP_TOKENS tokens and PREP_CHANNELS key
// channels: the tokens' low-rank inputs a = z[t, a_col ..] (rank values each) go to shared memory, and a thread reads its
// channel's row of W2 once for all of them (16 bytes at a time where the rank allows):
//     decay[t, c] = sigmoid(b[c] + W2[c, :] . a_t)^(1/tau) = exp(log_sigmoid(.) / tau),       z[t, q_col + c] *= q_scale
// log_sigmoid(x) = min(x, 0) - log1p(exp(-|x|)): no overflow on either side, and no 1 - tiny for decays near 1.
// A decode step's few tokens are spread over the SMs by the channels.
constexpr int PREP_TOKENS = 8;
constexpr int PREP_CHANNELS = 128;
template <bool VEC>
__global__ void __launch_bounds__(PREP_CHANNELS)
keyed_prepare_kernel(float* z, int ld, int q_col, int a_col, int rank, const float* __restrict__ w2,
                     const float* __restrict__ bias, float inv_tau, float q_scale, float* __restrict__ decay, int n_tokens,
                     int qdim) {
    extern __shared__ __align__(16) float a_sh[];                // [PREP_TOKENS][rank]
    const int c = blockIdx.y * PREP_CHANNELS + threadIdx.x;
    const float b = c < qdim ? bias[c] : 0.f;
    let_next_kernel_start();
    wait_for_previous_kernels();
    const int t0 = blockIdx.x * PREP_TOKENS;
    const int n_here = min(PREP_TOKENS, n_tokens - t0);
    for (int i = threadIdx.x; i < PREP_TOKENS * rank; i += blockDim.x) {
        const int k = i / rank, r = i % rank;
        a_sh[i] = k < n_here ? z[(size_t)(t0 + k) * ld + a_col + r] : 0.f;
    }
    __syncthreads();
    if (c >= qdim) return;
    float acc[PREP_TOKENS];
#pragma unroll
    for (int k = 0; k < PREP_TOKENS; ++k) acc[k] = b;
    const float* w = w2 + (size_t)c * rank;
    if (VEC) {
        for (int r = 0; r < rank; r += 4) {
            const float4 wv = *reinterpret_cast<const float4*>(w + r);
#pragma unroll
            for (int k = 0; k < PREP_TOKENS; ++k) {
                const float4 av = *reinterpret_cast<const float4*>(a_sh + k * rank + r);
                acc[k] = fmaf(wv.x, av.x, fmaf(wv.y, av.y, fmaf(wv.z, av.z, fmaf(wv.w, av.w, acc[k]))));
            }
        }
    } else {
        for (int r = 0; r < rank; ++r) {
            const float wv = w[r];
#pragma unroll
            for (int k = 0; k < PREP_TOKENS; ++k) acc[k] = fmaf(wv, a_sh[k * rank + r], acc[k]);
        }
    }
#pragma unroll
    for (int k = 0; k < PREP_TOKENS; ++k) {
        if (k >= n_here) break;
        const float x = acc[k];
        const float log_sig = fminf(x, 0.f) - log1pf(expf(-fabsf(x)));
        decay[(size_t)(t0 + k) * qdim + c] = expf(log_sig * inv_tau);
        z[(size_t)(t0 + k) * ld + q_col + c] *= q_scale;
    }
}


constexpr int SCAN_SMEM_LIMIT = 96 * 1024;       // two blocks to an SM

template <int ROWS, bool KEYED>
int launch_scan(bool vec, dim3 grid, cudaStream_t stream, const float* z, int ld, const float* fz, ScanCols at, float* o_raw,
                float* state, float* piece_state, float* piece_gates, const int* cu_seqlens, const int* seq_slot, int heads,
                int dim, int vdim, int mode, int piece, int max_pieces, int longest, const float* prep_bias,
                const float* prep_low, KeyedPrep keyed) {
    const int token_bytes = ScanTile<ROWS, KEYED>::TOKEN * (int)sizeof(float);
    int tile_t = SCAN_SMEM_LIMIT / token_bytes;
    if (tile_t > 64) tile_t = 64;
    if (tile_t > longest) tile_t = longest;                      // a decode step brings one token
    if (tile_t < 1) return fail("gated_recurrence: a token's %d bytes of gates do not fit shared memory", token_bytes);
    const size_t smem = (size_t)tile_t * token_bytes;
    cudaError_t e = cudaSuccess;
#define RI_LAUNCH(V, M)                                                                                                   \
    {                                                                                                                     \
        auto kernel = recurrence_scan_kernel<ROWS, V, M, KEYED>;                                                          \
        static PerDeviceOnce once;                                                                                        \
        if (int rc = raise_dynamic_smem(kernel, SCAN_SMEM_LIMIT, once, "gated_recurrence")) return rc;                    \
        e = launch_dependent(kernel, grid, SCAN_THREADS, smem, stream, z, ld, fz, at, o_raw, state, piece_state,          \
                             piece_gates, cu_seqlens, seq_slot, heads, dim, vdim, piece, max_pieces, tile_t, prep_bias,   \
                             prep_low, keyed);                                                                            \
    }
    if (vec) {
        if (mode == WHOLE) RI_LAUNCH(true, WHOLE) else if (mode == LOCAL) RI_LAUNCH(true, LOCAL) else RI_LAUNCH(true, FINAL)
    } else {
        if (mode == WHOLE) RI_LAUNCH(false, WHOLE) else if (mode == LOCAL) RI_LAUNCH(false, LOCAL) else RI_LAUNCH(false, FINAL)
    }
#undef RI_LAUNCH
    return check_launch(e, "gated_recurrence (scan)");
}

// The scan of every sequence's new tokens (one pass, or pieces side by side with a carry between two passes), then the
// per-head norm (with the gate, if any) into `out`.
template <bool KEYED>
int scan_and_norm(const float* z, int ld, const float* fz, ScanCols at, const float* prep_bias, const float* prep_low,
                  const float* norm_w, float* state, const int* cu_seqlens, const int* seq_slot, float* o_raw, void* out,
                  int dtype, int n_tokens, int n_seqs, int heads, int dim, int vdim, float eps, float out_scale, int piece,
                  int max_pieces, float* scratch, int longest_run, const float* gate, int gate_ld, int gate_col,
                  cudaStream_t stream, KeyedPrep keyed = KeyedPrep{nullptr, nullptr, 0, 0, 0.f, 1.f}) {
    int rows = (dim + R - 1) / R;
    rows = rows <= 4 ? 4 : rows <= 8 ? 8 : rows <= 16 ? 16 : rows <= 32 ? 32 : 64;
    const bool vec = dim % 4 == 0 && vdim % 4 == 0 && ld % 4 == 0 && at.f_ld % 4 == 0 && (uintptr_t)z % 16 == 0 &&
                     (uintptr_t)fz % 16 == 0 && at.q_col % 4 == 0 && at.f_col % 4 == 0 && at.v_col % 4 == 0 &&
                     at.k_col % 4 == 0;
    const int col_tiles = (vdim + COLS - 1) / COLS;
    float* piece_state = scratch;
    float* piece_gates = piece > 0 ? scratch + (size_t)n_seqs * max_pieces * heads * dim * vdim : nullptr;
    auto scan = [&](int mode) -> int {
        const int mp = mode == WHOLE ? 1 : max_pieces;
        dim3 grid(n_seqs * mp, heads, col_tiles);
        const int longest = mode == WHOLE ? (longest_run > 0 ? longest_run : n_tokens) : piece;
#define RI_SCAN(ROWS) launch_scan<ROWS, KEYED>(vec, grid, stream, z, ld, fz, at, o_raw, state, piece_state, piece_gates,        \
                                               cu_seqlens, seq_slot, heads, dim, vdim, mode, piece > 0 ? piece : 1, mp, longest, \
                                               mode == WHOLE ? prep_bias : nullptr, mode == WHOLE ? prep_low : nullptr, keyed)
        if (rows == 4) return RI_SCAN(4);
        if (rows == 8) return RI_SCAN(8);
        if (rows == 16) return RI_SCAN(16);
        if (rows == 32) return RI_SCAN(32);
        return RI_SCAN(64);
#undef RI_SCAN
    };
    if (piece <= 0) {
        if (scan(WHOLE)) return 1;
    } else {
        if (scan(LOCAL)) return 1;
        const size_t per_seq = (size_t)heads * dim * vdim;
        dim3 grid((unsigned)((per_seq + 255) / 256), n_seqs);
        cudaError_t e = launch_dependent(recurrence_carry_kernel, grid, 256, 0, stream, state, piece_state,
                                         (const float*)piece_gates, cu_seqlens, seq_slot, heads, dim, vdim, piece, max_pieces);
        if (check_launch(e, "gated_recurrence (carry)")) return 1;
        if (scan(FINAL)) return 1;
    }
    const long long warps = (long long)n_tokens * heads;
    const int blocks = (int)((warps * 32 + 255) / 256);
    cudaError_t e;
    if (dtype == RI_F32)
        e = launch_dependent(headwise_rmsnorm_kernel<float>, blocks, 256, 0, stream, (const float*)o_raw, heads * vdim, 0, norm_w,
                             (float*)out, heads * vdim, n_tokens, heads, vdim, eps, out_scale, gate, gate_ld, gate_col);
    else if (dtype == RI_BF16)
        e = launch_dependent(headwise_rmsnorm_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const float*)o_raw, heads * vdim, 0,
                             norm_w, (__nv_bfloat16*)out, heads * vdim, n_tokens, heads, vdim, eps, out_scale, gate, gate_ld,
                             gate_col);
    else
        return fail("gated_recurrence: unknown dtype %d", dtype);
    return check_launch(e, "gated_recurrence (norm)");
}

}  // namespace

// Floats of scratch a call with pieces needs: [n_seqs * max_pieces] states and gate products.
RI_API long long ri_gated_recurrence_scratch(int n_seqs, int max_pieces, int heads, int dim, int vdim) {
    return (long long)n_seqs * max_pieces * heads * dim * ((long long)vdim + 1);
}

// z: float32 [n_tokens, ld] = [zq (heads*dim) | zf (heads*dim) | v (heads*vdim)]; with pieces zq and zf are
// overwritten by q and f.  o_raw: float32 [n_tokens, heads*vdim] scratch.  state: float32 [slots, heads, dim, vdim].
// out: [n_tokens, heads*vdim] in `dtype`.  piece > 0: sequences' new tokens are cut into pieces of that many
// tokens, at most max_pieces per sequence (the longest run of new tokens / piece, rounded up), worked on side
// by side with `scratch` (ri_gated_recurrence_scratch floats); piece == 0: one pass per sequence.
// longest_run: the most new tokens any sequence brings (0: unknown), which sizes the scan's shared memory.
RI_API int ri_gated_recurrence(float* z, int ld, const float* bias, const float* low, const float* norm_w,
                               float* state, const int* cu_seqlens, const int* seq_slot, float* o_raw, void* out, int dtype,
                               int n_tokens, int n_seqs, int heads, int dim, int vdim, float eps, float out_scale,
                               int piece, int max_pieces, float* scratch, int longest_run, cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (ld < 2 * heads * dim + heads * vdim) return fail("gated_recurrence: rows of %d values are too short", ld);
    if (heads > 65535) return fail("gated_recurrence: %d heads exceed the grid limit", heads);
    if (dim > 64 * R) return fail("gated_recurrence: a head of %d channels exceeds %d", dim, 64 * R);
    if (piece > 0 && (max_pieces <= 0 || scratch == nullptr)) return fail("gated_recurrence: pieces need scratch");
    const int qdim = heads * dim;
    if (piece > 0) {                      // the one-pass scan applies the activations itself
        const size_t total = (size_t)n_tokens * qdim;
        const int blocks = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
        cudaError_t e = launch_dependent(recurrence_prepare_kernel, blocks, 256, 0, stream, z, ld, bias, low, n_tokens, qdim);
        if (check_launch(e, "gated_recurrence (prepare)")) return 1;
    }
    const ScanCols at{0, qdim, 2 * qdim, 0, ld};
    return scan_and_norm<false>(z, ld, z, at, bias, low, norm_w, state, cu_seqlens, seq_slot, o_raw, out, dtype, n_tokens,
                                n_seqs, heads, dim, vdim, eps, out_scale, piece, max_pieces, scratch, longest_run, nullptr, 0, 0,
                                stream);
}

// The keyed form (gated linear attention).  z: float32 [n_tokens, ld], a token's projections before anything else
// touched them: queries at q_col, keys at k_col (heads*dim each), values at v_col and the result's gates at g_col
// (heads*vdim each), the decay's low-rank input at a_col (rank values).  w2: float32 [heads*dim, rank], bias: float32
// [heads*dim]: decay = sigmoid(w2 a + bias)^(1/tau) into `decay` (float32 [n_tokens, heads*dim], scratch); the queries
// are scaled by q_scale in place.  Without pieces (a step's few tokens) the one-pass scan forms decays and scaled
// queries in its tile instead, and neither `decay` nor z is written.  Then S <- diag(decay) S + k v^T, o = S^T q per head from the slot's state, and
// out = o / rms(o) * norm_w * silu(gate) * out_scale per head.  Pieces, scratch, o_raw, longest_run: as above.
RI_API int ri_gated_linear_attention(float* z, int ld, int q_col, int k_col, int v_col, int g_col, int a_col, int rank,
                                     const float* w2, const float* bias, float tau, float q_scale, float* decay,
                                     const float* norm_w, float* state, const int* cu_seqlens, const int* seq_slot,
                                     float* o_raw, void* out, int dtype, int n_tokens, int n_seqs, int heads, int dim,
                                     int vdim, float eps, float out_scale, int piece, int max_pieces, float* scratch,
                                     int longest_run, cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    const int qdim = heads * dim;
    if (q_col < 0 || k_col < 0 || v_col < 0 || g_col < 0 || a_col < 0 || rank <= 0 ||
        ld < q_col + qdim || ld < k_col + qdim || ld < v_col + heads * vdim || ld < g_col + heads * vdim || ld < a_col + rank)
        return fail("gated_linear_attention: rows of %d values do not hold the columns asked for", ld);
    if (!(tau > 0.f)) return fail("gated_linear_attention: tau = %f must be positive", (double)tau);
    if (heads > 65535) return fail("gated_linear_attention: %d heads exceed the grid limit", heads);
    if (dim > 64 * R) return fail("gated_linear_attention: a head of %d channels exceeds %d", dim, 64 * R);
    if (piece > 0 && (max_pieces <= 0 || scratch == nullptr)) return fail("gated_linear_attention: pieces need scratch");
    const size_t smem = (size_t)PREP_TOKENS * rank * sizeof(float);
    if (smem > 48 * 1024) return fail("gated_linear_attention: a decay of rank %d exceeds the kernel's shared memory", rank);
    const dim3 prep_grid((n_tokens + PREP_TOKENS - 1) / PREP_TOKENS, (qdim + PREP_CHANNELS - 1) / PREP_CHANNELS);
    if (prep_grid.y > 65535) return fail("gated_linear_attention: %d key channels exceed the grid limit", qdim);
    const ScanCols at{q_col, 0, v_col, k_col, qdim};
    if (piece <= 0)           // a step's few tokens: the one-pass scan forms the decays in its tile
        return scan_and_norm<true>(z, ld, decay, at, nullptr, nullptr, norm_w, state, cu_seqlens, seq_slot, o_raw, out, dtype,
                                   n_tokens, n_seqs, heads, dim, vdim, eps, out_scale, piece, max_pieces, scratch, longest_run, z,
                                   ld, g_col, stream, KeyedPrep{w2, bias, rank, a_col, 1.f / tau, q_scale});
    const bool prep_vec = rank % 4 == 0 && (uintptr_t)w2 % 16 == 0;
    cudaError_t e = prep_vec
        ? launch_dependent(keyed_prepare_kernel<true>, prep_grid, PREP_CHANNELS, smem, stream, z, ld, q_col, a_col, rank, w2, bias,
                           1.f / tau, q_scale, decay, n_tokens, qdim)
        : launch_dependent(keyed_prepare_kernel<false>, prep_grid, PREP_CHANNELS, smem, stream, z, ld, q_col, a_col, rank, w2, bias,
                           1.f / tau, q_scale, decay, n_tokens, qdim);
    if (check_launch(e, "gated_linear_attention (prepare)")) return 1;
    return scan_and_norm<true>(z, ld, decay, at, nullptr, nullptr, norm_w, state, cu_seqlens, seq_slot, o_raw, out, dtype,
                               n_tokens, n_seqs, heads, dim, vdim, eps, out_scale, piece, max_pieces, scratch, longest_run, z, ld,
                               g_col, stream);
}

RI_DEFINE_LAST_ERROR()
