// Attention over the paged cache for any head size, any number of heads and groups and
// any mix of query lengths: the 32-bit path's kernel and the bf16 path's fallback.
//
// One block per (query token, query head).  The token at position p of its sequence
// sees the cached keys 0..p of its slot, nothing else: causal by construction, as in
// attention.rs:92-121.  scores = dot(q, k) * scale, the scale applied to the finished dot
// product (attention.rs:100-110); softmax with the maximum subtracted (math.rs:104-118),
// here computed online over chunks of keys; weighted sum of the values (attention.rs:
// 114-120).  Query head h reads kv head h / (n_heads / n_kv_heads) (attention.rs:95-98).
// All arithmetic is float32 with accurate expf.
//
// `window` > 0 limits the keys to the last `window` positions (p-window+1 .. p); `chunk` > 0
// limits them to the query's own block of `chunk` positions, counted from position 0 of the
// sequence (floor(p / chunk) * chunk .. p); the dense decoder passes 0 for both.  Values may
// have another head size than keys (`v_hd`), and the result is multiplied by `out_scale`
// before it is rounded to the output type.  A value row need not be dense: `v_ld` is the distance
// between the value rows of consecutive keys (v_hd when they have a cache of their own; the key head
// size when the values are the leading channels of the keys, vcache == kcache).  The result of token t
// and head h goes to out + t * out_ld + h * out_hs (out_hs = v_hd: heads side by side in a token's row;
// out_hs = n_tokens * v_hd with out_ld = v_hd: head-major, a head's tokens consecutive).
//
// Further forms of the score and of the mask, each off when its argument is zero or null:
//   softcap     s <- softcap * tanh(s / softcap), after the scale
//   dist        s <- s - r1_h * ln(1 + r2_h * (pos - j)): a bias that grows with the distance, two numbers per head
//               (dist[h] = r1, dist[n_heads + h] = r2), taken off after the cap
//   keep_first  with a window: the first keep_first positions of the sequence stay visible beyond it
//   sink        the softmax's denominator also holds exp(sink_h): a learned number per head without key or value
//   gate        the head's result is multiplied by sigmoid(gate[t * gate_ld + h])
#include "common.cuh"

using namespace ri;

namespace {

constexpr int THREADS = 128;
constexpr int MAX_ACC = 8;          // value head size <= THREADS * MAX_ACC

template <typename T>
__global__ void __launch_bounds__(THREADS)
attn_generic_kernel(const T* __restrict__ q, int q_ld, const T* __restrict__ kcache,
                    const T* __restrict__ vcache, const int* __restrict__ page_table, int max_pages,
                    const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                    const int* __restrict__ seq_slot, T* __restrict__ out, int out_ld, int n_heads,
                    int n_kv_heads, int hd, int v_hd, int page_size, float scale, int window, int chunk,
                    float out_scale, int v_ld, long long out_hs, float softcap, int keep_first,
                    const float* __restrict__ sink, const float* __restrict__ dist, const T* gate, int gate_ld) {
    extern __shared__ float smem[];
    float* qs = smem;                 // [hd]
    float* ps = smem + hd;            // [THREADS]
    int* key_off = reinterpret_cast<int*>(ps + THREADS);   // [THREADS] element offset of each key row / hd
    __shared__ float scratch[33];

    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int kvh = h / (n_heads / n_kv_heads);
    const int pos = token_pos[t];
    const int slot = seq_slot[token_seq[t]];
    const int* pages = page_table + (size_t)slot * max_pages;

    for (int d = tid; d < hd; d += THREADS) qs[d] = to_f32<T>(q[(size_t)t * q_ld + h * hd + d]);

    int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    if (chunk > 0) first = max(first, pos - pos % chunk);
    // the keys in the order they are visited: the kept first positions the window has left behind, then the window
    const int n_kept = (window > 0 && keep_first > 0) ? min(keep_first, first) : 0;
    const int n_keys = n_kept + pos + 1 - first;
    const float r1 = dist != nullptr ? dist[h] : 0.f, r2 = dist != nullptr ? dist[n_heads + h] : 0.f;

    float m = -INFINITY, l = 0.f;
    float acc[MAX_ACC];
#pragma unroll
    for (int a = 0; a < MAX_ACC; ++a) acc[a] = 0.f;

    for (int c0 = 0; c0 < n_keys; c0 += THREADS) {
        const int jv = c0 + tid;
        const int j = jv < n_kept ? jv : first + (jv - n_kept);
        float s = -INFINITY;
        __syncthreads();              // qs ready (first pass); ps / key_off free (later passes)
        if (jv < n_keys) {
            int page = pages[j / page_size];
            if (!RI_IN_LIMIT(page, RI_LIMIT_PAGES, RI_CHECK_PAGE)) page = 0;      // checked build: recorded, read from a page that exists
            const size_t row = ((size_t)page * n_kv_heads + kvh) * page_size + (j % page_size);
            key_off[tid] = (int)row;  // rows fit in 31 bits: checked on the host
            const T* kr = kcache + row * hd;
            float dot = 0.f;
            for (int d = 0; d < hd; ++d) dot = fmaf(qs[d], to_f32<T>(kr[d]), dot);
            s = dot * scale;
            if (softcap > 0.f) s = softcap * tanhf(s / softcap);
            if (dist != nullptr) s -= r1 * log1pf(r2 * (float)(pos - j));
        }
        const float cmax = block_max(s, scratch);
        const float m_new = fmaxf(m, cmax);
        const float p = (jv < n_keys) ? expf(s - m_new) : 0.f;
        ps[tid] = p;
        const float csum = block_sum(p, scratch);      // also makes ps / key_off visible
        const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * alpha + csum;
        m = m_new;
        const int cn = min(THREADS, n_keys - c0);
#pragma unroll
        for (int a = 0; a < MAX_ACC; ++a) {
            const int d = tid + a * THREADS;
            if (d < v_hd) {
                float o = acc[a] * alpha;
                for (int jj = 0; jj < cn; ++jj)
                    o = fmaf(ps[jj], to_f32<T>(vcache[(size_t)key_off[jj] * v_ld + d]), o);
                acc[a] = o;
            }
        }
    }
    if (sink != nullptr) {            // one more term of the denominator, with no value behind it
        const float sk = sink[h];
        const float m_new = fmaxf(m, sk);
        const float alpha = expf(m - m_new);
        l = l * alpha + expf(sk - m_new);
#pragma unroll
        for (int a = 0; a < MAX_ACC; ++a) acc[a] *= alpha;
    }
    float inv = out_scale / l;
    if (gate != nullptr) {
        const float gv = to_f32<T>(gate[(size_t)t * gate_ld + h]);
        inv *= gv >= 0.f ? 1.f / (1.f + expf(-gv)) : expf(gv) / (1.f + expf(gv));
    }
#pragma unroll
    for (int a = 0; a < MAX_ACC; ++a) {
        const int d = tid + a * THREADS;
        if (d < v_hd) out[(size_t)t * out_ld + (size_t)h * out_hs + d] = from_f32<T>(acc[a] * inv);
    }
}

}  // namespace

RI_API int ri_attention_generic(const void* q, int q_ld, const void* kcache, const void* vcache,
                                const int* page_table, int max_pages, const int* token_pos,
                                const int* token_seq, const int* seq_slot, void* out, int out_ld, int dtype,
                                int n_tokens, int n_heads, int n_kv_heads, int hd, int v_hd, int page_size,
                                long long cache_rows, float scale, int window, int chunk, float out_scale,
                                int v_ld, long long out_hs, float softcap, int keep_first, const float* sink,
                                const float* dist, const void* gate, int gate_ld, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads)
        return fail("attention: %d heads are not a multiple of %d kv heads", n_heads, n_kv_heads);
    if (v_hd <= 0) v_hd = hd;
    if (v_ld <= 0) v_ld = v_hd;
    if (out_hs <= 0) out_hs = v_hd;
    if (v_ld < v_hd) return fail("attention: value rows %d apart hold %d values", v_ld, v_hd);
    if (v_hd > THREADS * MAX_ACC) return fail("attention: value head size %d exceeds %d", v_hd, THREADS * MAX_ACC);
    if (hd <= 0 || window < 0 || chunk < 0) return fail("attention: head size %d, window %d, chunk %d", hd, window, chunk);
    if (keep_first < 0 || softcap < 0.f) return fail("attention: %d kept positions, a cap of %g", keep_first, softcap);
    if (keep_first > 0 && chunk > 0) return fail("attention: kept first positions go with a window, not with chunks");
    if (cache_rows > 0x7fffffffLL) return fail("attention: cache of %lld rows exceeds 2^31", cache_rows);
    if (n_heads > 65535) return fail("attention: %d heads exceed the grid limit", n_heads);
    const size_t smem = (size_t)(hd + 2 * THREADS) * sizeof(float);
    dim3 grid(n_tokens, n_heads);
    if (dtype == RI_F32)
        attn_generic_kernel<float><<<grid, THREADS, smem, stream>>>(
            (const float*)q, q_ld, (const float*)kcache, (const float*)vcache, page_table, max_pages, token_pos,
            token_seq, seq_slot, (float*)out, out_ld, n_heads, n_kv_heads, hd, v_hd, page_size, scale, window, chunk, out_scale, v_ld, out_hs,
            softcap, keep_first, sink, dist, (const float*)gate, gate_ld);
    else if (dtype == RI_BF16)
        attn_generic_kernel<__nv_bfloat16><<<grid, THREADS, smem, stream>>>(
            (const __nv_bfloat16*)q, q_ld, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, page_table,
            max_pages, token_pos, token_seq, seq_slot, (__nv_bfloat16*)out, out_ld, n_heads, n_kv_heads, hd,
            v_hd, page_size, scale, window, chunk, out_scale, v_ld, out_hs, softcap, keep_first, sink, dist,
            (const __nv_bfloat16*)gate, gate_ld);
    else
        return fail("attention: unknown dtype %d", dtype);
    return check_launch("attention_generic");
}

RI_DEFINE_LAST_ERROR()
