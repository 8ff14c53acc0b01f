// The experts' contractions on the tensor cores: a grouped form of the token-major tcgen05 product.
//
// The (token, choice) pairs have been listed expert by expert and their activations gathered in that
// order, so an expert's rows are consecutive in X [pairs, K]; the experts' matrices are stacked,
// W [experts * N, K].  A work item is (row tile, feature tile): 128 consecutive rows of one expert
// (the list of row tiles, `tiles`, is made on the device by the arrange kernel: expert and first
// row; their number is read from device memory) times 256 rows of that expert's matrix (SiLU-gate:
// 128 gate rows stacked on the 128 up rows of the same features, one N = 256 MMA per K-slice feeding
// both).  A row tile may run past its expert's last row into the next expert's rows, and a feature
// tile past its expert's last feature into the next expert's matrix: what is computed there is not
// stored (the epilogue knows the expert's last row and N).
//
// Persistent grid, one CTA per SM: warp 0 loads by TMA into a ring of mbarrier stages, warp 1 issues
// the MMAs into one of two accumulator buffers in tensor memory, warps 2..5 read the other with
// tcgen05.ld and write it.  Every wait is bounded; a wait that runs out stores a code in the
// host-visible status word and the CTA winds down.  No load uses cluster multicast.
//
//   gate != 0  out<bf16>[row, n] = silu(X W[e]^T) * (X W2[e]^T)
//   gate == 0  out<f32>[row, n]  = X W[e]^T
#include "tcgen05_common.cuh"

using namespace ri;
using namespace ri::tc;

namespace {

constexpr int BLOCK_K = 64;                         // bf16 per k-block: one 128-byte swizzled row
constexpr int HALF_BYTES = 128 * BLOCK_K * 2;       // 128 rows of a k-block: 16 KiB
constexpr int TM_TOK = 128;                         // rows per tile (MMA M)
constexpr int TM_ROWS = 256;                        // rows of W per tile (MMA N)
constexpr int STAGE_BYTES = (TM_TOK + TM_ROWS) * BLOCK_K * 2;     // 48 KiB
constexpr int MAX_STAGES = 8;
constexpr int THREADS = 192;
constexpr int SMEM_BUDGET = 200 * 1024;

enum Status { ST_PRODUCER_TIMEOUT = 31, ST_MMA_TIMEOUT = 32, ST_EPILOGUE_TIMEOUT = 33, ST_DRAIN_TIMEOUT = 34 };

// The gate of the gated form (`GateForm`, common.cuh; without constants SiLU(g) * u, bit for bit), with the hardware's
// fast exponential and division: the result is rounded to bf16 right away.
__device__ __forceinline__ float gated_to_bf16(float g, float u, const GateForm& f) {
    g = fminf(g, f.limit);
    u = fmaxf(fminf(u, f.limit), -f.limit) + f.shift;
    return __fdividef(g, 1.f + __expf(-f.alpha * g * fmaf(f.cubic * g, g, 1.f))) * u * f.mult;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// The thread's row (TMEM lane) times the tile's features, 16 at a time.
// `spread` (plain form only): the result is rounded to bf16 and the row goes to out + out_row * out_ld instead of
// out + row * n_feat (rows of a wider matrix, in another order: see the kernel).
template <bool GATE>
__device__ __forceinline__ void write_tile(uint32_t trow, int row, bool row_ok, int f0, int n_feat, bool aligned,
                                           void* __restrict__ out_, const GateForm& gf, bool spread = false,
                                           size_t out_row = 0, int out_ld = 0) {
    constexpr int FEATS = GATE ? TM_ROWS / 2 : TM_ROWS;
    const bool narrow = GATE || spread;                     // the result is bf16
#pragma unroll 1
    for (int c0 = 0; c0 < FEATS; c0 += 16) {
        if (f0 + c0 >= n_feat) break;                       // uniform over the warp
        uint32_t v[16], u[16];
        tmem_ld16(trow + c0, v);
        if (GATE) tmem_ld16(trow + TM_ROWS / 2 + c0, u);
        tmem_wait_ld();
        if (!row_ok) continue;
        const size_t o0 = spread ? out_row * (size_t)out_ld + f0 + c0 : (size_t)row * n_feat + f0 + c0;
        float r[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float a = __uint_as_float(v[j]);
            r[j] = GATE ? gated_to_bf16(a, __uint_as_float(u[j]), gf) : a;
        }
        if (aligned && f0 + c0 + 16 <= n_feat) {
            if (narrow) {
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out_) + o0;
                uint4 lo, hi;
                lo.x = pack_bf16x2(r[0], r[1]);  lo.y = pack_bf16x2(r[2], r[3]);
                lo.z = pack_bf16x2(r[4], r[5]);  lo.w = pack_bf16x2(r[6], r[7]);
                hi.x = pack_bf16x2(r[8], r[9]);  hi.y = pack_bf16x2(r[10], r[11]);
                hi.z = pack_bf16x2(r[12], r[13]); hi.w = pack_bf16x2(r[14], r[15]);
                *reinterpret_cast<uint4*>(dst) = lo;
                *reinterpret_cast<uint4*>(dst + 8) = hi;
            } else {
                float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(out_) + o0);
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) dst[q4] = make_float4(r[4 * q4], r[4 * q4 + 1], r[4 * q4 + 2], r[4 * q4 + 3]);
            }
        } else {
            for (int j = 0; j < 16; ++j)
                if (f0 + c0 + j < n_feat) {
                    if (narrow) reinterpret_cast<__nv_bfloat16*>(out_)[o0 + j] = __float2bfloat16_rn(r[j]);
                    else reinterpret_cast<float*>(out_)[o0 + j] = r[j];
                }
        }
    }
}

template <bool GATE>
__global__ void __launch_bounds__(THREADS, 1)
moe_grouped_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
                      const __grid_constant__ CUtensorMap map_x, void* __restrict__ out_, const int* offsets,
                      const int* tiles, const int* n_tiles, int n_feat, int K, int stages,
                      int* status, int spread_groups, int spread_ld, const float* __restrict__ gate_form) {
    // spread_groups > 0 (plain form): out is bf16 with rows of spread_ld values, and row i of group e goes to row
    // i * spread_groups + e of it (the groups' rows interleaved: a group is a head, a row a token, and out a matrix
    // [tokens, heads, spread_ld] whose first n_feat channels per head are written).
    constexpr int FEATS = GATE ? TM_ROWS / 2 : TM_ROWS;        // output features per tile
    constexpr int X_BYTES = TM_TOK * BLOCK_K * 2;
    constexpr int TMEM_COLS = 2 * TM_ROWS;                     // two accumulator buffers
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TM_ROWS >> 3) << 17) |
                               ((uint32_t)(TM_TOK >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[MAX_STAGES];
    __shared__ __align__(8) uint64_t empty_bar[MAX_STAGES];
    __shared__ __align__(8) uint64_t acc_full[2];
    __shared__ __align__(8) uint64_t acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_kb = (K + BLOCK_K - 1) / BLOCK_K;
    const int n_feat_tiles = (n_feat + FEATS - 1) / FEATS;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&acc_full[i]), 1);
            mbar_init(smem_u32(&acc_empty[i]), 4);
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    const uint32_t full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);
    let_next_kernel_start();
    // The list of row tiles, the rows themselves and their number come from the kernels before: they are
    // read after the wait, through pointers that promise the compiler nothing (a `const __restrict__` load
    // may be moved ahead of the wait, where the arrays still hold the previous layer's lists).
    wait_for_previous_kernels();
    const int n_row_tiles = *reinterpret_cast<const volatile int*>(n_tiles);
    const int total_tiles = n_row_tiles * n_feat_tiles;
    const int my_tiles = ((int)blockIdx.x < total_tiles) ? (total_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    // row tiles vary fastest: CTAs that run together work on different experts
    auto tile_coords = [&](int i, int& e, int& row0, int& f0) {
        const int tile = (int)blockIdx.x + i * (int)gridDim.x;
        const int rt = tile % n_row_tiles;
        e = tiles[2 * rt];
        row0 = tiles[2 * rt + 1];
        f0 = (tile / n_row_tiles) * FEATS;
    };
    auto load_stage = [&](uint32_t stage, uint32_t bar, int kx, int w_row, int row0) {
        mbar_expect_tx(bar, STAGE_BYTES);
        tma_load_2d(stage + X_BYTES, &map_w, bar, kx, w_row);
        if (GATE) tma_load_2d(stage + X_BYTES + HALF_BYTES, &map_w2, bar, kx, w_row);
        else tma_load_2d(stage + X_BYTES + HALF_BYTES, &map_w, bar, kx, w_row + 128);
        tma_load_2d(stage, &map_x, bar, kx, row0);
    };

    if (warp == 0) {
        if (lane == 0) {
            int it = 0, s = 0;
            uint32_t ph = 0;
            bool alive = true;
            for (int i = 0; i < my_tiles && alive; ++i) {
                int e, row0, f0;
                tile_coords(i, e, row0, f0);
                if (abort_flag) break;
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    if (it >= stages && !mbar_wait(empty0 + 8u * s, ph ^ 1u)) {
                        if (!abort_flag) report(status, ST_PRODUCER_TIMEOUT);
                        abort_flag = 1;
                        alive = false;
                        break;
                    }
                    load_stage(smem_base + (uint32_t)s * STAGE_BYTES, full0 + 8u * s, kb * BLOCK_K, e * n_feat + f0, row0);
                    if (++s == stages) { s = 0; ph ^= 1u; }
                }
            }
            for (int j = max(0, it - stages); j < it; ++j)
                if (!mbar_wait(smem_u32(&full_bar[j % stages]), (uint32_t)(j / stages) & 1u)) {
                    report(status, ST_DRAIN_TIMEOUT);
                    break;
                }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool alive = true;
            const uint64_t desc_x0 = make_smem_desc(smem_base), desc_w0 = make_smem_desc(smem_base + X_BYTES);
            for (int i = 0; i < my_tiles && alive; ++i) {
                const int buf = i & 1;
                if (!mbar_wait(smem_u32(&acc_empty[buf]), ((uint32_t)(i >> 1) & 1u) ^ 1u)) {
                    report(status, ST_MMA_TIMEOUT);
                    abort_flag = 1;
                    break;
                }
                tc_fence_after();
                const uint32_t acc = tmem_base + (uint32_t)(buf * TM_ROWS);
                for (int kb = 0; kb < n_kb; ++kb) {
                    if (!mbar_wait(full0 + 8u * s, ph)) {
                        report(status, ST_MMA_TIMEOUT);
                        abort_flag = 1;
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t off = (uint64_t)((uint32_t)s * (uint32_t)(STAGE_BYTES >> 4));
#pragma unroll
                    for (int k = 0; k < BLOCK_K / 16; ++k)
                        umma(acc, desc_x0 + off + 2 * k, desc_w0 + off + 2 * k, IDESC, kb > 0 || k > 0);
                    umma_commit(empty0 + 8u * s);
                    if (++s == stages) { s = 0; ph ^= 1u; }
                }
                umma_commit(smem_u32(&acc_full[buf]));
            }
        }
    } else {
        const int lane_base = (warp & 3) * 32;
        const bool spread = !GATE && spread_groups > 0;
        const GateForm gf = load_gate_form(GATE ? gate_form : nullptr);       // constants no kernel of the step writes
        const bool aligned = spread ? spread_ld % 8 == 0 : n_feat % 8 == 0;      // rows of `out` keep 16-byte alignment
        for (int i = 0; i < my_tiles; ++i) {
            int e, row0, f0;
            tile_coords(i, e, row0, f0);
            const int row_end = offsets[e + 1];
            const int buf = i & 1;
            const bool landed = mbar_wait(smem_u32(&acc_full[buf]), (uint32_t)(i >> 1) & 1u);
            if (!landed && lane == 0) {
                report(status, ST_EPILOGUE_TIMEOUT);
                abort_flag = 1;
            }
            tc_fence_after();
            if (!landed || abort_flag) break;
            const int row = row0 + lane_base + lane;
            const uint32_t trow = tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)(buf * TM_ROWS);
            write_tile<GATE>(trow, row, row < row_end, f0, n_feat, aligned, out_, gf, spread,
                             spread ? (size_t)(row - offsets[e]) * spread_groups + e : 0, spread_ld);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

template <bool GATE>
int launch(const CUtensorMap& mw, const CUtensorMap& mw2, const CUtensorMap& mx, void* out, const int* offsets,
           const int* tiles, const int* n_tiles, int n_pairs, int experts, int N, int K, int* status, cudaStream_t stream,
           int spread_groups = 0, int spread_ld = 0, const float* gate_form = nullptr) {
    const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
    int stages = SMEM_BUDGET / STAGE_BYTES;
    if (stages > total_kb) stages = total_kb;
    // Always the whole budget, also where fewer stages would do: a CTA then has its SM to itself, so no CTA
    // of a kernel that starts early behind this one can sit on the same SM and wait for tensor memory
    // (a CTA here takes all 512 columns).
    const size_t smem = (size_t)SMEM_BUDGET + 1024;
    auto kernel = moe_grouped_tc_kernel<GATE>;
    static PerDeviceOnce configured;
    if (int rc = raise_dynamic_smem(kernel, SMEM_BUDGET + 1024, configured, "moe_grouped_tcgen05")) return rc;
    constexpr int FEATS = GATE ? TM_ROWS / 2 : TM_ROWS;
    const long long most = (long long)((n_pairs + TM_TOK - 1) / TM_TOK + experts) * ((N + FEATS - 1) / FEATS);
    long long ctas = sm_count();
    if (ctas > most) ctas = most;
    cudaError_t e = launch_dependent(kernel, dim3((unsigned)ctas), dim3(THREADS), smem, stream, mw, mw2, mx, out, offsets,
                                     tiles, n_tiles, N, K, stages, status, spread_groups, spread_ld, gate_form);
    return check_launch(e, "moe_grouped_tcgen05");
}

}  // namespace

RI_API int ri_moe_tcgen05_tile_rows() { return TM_TOK; }

// map_x: X [pairs, K] with a box of 128 rows; map_w, map_w2: [experts * N, K] with a box of 128 rows
// (`ri_gemm_tcgen05_encode` makes them).  offsets / tiles / n_tiles: the arrange kernel's, for tiles of 128 rows.
// gate_form (gated form only): the five constants of another gate than SiLU, in device memory, or null.
RI_API int ri_moe_grouped_tcgen05(const void* map_x, const void* map_w, const void* map_w2, void* out, int gate,
                                  const int* offsets, const int* tiles, const int* n_tiles, int n_pairs, int experts, int N,
                                  int K, const float* gate_form, int* status, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (K <= 0 || K % 8) return fail("moe_grouped_tcgen05: K = %d must be a positive multiple of 8 (16-byte rows for TMA)", K);
    if (gate && map_w2 == nullptr) return fail("moe_grouped_tcgen05: the SiLU-gate form needs a second matrix");
    if ((long long)experts * N > 0x7fffffffLL) return fail("moe_grouped_tcgen05: %d experts of %d rows exceed the index range", experts, N);
    const CUtensorMap& mx = *reinterpret_cast<const CUtensorMap*>(map_x);
    const CUtensorMap& mw = *reinterpret_cast<const CUtensorMap*>(map_w);
    const CUtensorMap& mw2 = *reinterpret_cast<const CUtensorMap*>(gate ? map_w2 : map_w);
    if (gate) return launch<true>(mw, mw2, mx, out, offsets, tiles, n_tiles, n_pairs, experts, N, K, status, stream, 0, 0, gate_form);
    return launch<false>(mw, mw2, mx, out, offsets, tiles, n_tiles, n_pairs, experts, N, K, status, stream);
}

// The plain form with its result rounded to bf16 and the groups' rows interleaved: row i of group e goes to
// out + (i * experts + e) * out_ld (out: bf16 [rows per group, experts, out_ld], of which the first N channels of every
// (row, group) are written).  For per-head maps whose result is wanted token by token.
RI_API int ri_moe_grouped_tcgen05_spread(const void* map_x, const void* map_w, void* out, int out_ld, const int* offsets,
                                         const int* tiles, const int* n_tiles, int n_pairs, int experts, int N, int K,
                                         int* status, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (K <= 0 || K % 8) return fail("moe_grouped_tcgen05: K = %d must be a positive multiple of 8 (16-byte rows for TMA)", K);
    if (out_ld < N) return fail("moe_grouped_tcgen05: rows of %d values cannot hold %d", out_ld, N);
    if ((long long)experts * N > 0x7fffffffLL) return fail("moe_grouped_tcgen05: %d experts of %d rows exceed the index range", experts, N);
    const CUtensorMap& mx = *reinterpret_cast<const CUtensorMap*>(map_x);
    const CUtensorMap& mw = *reinterpret_cast<const CUtensorMap*>(map_w);
    return launch<false>(mw, mw, mx, out, offsets, tiles, n_tiles, n_pairs, experts, N, K, status, stream, experts, out_ld);
}

RI_DEFINE_LAST_ERROR()
