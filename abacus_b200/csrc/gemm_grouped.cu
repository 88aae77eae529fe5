// The products of routed experts for many rows, on the tcgen05 tensor cores: rows sorted by expert, every expert's
// run of rows padded to whole tiles of 128, so that a tile has one expert and the product is an ordinary tiled one
// whose weight operand is chosen per row tile.
//
//   moe_sort      pairs (token, k-th choice) -> places in the sorted order. Three launches: a count per expert (each
//                 pair draws its rank within its expert with an atomic: the order within an expert is whatever the
//                 hardware made it, which no result depends on, a row's product being its own); the experts' first
//                 places (runs padded to 128 rows) and the expert of every row tile (-1 beyond the last); the rows
//                 themselves gathered into their places, multiplied by the pair's weight where the weight acts on
//                 the expert's input (rounded to bfloat16 like any stored activation).
//   gemm_grouped  out[p, :] = act(W[expert of p's tile] x[p, :]) for the sorted rows: TMA (128-byte swizzle) -> ring
//                 of stages -> tcgen05.mma 128 x 128 x 16 into tensor memory -> tcgen05.ld epilogue, one warp that
//                 loads, one that multiplies, four that store. The weights are one matrix [experts * N, K]; a tile's
//                 weight rows start at expert * N + its column. Tiles beyond the last used one leave at once. Rows of
//                 padding hold whatever the buffer held; their results are never read.
//   moe_unsort    out[t] (+)= sum over k of sorted[place of pair t * top + k], in the order of k.
// All waits on barriers are bounded (tc::mbar_wait); a wait that runs out sets status word 1.
#define ABK_DEFINE_ERROR
#include "common.cuh"
#include "tc_common.cuh"
#include "tensor_map.cuh"

#define GG_ROWS 128
#define GG_BN 128
#define GG_K 64
#define GG_STAGES 4
#define GG_THREADS 192
enum { GG_NONE = 0, GG_RELU_SQUARED = 1 };

// ---------------------------------------------------------------- sorting pairs by expert
__global__ void __launch_bounds__(256) moe_count_kernel(const int *pair_expert, int n_pairs, int *counts, int *rank) {
    pdl_wait();
    const int p = blockIdx.x * 256 + threadIdx.x;
    if (p >= n_pairs) return;
    const int e = pair_expert[p];
    rank[p] = e >= 0 ? atomicAdd(&counts[e], 1) : 0;
}

// first[e]: the first sorted row of expert e; tile_expert[t]: the expert of row tile t, -1 beyond the used tiles.
__global__ void __launch_bounds__(256) moe_offsets_kernel(const int *counts, int experts, int *first, int *tile_expert,
                                                          int max_tiles) {
    extern __shared__ int mo_tiles[];  // [experts + 1] first tile of each expert
    pdl_wait();
    if (threadIdx.x == 0) {
        int tile = 0;
        for (int e = 0; e < experts; e++) {
            mo_tiles[e] = tile;
            first[e] = tile * GG_ROWS;
            tile += (counts[e] + GG_ROWS - 1) / GG_ROWS;
        }
        mo_tiles[experts] = tile;
    }
    __syncthreads();
    for (int t = threadIdx.x; t < max_tiles; t += 256) {
        int e = -1;
        if (t < mo_tiles[experts]) {
            int lo = 0, hi = experts - 1;  // the last expert whose first tile is <= t and that has tiles
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (mo_tiles[mid] <= t) lo = mid; else hi = mid - 1;
            }
            e = lo;
        }
        tile_expert[t] = e;
    }
}

// x row of pair p: x + (p / pairs_per_row) * ldx; its place: first[expert] + rank; sorted[place] = scale * x (bfloat16).
__global__ void __launch_bounds__(128) moe_gather_kernel(const __nv_bfloat16 *x, long long ldx, int pairs_per_row,
                                                         const int *pair_expert, const float *pair_scale, const int *rank,
                                                         const int *first, int *place, __nv_bfloat16 *sorted, int d) {
    const int p = blockIdx.x;
    pdl_wait();
    const int e = pair_expert[p];
    if (e < 0) {
        if (threadIdx.x == 0) place[p] = -1;
        return;
    }
    const int at = first[e] + rank[p];
    if (threadIdx.x == 0) place[p] = at;
    const __nv_bfloat16 *src = x + (long long)(p / pairs_per_row) * ldx;
    __nv_bfloat16 *dst = sorted + (long long)at * d;
    if (d % 8 == 0 && ldx % 8 == 0 && (((uintptr_t)x | (uintptr_t)sorted) & 15) == 0) {  // 16-byte pieces
        const float sc = pair_scale ? pair_scale[p] : 1.0f;
        for (int i = threadIdx.x * 8; i < d; i += 128 * 8) {
            uint4 raw = *(const uint4 *)(src + i);
            if (pair_scale) {
                __nv_bfloat162 *h = (__nv_bfloat162 *)&raw;
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const float2 f = __bfloat1622float2(h[u]);
                    h[u] = __floats2bfloat162_rn(sc * f.x, sc * f.y);
                }
            }
            *(uint4 *)(dst + i) = raw;
        }
    } else if (pair_scale) {
        const float sc = pair_scale[p];
        for (int i = threadIdx.x; i < d; i += 128) dst[i] = __float2bfloat16_rn(sc * __bfloat162float(src[i]));
    } else {
        for (int i = threadIdx.x; i < d; i += 128) dst[i] = src[i];
    }
}

// counts [experts], rank and place [n_pairs], first [experts], tile_expert [max_tiles] int32; sorted bfloat16
// [max_tiles * 128, d]. max_tiles >= ceil(n_pairs / 128) + experts.
extern "C" int abk_moe_sort(const void *x, long long ldx, int pairs_per_row, const int *pair_expert, const float *pair_scale,
                            int n_pairs, int experts, int d, int *counts, int *rank, int *first, int *place,
                            int *tile_expert, int max_tiles, void *sorted, void *stream) {
    if (n_pairs <= 0) return 0;
    if (max_tiles < (n_pairs + GG_ROWS - 1) / GG_ROWS + experts)
        ABK_REFUSE("moe_sort: %d row tiles do not hold %d pairs of %d experts", max_tiles, n_pairs, experts);
    if (experts > 8192) ABK_REFUSE("moe_sort: %d experts", experts);
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t err = cudaMemsetAsync(counts, 0, (size_t)experts * sizeof(int), s);
    if (err != cudaSuccess) return (int)err;
    moe_count_kernel<<<(n_pairs + 255) / 256, 256, 0, s>>>(pair_expert, n_pairs, counts, rank);
    moe_offsets_kernel<<<1, 256, (size_t)(experts + 1) * sizeof(int), s>>>(counts, experts, first, tile_expert, max_tiles);
    abk_launch(moe_gather_kernel, dim3(n_pairs), dim3(128), 0, s, (const __nv_bfloat16 *)x, ldx, pairs_per_row < 1 ? 1 : pairs_per_row,
               pair_expert, pair_scale, (const int *)rank, (const int *)first, place, (__nv_bfloat16 *)sorted, d);
    return ABK_LAUNCH_RESULT();
}

// ---------------------------------------------------------------- the product
struct GemmGrouped {
    void *out;
    long long ldo;
    int N, K, k_blocks;
    const int *tile_expert;
    int *status;
    int vec;  // every 16-column run of an output row starts on a 16-byte boundary
};

struct GroupedSmem {
    static constexpr int A_BYTES = GG_ROWS * GG_K * 2, B_BYTES = GG_BN * GG_K * 2;
    static constexpr int BYTES = GG_STAGES * (A_BYTES + B_BYTES) + 1024 /* alignment */ + 256 /* barriers */;
};

__device__ __forceinline__ void gg_store16(float *dst, const uint32_t *v) {
#pragma unroll
    for (int j = 0; j < 16; j += 4) *(uint4 *)(dst + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
}
__device__ __forceinline__ void gg_store16(__nv_bfloat16 *dst, const uint32_t *v) {
    uint32_t h[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        __nv_bfloat162 t = __floats2bfloat162_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
        h[j] = *(uint32_t *)&t;
    }
    *(uint4 *)dst = make_uint4(h[0], h[1], h[2], h[3]);
    *(uint4 *)(dst + 8) = make_uint4(h[4], h[5], h[6], h[7]);
}

template <typename TO, int ACT>
__global__ void __launch_bounds__(GG_THREADS) gemm_grouped_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                  const __grid_constant__ CUtensorMap map_w, GemmGrouped g) {
    using S = GroupedSmem;
    // the tile's expert was written at least two launches back (the gather stands between): it may be read at once
    const int expert = g.tile_expert[blockIdx.x];
    if (expert < 0) return;
    extern __shared__ uint8_t gg_smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)gg_smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *a_tiles = smem, *b_tiles = smem + GG_STAGES * S::A_BYTES;
    uint64_t *full = (uint64_t *)(smem + GG_STAGES * (S::A_BYTES + S::B_BYTES));
    uint64_t *empty = full + GG_STAGES, *acc_ready = empty + GG_STAGES;
    uint32_t *tmem_holder = (uint32_t *)(acc_ready + 1);
    volatile int *flags = (volatile int *)(tmem_holder + 1);  // [0]: a wait ran out

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p0 = blockIdx.x * GG_ROWS, q0 = blockIdx.y * GG_BN;
    const int w_row = expert * g.N + q0;
    if (threadIdx.x == 0) {
        for (int s = 0; s < GG_STAGES; s++) tc::mbar_init(&full[s], 1), tc::mbar_init(&empty[s], 1);
        tc::mbar_init(acc_ready, 1);
        flags[0] = 0;
        tc::mbar_init_fence();
        tc::tma_prefetch_map(&map_x), tc::tma_prefetch_map(&map_w);
    }
    if (warp == 1) tc::tmem_alloc(tmem_holder, GG_BN);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = *tmem_holder;
    if (warp == 0) {
        if (lane == 0) {
            // the weights' first stages are asked for at once; the rows (the launch before wrote them) after the wait
            const int ahead = min(GG_STAGES, g.k_blocks);
            for (int i = 0; i < ahead; i++) {
                tc::mbar_expect_tx(&full[i], S::A_BYTES + S::B_BYTES);
                tc::tma_load_2d(b_tiles + i * S::B_BYTES, &map_w, i * GG_K, w_row, &full[i]);
            }
            pdl_wait();
            int issued = 0;
            for (int kb = 0; kb < g.k_blocks; kb++, issued++) {
                const int s = issued % GG_STAGES;
                if (issued >= ahead) {
                    if (!tc::mbar_wait(&empty[s], ((issued / GG_STAGES) & 1) ^ 1)) {
                        flags[0] = 1;
                        break;
                    }
                    tc::mbar_expect_tx(&full[s], S::A_BYTES + S::B_BYTES);
                    tc::tma_load_2d(b_tiles + s * S::B_BYTES, &map_w, kb * GG_K, w_row, &full[s]);
                }
                tc::tma_load_2d(a_tiles + s * S::A_BYTES, &map_x, kb * GG_K, p0, &full[s]);
            }
            if (flags[0]) {  // let the copies still in flight land before the CTA's memory goes away
                for (int i = max(0, issued - GG_STAGES); i < issued; i++) tc::mbar_wait(&full[i % GG_STAGES], (i / GG_STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = tc::idesc_bf16_f32(GG_ROWS, GG_BN);
            int done = 0;
            for (int kb = 0; kb < g.k_blocks; kb++, done++) {
                const int s = done % GG_STAGES;
                if (!tc::mbar_wait(&full[s], (done / GG_STAGES) & 1)) {
                    flags[0] = 1;
                    break;
                }
                tc::fence_after_sync();
                const uint32_t a = tc::smem_addr(a_tiles + s * S::A_BYTES), b = tc::smem_addr(b_tiles + s * S::B_BYTES);
#pragma unroll
                for (int k = 0; k < GG_K / 16; k++)
                    tc::mma_ss(tmem, tc::smem_desc_k_sw128(a + k * 32), tc::smem_desc_k_sw128(b + k * 32), idesc, done > 0 || k > 0);
                tc::mma_commit(&empty[s]);
            }
            tc::mma_commit(acc_ready);
        }
    } else {
        // epilogue: warp w reads lanes 32 * (w % 4) .. + 31 of the accumulator
        const int quarter = warp & 3, row = quarter * 32 + lane;
        const bool ok = tc::mbar_wait(acc_ready, 0);
        if (!ok) flags[0] = 1;
        tc::fence_after_sync();
        TO *out = (TO *)g.out + (long long)(p0 + row) * g.ldo;
        if (ok) {
#pragma unroll 1
            for (int c0 = 0; c0 < GG_BN; c0 += 16) {
                if (q0 + c0 >= g.N) break;
                uint32_t v[16];
                tc::tmem_ld16(tmem + ((uint32_t)(quarter * 32) << 16) + c0, v);
                tc::tmem_ld_wait();
                if (ACT == GG_RELU_SQUARED) {
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const float f = __uint_as_float(v[j]);
                        v[j] = __float_as_uint(f > 0.0f ? f * f : 0.0f);
                    }
                }
                if (g.vec && q0 + c0 + 16 <= g.N) {
                    gg_store16(out + q0 + c0, v);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j++)
                        if (q0 + c0 + j < g.N) out[q0 + c0 + j] = from_float<TO>(__uint_as_float(v[j]));
                }
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (flags[0] && threadIdx.x == 0) atomicOr(g.status + 1, 1);
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_free(tmem, GG_BN);
    }
}

// x bfloat16 [max_tiles * 128, K] (sorted rows); w bfloat16 [experts, N, K]; out [max_tiles * 128, ldo] bfloat16 or
// (out_f32) float32; tile_expert int32 [max_tiles]; status int32 [>= 2].
extern "C" int abk_gemm_grouped(const void *x, const void *w, void *out, long long ldo, int out_f32, int activation,
                                int max_tiles, int experts, int N, int K, const int *tile_expert, int *status, void *stream) {
    if (max_tiles <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8) ABK_REFUSE("gemm_grouped: K = %d must be a multiple of 8", K);
    if (activation != GG_NONE && activation != GG_RELU_SQUARED) ABK_REFUSE("gemm_grouped: activation %d is not built", activation);
    CUtensorMap mx, mw;
    int rc = tmap::bf16_rows_of_128_bytes(x, (long long)max_tiles * GG_ROWS, K, K, GG_ROWS, &mx);
    if (rc) return rc;
    rc = tmap::bf16_rows_of_128_bytes(w, (long long)experts * N, K, K, GG_BN, &mw);
    if (rc) return rc;
    GemmGrouped g;
    g.out = out, g.ldo = ldo, g.N = N, g.K = K, g.k_blocks = (K + GG_K - 1) / GG_K, g.tile_expert = tile_expert, g.status = status;
    g.vec = ((uintptr_t)out % 16 == 0) && (ldo * (out_f32 ? 4 : 2)) % 16 == 0;
    dim3 grid(max_tiles, (N + GG_BN - 1) / GG_BN);
    if (grid.y > 65535) ABK_REFUSE("gemm_grouped: %d output features are more than a grid takes", N);
    cudaStream_t s = (cudaStream_t)stream;
#define GG_LAUNCH(TO, ACT)                                                                                          \
    do {                                                                                                            \
        if (cudaError_t e = abk_allow_shared_memory((const void *)gemm_grouped_kernel<TO, ACT>, GroupedSmem::BYTES)) \
            return (int)e;                                                                                          \
        abk_launch(gemm_grouped_kernel<TO, ACT>, grid, dim3(GG_THREADS), (size_t)GroupedSmem::BYTES, s, mx, mw, g); \
    } while (0)
    if (out_f32) { if (activation) GG_LAUNCH(float, 1); else GG_LAUNCH(float, 0); }
    else { if (activation) GG_LAUNCH(__nv_bfloat16, 1); else GG_LAUNCH(__nv_bfloat16, 0); }
#undef GG_LAUNCH
    return ABK_LAUNCH_RESULT();
}

// ---------------------------------------------------------------- back to the tokens' order
// A CTA a token; VEC: four columns a thread as one 16-byte piece (d a multiple of 4).
template <bool VEC>
__global__ void __launch_bounds__(256) moe_unsort_kernel(const float *sorted, const int *place, float *out, int d, int top, int add) {
    pdl_wait();
    const long long t = blockIdx.x;
    constexpr int W = VEC ? 4 : 1;
    for (int j = threadIdx.x * W; j < d; j += 256 * W) {
        float acc[W];
        bool any = false;
        for (int k = 0; k < top; k++) {
            const int at = place[t * top + k];
            if (at < 0) continue;
            float v[W];
            if (VEC) {
                const float4 r = *(const float4 *)(sorted + (long long)at * d + j);
                v[0] = r.x, v[W > 1 ? 1 : 0] = r.y, v[W > 2 ? 2 : 0] = r.z, v[W > 3 ? 3 : 0] = r.w;
            } else {
                v[0] = sorted[(long long)at * d + j];
            }
#pragma unroll
            for (int u = 0; u < W; u++) acc[u] = any ? acc[u] + v[u] : v[u];
            any = true;
        }
#pragma unroll
        for (int u = 0; u < W; u++) {
            const float a = any ? acc[u] : 0.0f;
            out[t * d + j + u] = add ? out[t * d + j + u] + a : a;
        }
    }
}

extern "C" int abk_moe_unsort(const float *sorted, const int *place, float *out, int n_tokens, int d, int top, int add,
                              void *stream) {
    if (n_tokens <= 0 || d <= 0) return 0;
    if (d % 4 == 0 && (((uintptr_t)sorted | (uintptr_t)out) & 15) == 0)
        abk_launch(moe_unsort_kernel<true>, dim3(n_tokens), dim3(256), 0, (cudaStream_t)stream, sorted, place, out, d, top, add);
    else
        abk_launch(moe_unsort_kernel<false>, dim3(n_tokens), dim3(256), 0, (cudaStream_t)stream, sorted, place, out, d, top, add);
    return ABK_LAUNCH_RESULT();
}
