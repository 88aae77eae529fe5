// Linear attention with a fixed decay per head ("lightning" attention): a recurrent mixer whose state is one
// [key, value] matrix per head,
//     S_t = decay_h S_(t-1) + k_t v_t^T,    o_t = S_t^T q_t,
// float32, zero at a sequence's start and carried from step to step in the sequence's slot. q, k and v are the SiLU of
// their projections (the activation is taken here, in float32, as the rows are staged).
//
//   lightning_scan   a CTA walks one sequence's tokens for one head and 16 (32 for heads of up to 32 channels) value
//                    columns. Its threads are those columns x 4, 8 or 16 parts of the key channels (heads of 128: 16
//                    parts, 256 threads), so a thread keeps 4 to 16 state values in registers and a token costs it that
//                    many multiply-adds twice; the parts' partial outputs of a column meet by shuffles, four tokens at a time. Rows come sixteen tokens at a time: asked for a
//                    chunk ahead into registers, their activation taken on the way into shared memory, read from
//                    there as 16-byte pieces. A sequence that brings no token to the step is left alone.
//   gated_row_norm   out = w * o / sqrt(mean(o^2) + eps) * sigmoid(g) over a token's whole row (all heads together).
#define ABK_DEFINE_ERROR
#include "common.cuh"

#define LS_TOKENS 16

struct LightningScan {
    const void *proj;  // row t at proj + t * ld: q head h at q_at + h * dim, k at k_at + h * dim, v at v_at + h * vdim
    long long ld;
    int q_at, k_at, v_at;
    int n_heads, dim, vdim;
    const float *decay;  // [heads]
    float *state;        // [slots][heads][dim][vdim]
    float *out;          // [tokens][heads * vdim]
    const int *seq_start, *seq_slot;
};

__device__ __forceinline__ float silu_exact(float z) { return z / (1.0f + expf(-z)); }
// The activation of a staged element: to the last bit where the model is float32; where its operands are bfloat16
// numbers, by the special-function unit (a few units in the last place of float32: far below what was rounded away).
template <typename T> __device__ __forceinline__ float silu_staged(float z) { return silu_exact(z); }
template <> __device__ __forceinline__ float silu_staged<__nv_bfloat16>(float z) { return silu_mul_fast(z, 1.0f); }

// N tokens of one thread's share: q, k point at the thread's channels of the first token (tokens `pitch` floats apart),
// v at its column's value (tokens `v_pitch` apart); the column's output goes to out (tokens `out_pitch` apart) if `writes`.
template <int DPT, int PARTS, int N>
__device__ __forceinline__ void scan_tokens(float *s, float decay, const float *q, const float *k, int pitch, const float *v,
                                            int v_pitch, bool writes, float *out, long long out_pitch) {
    float vv[N], o[N];
#pragma unroll
    for (int n = 0; n < N; n++) vv[n] = v[n * v_pitch], o[n] = 0.0f;
#pragma unroll
    for (int i = 0; i < DPT / 4; i++) {
        float4 kk[N], qq[N];
#pragma unroll
        for (int n = 0; n < N; n++) kk[n] = *(const float4 *)(k + n * pitch + 4 * i), qq[n] = *(const float4 *)(q + n * pitch + 4 * i);
#pragma unroll
        for (int n = 0; n < N; n++) {
            s[4 * i] = fmaf(decay, s[4 * i], kk[n].x * vv[n]), s[4 * i + 1] = fmaf(decay, s[4 * i + 1], kk[n].y * vv[n]);
            s[4 * i + 2] = fmaf(decay, s[4 * i + 2], kk[n].z * vv[n]), s[4 * i + 3] = fmaf(decay, s[4 * i + 3], kk[n].w * vv[n]);
            o[n] = fmaf(s[4 * i + 3], qq[n].w, fmaf(s[4 * i + 2], qq[n].z, fmaf(s[4 * i + 1], qq[n].y, fmaf(s[4 * i], qq[n].x, o[n]))));
        }
    }
#pragma unroll
    for (int m = 1; m < PARTS; m <<= 1)
#pragma unroll
        for (int n = 0; n < N; n++) o[n] += __shfl_xor_sync(0xffffffffu, o[n], m);
    if (writes)
#pragma unroll
        for (int n = 0; n < N; n++) out[n * out_pitch] = o[n];
}

// DPT key channels a thread, PARTS threads a value column (DPT * PARTS >= dim); a CTA has COLS columns.
template <typename T, int DPT, int PARTS, int COLS> __global__ void __launch_bounds__(PARTS * COLS, 2) lightning_scan_kernel(LightningScan p) {
    constexpr int DP = DPT * PARTS;             // key channels, padded
    constexpr int PITCH = PARTS * (DPT + 4);    // a token's channels in shared memory: a part's run, then 4 floats of
    constexpr int THREADS = PARTS * COLS;       // padding, so that the parts' 16-byte reads meet no bank twice
    constexpr int PER = LS_TOKENS * DP / THREADS;  // elements of q (and of k) a thread stages a chunk
    constexpr int PER_V = (LS_TOKENS * COLS + THREADS - 1) / THREADS;
    __shared__ __align__(16) float q_s[LS_TOKENS][PITCH], k_s[LS_TOKENS][PITCH];
    __shared__ float v_s[LS_TOKENS][COLS];
    const int tile = blockIdx.x, h = blockIdx.y, seq = blockIdx.z, tid = threadIdx.x, part = tid % PARTS, vc = tid / PARTS;
    const int col = tile * COLS + vc;
    const float decay = p.decay[h];
    pdl_wait();
    const int row0 = p.seq_start[seq], n = p.seq_start[seq + 1] - row0;
    if (n <= 0) return;  // (a sequence of the step's padding: its slot is someone else's)
    float *state = p.state + ((long long)p.seq_slot[seq] * p.n_heads + h) * p.dim * p.vdim;
    float s[DPT];
#pragma unroll
    for (int i = 0; i < DPT; i++) {
        const int d = part * DPT + i;
        s[i] = d < p.dim && col < p.vdim ? state[(long long)d * p.vdim + col] : 0.0f;
    }
    const T *proj = (const T *)p.proj;
    // a chunk's rows are asked for a chunk ahead, into registers, so that their way from memory lies under the
    // chunk before; the activation is taken as they go into shared memory
    float rq[PER], rk[PER], rv[PER_V];
    auto fetch = [&](int c0) {
        const int cnt = n - c0 < LS_TOKENS ? n - c0 : LS_TOKENS;
#pragma unroll
        for (int it = 0; it < PER; it++) {
            // (every load is made, from a place that exists, and dropped where it is not wanted: loads that hang on no
            // branch are all in flight together)
            if (it * THREADS >= cnt * DP) break;  // (the same for every thread: the chunk has no such token)
            const int e = tid + it * THREADS, tok = e / DP, d = e % DP;
            const bool in = tok < cnt && d < p.dim;
            const T *r = proj + (long long)(row0 + c0 + (tok < cnt ? tok : cnt - 1)) * p.ld + (long long)h * p.dim + (d < p.dim ? d : 0);
            const float q = to_float(r[p.q_at]), k = to_float(r[p.k_at]);
            rq[it] = in ? q : 0.0f, rk[it] = in ? k : 0.0f;
        }
#pragma unroll
        for (int it = 0; it < PER_V; it++) {
            if (it * THREADS >= cnt * COLS) break;
            const int e = tid + it * THREADS, tok = e / COLS, c = tile * COLS + e % COLS;
            const float v = to_float(proj[(long long)(row0 + c0 + (tok < cnt ? tok : cnt - 1)) * p.ld + p.v_at + (long long)h * p.vdim +
                                          (c < p.vdim ? c : 0)]);
            rv[it] = tok < cnt && c < p.vdim ? v : 0.0f;
        }
    };
    fetch(0);
    for (int c0 = 0; c0 < n; c0 += LS_TOKENS) {
        const int cnt = n - c0 < LS_TOKENS ? n - c0 : LS_TOKENS;
        __syncthreads();  // the chunk before is done with
#pragma unroll
        for (int it = 0; it < PER; it++) {
            if (it * THREADS >= cnt * DP) break;
            const int e = tid + it * THREADS, tok = e / DP, d = e % DP, at = (d / DPT) * (DPT + 4) + d % DPT;
            q_s[tok][at] = silu_staged<T>(rq[it]), k_s[tok][at] = silu_staged<T>(rk[it]);
        }
#pragma unroll
        for (int it = 0; it < PER_V; it++) {
            const int e = tid + it * THREADS;
            if (e < cnt * COLS) v_s[e / COLS][e % COLS] = silu_staged<T>(rv[it]);
        }
        __syncthreads();
        if (c0 + LS_TOKENS < n) fetch(c0 + LS_TOKENS);
        // four tokens at a time: their reads from shared memory and their shuffles overlap, and only the state's own
        // multiply-adds follow one another
        int tok = 0;
        for (; tok + 4 <= cnt; tok += 4) scan_tokens<DPT, PARTS, 4>(s, decay, &q_s[tok][part * (DPT + 4)], &k_s[tok][part * (DPT + 4)], PITCH,
                                                                    &v_s[tok][vc], COLS, part == 0 && col < p.vdim,
                                                                    p.out + (long long)(row0 + c0 + tok) * p.n_heads * p.vdim + (long long)h * p.vdim + col,
                                                                    (long long)p.n_heads * p.vdim);
        for (; tok < cnt; tok++) scan_tokens<DPT, PARTS, 1>(s, decay, &q_s[tok][part * (DPT + 4)], &k_s[tok][part * (DPT + 4)], PITCH,
                                                            &v_s[tok][vc], COLS, part == 0 && col < p.vdim,
                                                            p.out + (long long)(row0 + c0 + tok) * p.n_heads * p.vdim + (long long)h * p.vdim + col,
                                                            (long long)p.n_heads * p.vdim);
    }
#pragma unroll
    for (int i = 0; i < DPT; i++) {
        const int d = part * DPT + i;
        if (d < p.dim && col < p.vdim) state[(long long)d * p.vdim + col] = s[i];
    }
}

extern "C" int abk_lightning_scan(const void *proj, long long ld, int dtype, int q_at, int k_at, int v_at, int n_heads,
                                  int dim, int vdim, const float *decay, float *state, float *out, const int *seq_start,
                                  const int *seq_slot, int n_seqs, void *stream) {
    if (n_seqs <= 0) return 0;
    if (dim < 1 || dim > 256) ABK_REFUSE("lightning_scan: %d key channels a head are not 1 to 256", dim);
    if (vdim < 1 || n_heads < 1 || n_heads > 65535 || n_seqs > 65535)
        ABK_REFUSE("lightning_scan: %d heads of %d values, %d sequences", n_heads, vdim, n_seqs);
    LightningScan p;
    p.proj = proj, p.ld = ld, p.q_at = q_at, p.k_at = k_at, p.v_at = v_at, p.n_heads = n_heads, p.dim = dim, p.vdim = vdim;
    p.decay = decay, p.state = state, p.out = out, p.seq_start = seq_start, p.seq_slot = seq_slot;
    cudaStream_t s = (cudaStream_t)stream;
    const int cols = dim <= 32 ? 32 : 16;  // value columns a CTA has
    dim3 grid((vdim + cols - 1) / cols, n_heads, n_seqs);
#define LS_LAUNCH(T)                                                                                \
    do {                                                                                            \
        if (dim <= 16) abk_launch(lightning_scan_kernel<T, 4, 4, 32>, grid, dim3(128), 0, s, p);        \
        else if (dim <= 32) abk_launch(lightning_scan_kernel<T, 8, 4, 32>, grid, dim3(128), 0, s, p);   \
        else if (dim <= 64) abk_launch(lightning_scan_kernel<T, 8, 8, 16>, grid, dim3(128), 0, s, p);   \
        else if (dim <= 128) abk_launch(lightning_scan_kernel<T, 8, 16, 16>, grid, dim3(256), 0, s, p); \
        else abk_launch(lightning_scan_kernel<T, 16, 16, 16>, grid, dim3(256), 0, s, p);                \
    } while (0)
    if (dtype == ABK_BF16) LS_LAUNCH(__nv_bfloat16);
    else LS_LAUNCH(float);
#undef LS_LAUNCH
    return ABK_LAUNCH_RESULT();
}

// ---------------------------------------------------------------- the same recurrence in chunks, for prompts
// A sequence's tokens in chunks of 64. With a the head's decay, S the state before a chunk, i and j tokens of it:
//     o_i = a^(i+1) S^T q_i + sum over j <= i of a^(i-j) (q_i . k_j) v_j,      S' = a^n S + sum_j a^(n-1-j) k_j v_j^T
// so the chunks' own sums are made side by side (chunk_states), the states before every chunk follow from them in
// one walk over whole matrices (chunk_prefix), and the outputs again side by side (chunk_outputs): what runs along
// the sequence is one multiply-add a chunk and state value instead of a token's whole chain. All float32, on the
// CUDA cores (scores and the state are float32 by the design's rule); sums are taken in another order than token by
// token, within float32's rounding.
#define LC_TOKENS 64
#define LC_PITCH 68  // floats between rows of the transposed tiles (a multiple of 4 that is no multiple of 32)

struct LightningChunks {
    LightningScan s;
    float *sums;   // [chunks][heads][dim][vdim]: a chunk's own sum, then (after the prefix) the state before it
    int n_seqs, max_chunks;
};

// (sequence, chunk within it) of chunk number c in the step's order, or false beyond the last
__device__ __forceinline__ bool chunk_of(const LightningChunks &p, int c, int &seq, int &chunk, int &first_chunk) {
    int before = 0;
    for (seq = 0; seq < p.n_seqs; seq++) {
        const int n = p.s.seq_start[seq + 1] - p.s.seq_start[seq], nc = (n + LC_TOKENS - 1) / LC_TOKENS;
        if (c < before + nc) {
            chunk = c - before, first_chunk = before;
            return true;
        }
        before += nc;
    }
    return false;
}

// sums[c][h][d][col] = sum_j a^(n-1-j) k_j[d] v_j[col] over the chunk's n tokens. A CTA: 128 channels x 128 columns,
// a thread 8 x 8 of them.
template <typename T> __global__ void __launch_bounds__(256) chunk_states_kernel(LightningChunks p, int v_tiles) {
    extern __shared__ __align__(16) float lc_smem[];
    float *k_s = lc_smem, *v_s = lc_smem + LC_TOKENS * 128;  // [64][128] each
    __shared__ float pw[LC_TOKENS];                            // pw[m] = a^m
    const int c = blockIdx.x, h = blockIdx.y, d_tile = blockIdx.z / v_tiles, v_tile = blockIdx.z % v_tiles, tid = threadIdx.x;
    const int dim = p.s.dim, vdim = p.s.vdim;
    const float a = p.s.decay[h];
    pdl_wait();
    int seq, chunk, first;
    if (!chunk_of(p, c, seq, chunk, first)) return;
    const int row0 = p.s.seq_start[seq] + chunk * LC_TOKENS;
    const int n = min(LC_TOKENS, p.s.seq_start[seq + 1] - row0);
    const T *proj = (const T *)p.s.proj;
    if (tid < LC_TOKENS) pw[tid] = powf(a, (float)tid);
    __syncthreads();
    for (int e = tid; e < LC_TOKENS * 128; e += 256) {
        const int j = e >> 7, x = e & 127, d = d_tile * 128 + x, col = v_tile * 128 + x;
        float k = 0.0f, v = 0.0f;
        if (j < n) {
            const T *r = proj + (long long)(row0 + j) * p.s.ld;
            if (d < dim) k = silu_staged<T>(to_float(r[p.s.k_at + (long long)h * dim + d])) * pw[n - 1 - j];
            if (col < vdim) v = silu_staged<T>(to_float(r[p.s.v_at + (long long)h * vdim + col]));
        }
        k_s[e] = k, v_s[e] = v;
    }
    __syncthreads();
    const int ty = tid >> 4, tx = tid & 15;
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int u = 0; u < 8; u++) acc[i][u] = 0.0f;
    for (int j = 0; j < n; j++) {
        const float4 k0 = *(const float4 *)(k_s + j * 128 + ty * 8), k1 = *(const float4 *)(k_s + j * 128 + ty * 8 + 4);
        const float4 v0 = *(const float4 *)(v_s + j * 128 + tx * 8), v1 = *(const float4 *)(v_s + j * 128 + tx * 8 + 4);
        const float kk[8] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w}, vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
        for (int i = 0; i < 8; i++)
#pragma unroll
            for (int u = 0; u < 8; u++) acc[i][u] = fmaf(kk[i], vv[u], acc[i][u]);
    }
    float *dst = p.sums + ((long long)c * p.s.n_heads + h) * dim * vdim;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int d = d_tile * 128 + ty * 8 + i;
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int col = v_tile * 128 + tx * 8 + u;
            if (d < dim && col < vdim) dst[(long long)d * vdim + col] = acc[i][u];
        }
    }
}

// Along a sequence: sums[c] becomes the state before chunk c, and the slot's state the one after the last chunk.
__global__ void __launch_bounds__(256) chunk_prefix_kernel(LightningChunks p) {
    const int seq = blockIdx.z, h = blockIdx.y;
    const long long per_head = (long long)p.s.dim * p.s.vdim, e = (long long)blockIdx.x * 256 + threadIdx.x;
    const float a = p.s.decay[h];
    pdl_wait();
    const int n = p.s.seq_start[seq + 1] - p.s.seq_start[seq];
    if (n <= 0 || e >= per_head) return;
    int first = 0;
    for (int q = 0; q < seq; q++) first += (p.s.seq_start[q + 1] - p.s.seq_start[q] + LC_TOKENS - 1) / LC_TOKENS;
    float *state = p.s.state + ((long long)p.s.seq_slot[seq] * p.s.n_heads + h) * per_head + e;
    float s = *state;
    const float full = powf(a, (float)LC_TOKENS);
    const int chunks = (n + LC_TOKENS - 1) / LC_TOKENS;
    const long long step = (long long)p.s.n_heads * per_head;
    float *at = p.sums + ((long long)first * p.s.n_heads + h) * per_head + e;
    for (int c0 = 0; c0 < chunks; c0 += 8) {  // eight chunks' own sums are asked for together, then walked
        float own[8];
#pragma unroll
        for (int i = 0; i < 8; i++) own[i] = c0 + i < chunks ? at[(c0 + i) * step] : 0.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            if (c0 + i >= chunks) break;
            const int left = n - (c0 + i) * LC_TOKENS;
            at[(c0 + i) * step] = s;
            s = fmaf(left >= LC_TOKENS ? full : powf(a, (float)left), s, own[i]);
        }
    }
    *state = s;
}

// The chunk's outputs for 128 value columns. Shared memory: q and k transposed [channel][token], v [token][column],
// the decayed causal scores transposed [j][i] (where k was). A thread: 4 x 4 scores, then 4 tokens x 8 columns of the output.
template <typename T> __global__ void __launch_bounds__(256) chunk_outputs_kernel(LightningChunks p, int dim_pad) {
    extern __shared__ __align__(16) float lc_smem[];
    // (the scores take k's place once every thread has made its own: two CTAs then share an SM)
    const int k_rows = dim_pad > LC_TOKENS ? dim_pad : LC_TOKENS;
    float *q_t = lc_smem, *k_t = q_t + dim_pad * LC_PITCH, *v_s = k_t + k_rows * LC_PITCH;  // v_s [64][128]
    float *p_t = k_t, *pw = v_s + LC_TOKENS * 128;                                          // pw[n] = a^n, n <= 64
    const int c = blockIdx.x, h = blockIdx.y, v_tile = blockIdx.z, tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int dim = p.s.dim, vdim = p.s.vdim;
    const float a = p.s.decay[h];
    pdl_wait();
    int seq, chunk, first;
    if (!chunk_of(p, c, seq, chunk, first)) return;
    const int row0 = p.s.seq_start[seq] + chunk * LC_TOKENS;
    const int n = min(LC_TOKENS, p.s.seq_start[seq + 1] - row0);
    const T *proj = (const T *)p.s.proj;
    if (tid <= LC_TOKENS) pw[tid] = powf(a, (float)tid);
    for (int e = tid; e < LC_TOKENS * dim_pad; e += 256) {
        const int j = e / dim_pad, d = e - j * dim_pad;
        float q = 0.0f, k = 0.0f;
        if (j < n && d < dim) {
            const T *r = proj + (long long)(row0 + j) * p.s.ld + (long long)h * dim + d;
            q = silu_staged<T>(to_float(r[p.s.q_at])), k = silu_staged<T>(to_float(r[p.s.k_at]));
        }
        q_t[d * LC_PITCH + j] = q, k_t[d * LC_PITCH + j] = k;
    }
    for (int e = tid; e < LC_TOKENS * 128; e += 256) {
        const int j = e >> 7, col = v_tile * 128 + (e & 127);
        v_s[e] = j < n && col < vdim
            ? silu_staged<T>(to_float(proj[(long long)(row0 + j) * p.s.ld + p.s.v_at + (long long)h * vdim + col])) : 0.0f;
    }
    __syncthreads();
    {   // scores: tokens i0..i0+3 against j0..j0+3, nothing above the diagonal
        const int i0 = ty * 4, j0 = tx * 4;
        float sc[4][4];
#pragma unroll
        for (int i = 0; i < 4; i++) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.0f;
        if (j0 <= i0 + 3) {
            for (int d = 0; d < dim; d++) {
                const float4 q = *(const float4 *)(q_t + d * LC_PITCH + i0), k = *(const float4 *)(k_t + d * LC_PITCH + j0);
                const float qq[4] = {q.x, q.y, q.z, q.w}, kk[4] = {k.x, k.y, k.z, k.w};
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) sc[i][j] = fmaf(qq[i], kk[j], sc[i][j]);
            }
        }
        __syncthreads();  // every thread is done with k
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++)
                p_t[(j0 + j) * LC_PITCH + i0 + i] = j0 + j <= i0 + i ? sc[i][j] * pw[i0 + i - j0 - j] : 0.0f;
    }
    __syncthreads();
    const int i0 = ty * 4, c0 = tx * 8;
    float acc[4][8];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int u = 0; u < 8; u++) acc[i][u] = 0.0f;
    // what the state before the chunk gives: q_i^T S, then a^(i+1) on it
    const float *state = p.sums + ((long long)c * p.s.n_heads + h) * dim * vdim;
    const int col0 = v_tile * 128 + c0;
    const bool whole = col0 + 8 <= vdim && vdim % 4 == 0;
    for (int d0 = 0; d0 < dim; d0 += 4) {  // four channels' rows of the state are asked for together
        float ss[4][8];
#pragma unroll
        for (int x = 0; x < 4; x++) {
            const float *sr = state + (long long)(d0 + x < dim ? d0 + x : dim - 1) * vdim + col0;
            if (whole) {
                const float4 s0 = *(const float4 *)sr, s1 = *(const float4 *)(sr + 4);
                ss[x][0] = s0.x, ss[x][1] = s0.y, ss[x][2] = s0.z, ss[x][3] = s0.w;
                ss[x][4] = s1.x, ss[x][5] = s1.y, ss[x][6] = s1.z, ss[x][7] = s1.w;
            } else {
#pragma unroll
                for (int u = 0; u < 8; u++) ss[x][u] = col0 + u < vdim ? sr[u] : 0.0f;
            }
        }
#pragma unroll
        for (int x = 0; x < 4; x++) {
            // (channels beyond dim are rows of zeros in q_t: dim_pad is dim rounded up to 4)
            const float4 q = *(const float4 *)(q_t + (d0 + x) * LC_PITCH + i0);
            const float qq[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int u = 0; u < 8; u++) acc[i][u] = fmaf(qq[i], ss[x][u], acc[i][u]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int u = 0; u < 8; u++) acc[i][u] *= pw[i0 + i + 1];
    // what the chunk's own tokens give
    for (int j = 0; j < n; j++) {
        const float4 w = *(const float4 *)(p_t + j * LC_PITCH + i0);
        const float4 v0 = *(const float4 *)(v_s + j * 128 + c0), v1 = *(const float4 *)(v_s + j * 128 + c0 + 4);
        const float ww[4] = {w.x, w.y, w.z, w.w}, vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int u = 0; u < 8; u++) acc[i][u] = fmaf(ww[i], vv[u], acc[i][u]);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        if (i0 + i >= n) break;
        float *dst = p.s.out + (long long)(row0 + i0 + i) * p.s.n_heads * vdim + (long long)h * vdim + col0;
#pragma unroll
        for (int u = 0; u < 8; u++)
            if (col0 + u < vdim) dst[u] = acc[i][u];
    }
}

// The recurrence of a step that brings prompts, in chunks of 64 tokens. sums: float32 scratch of at least
// max_chunks * heads * dim * vdim, max_chunks >= ceil(tokens / 64) + sequences.
extern "C" int abk_lightning_chunks(const void *proj, long long ld, int dtype, int q_at, int k_at, int v_at, int n_heads,
                                    int dim, int vdim, const float *decay, float *state, float *out, const int *seq_start,
                                    const int *seq_slot, int n_seqs, int max_chunks, float *sums, long long sums_floats,
                                    void *stream) {
    if (n_seqs <= 0 || max_chunks <= 0) return 0;
    if (dim < 1 || dim > 256) ABK_REFUSE("lightning_chunks: %d key channels a head are not 1 to 256", dim);
    if (vdim < 1 || n_heads < 1 || n_heads > 65535 || n_seqs > 65535)
        ABK_REFUSE("lightning_chunks: %d heads of %d values, %d sequences", n_heads, vdim, n_seqs);
    if ((long long)max_chunks * n_heads * dim * vdim > sums_floats)
        ABK_REFUSE("lightning_chunks: the scratch memory holds %lld floats, the step needs %lld", sums_floats,
                   (long long)max_chunks * n_heads * dim * vdim);
    LightningChunks p;
    p.s.proj = proj, p.s.ld = ld, p.s.q_at = q_at, p.s.k_at = k_at, p.s.v_at = v_at, p.s.n_heads = n_heads, p.s.dim = dim;
    p.s.vdim = vdim, p.s.decay = decay, p.s.state = state, p.s.out = out, p.s.seq_start = seq_start, p.s.seq_slot = seq_slot;
    p.sums = sums, p.n_seqs = n_seqs, p.max_chunks = max_chunks;
    cudaStream_t s = (cudaStream_t)stream;
    const int d_tiles = (dim + 127) / 128, v_tiles = (vdim + 127) / 128, dim_pad = (dim + 3) & ~3;
    const size_t smem_a = (size_t)2 * LC_TOKENS * 128 * 4;
    const size_t smem_c = ((size_t)(dim_pad + (dim_pad > LC_TOKENS ? dim_pad : LC_TOKENS)) * LC_PITCH + LC_TOKENS * 128 + LC_TOKENS + 4) * 4;
    const long long per_head = (long long)dim * vdim;
#define LC_LAUNCH(T)                                                                                                   \
    do {                                                                                                               \
        cudaError_t e = abk_allow_shared_memory((const void *)chunk_states_kernel<T>, (int)smem_a);                    \
        if (e == cudaSuccess) e = abk_allow_shared_memory((const void *)chunk_outputs_kernel<T>, (int)smem_c);         \
        if (e != cudaSuccess) return (int)e;                                                                           \
        abk_launch(chunk_states_kernel<T>, dim3(max_chunks, n_heads, d_tiles * v_tiles), dim3(256), smem_a, s, p, v_tiles); \
        abk_launch(chunk_prefix_kernel, dim3((unsigned)((per_head + 255) / 256), n_heads, n_seqs), dim3(256), 0, s, p); \
        abk_launch(chunk_outputs_kernel<T>, dim3(max_chunks, n_heads, v_tiles), dim3(256), smem_c, s, p, dim_pad);     \
    } while (0)
    if (dtype == ABK_BF16) LC_LAUNCH(__nv_bfloat16);
    else LC_LAUNCH(float);
#undef LC_LAUNCH
    return ABK_LAUNCH_RESULT();
}

// out[t] = w * o[t] / sqrt(mean(o[t]^2) + eps) * sigmoid(gate[t]); o float32 [tokens, width]; gate (the output type's)
// at gate + t * ld_gate; rows of the step's padding (token_seq < 0) become zeros.
template <typename T>
__global__ void __launch_bounds__(128) gated_row_norm_kernel(const float *o, const T *gate, long long ld_gate, const float *w,
                                                             T *out, int width, float eps, const int *token_seq) {
    __shared__ float scratch[33];
    const int t = blockIdx.x, tid = threadIdx.x;
    pdl_wait();
    T *dst = out + (long long)t * width;
    if (token_seq[t] < 0) {
        for (int i = tid; i < width; i += 128) dst[i] = from_float<T>(0.0f);
        return;
    }
    const float *src = o + (long long)t * width;
    const T *g = gate + (long long)t * ld_gate;
    float ss = 0.0f;
    for (int i = tid; i < width; i += 128) ss = fmaf(src[i], src[i], ss);
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = tid; i < width; i += 128)
        dst[i] = from_float<T>(src[i] * inv * w[i] * (1.0f / (1.0f + expf(-to_float(g[i])))));
}

extern "C" int abk_gated_row_norm(const float *o, const void *gate, long long ld_gate, const float *w, void *out, int dtype,
                                  int n_tokens, int width, float eps, const int *token_seq, void *stream) {
    if (n_tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == ABK_BF16)
        abk_launch(gated_row_norm_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(128), 0, s, o, (const __nv_bfloat16 *)gate,
                   ld_gate, w, (__nv_bfloat16 *)out, width, eps, token_seq);
    else
        abk_launch(gated_row_norm_kernel<float>, dim3(n_tokens), dim3(128), 0, s, o, (const float *)gate, ld_gate, w,
                   (float *)out, width, eps, token_seq);
    return ABK_LAUNCH_RESULT();
}
