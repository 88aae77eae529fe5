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
            const int e = tid + it * THREADS, tok = e / DP, d = e % DP;
            const bool in = tok < cnt && d < p.dim;
            const T *r = proj + (long long)(row0 + c0 + (tok < cnt ? tok : cnt - 1)) * p.ld + (long long)h * p.dim + (d < p.dim ? d : 0);
            const float q = to_float(r[p.q_at]), k = to_float(r[p.k_at]);
            rq[it] = in ? q : 0.0f, rk[it] = in ? k : 0.0f;
        }
#pragma unroll
        for (int it = 0; it < PER_V; it++) {
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
            const int e = tid + it * THREADS, tok = e / DP, d = e % DP, at = (d / DPT) * (DPT + 4) + d % DPT;
            q_s[tok][at] = silu_staged<T>(rq[it]), k_s[tok][at] = silu_staged<T>(rk[it]);
        }
#pragma unroll
        for (int it = 0; it < PER_V; it++) {
            const int e = tid + it * THREADS;
            if (e < LS_TOKENS * COLS) v_s[e / COLS][e % COLS] = silu_staged<T>(rv[it]);
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
