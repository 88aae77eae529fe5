// Linear attention with a fixed decay per head ("lightning" attention): a recurrent mixer whose state is one
// [key, value] matrix per head,
//     S_t = decay_h S_(t-1) + k_t v_t^T,    o_t = S_t^T q_t,
// float32, zero at a sequence's start and carried from step to step in the sequence's slot. q, k and v are the SiLU of
// their projections (the activation is taken here, in float32, as the rows are staged).
//
//   lightning_scan   a CTA walks one sequence's tokens for one head and 32 value columns. Its 128 threads are 32
//                    columns x 4 quarters of the key channels (channel d belongs to quarter d % 4), so a thread keeps
//                    dim / 4 state values in registers and a token costs it that many multiply-adds twice; the four
//                    partial outputs of a column meet by two shuffles. Rows come into shared memory sixteen tokens at
//                    a time. A sequence that brings no token to the step is left alone.
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

template <typename T, int DPT> __global__ void __launch_bounds__(128) lightning_scan_kernel(LightningScan p) {
    constexpr int DP = 4 * DPT;  // key channels, padded
    __shared__ float q_s[LS_TOKENS][DP], k_s[LS_TOKENS][DP], v_s[LS_TOKENS][32];
    const int tile = blockIdx.x, h = blockIdx.y, seq = blockIdx.z, tid = threadIdx.x, part = tid & 3, vc = tid >> 2;
    const int col = tile * 32 + vc;
    const float decay = p.decay[h];
    pdl_wait();
    const int row0 = p.seq_start[seq], n = p.seq_start[seq + 1] - row0;
    if (n <= 0) return;  // (a sequence of the step's padding: its slot is someone else's)
    float *state = p.state + ((long long)p.seq_slot[seq] * p.n_heads + h) * p.dim * p.vdim;
    float s[DPT];
#pragma unroll
    for (int i = 0; i < DPT; i++) {
        const int d = i * 4 + part;
        s[i] = d < p.dim && col < p.vdim ? state[(long long)d * p.vdim + col] : 0.0f;
    }
    const T *proj = (const T *)p.proj;
    for (int c0 = 0; c0 < n; c0 += LS_TOKENS) {
        const int cnt = n - c0 < LS_TOKENS ? n - c0 : LS_TOKENS;
        __syncthreads();
        for (int e = tid; e < LS_TOKENS * DP; e += 128) {
            const int tok = e / DP, d = e - tok * DP;
            float q = 0.0f, k = 0.0f;
            if (tok < cnt && d < p.dim) {
                const T *r = proj + (long long)(row0 + c0 + tok) * p.ld + (long long)h * p.dim + d;
                q = silu_exact(to_float(r[p.q_at])), k = silu_exact(to_float(r[p.k_at]));
            }
            q_s[tok][d] = q, k_s[tok][d] = k;
        }
        for (int e = tid; e < LS_TOKENS * 32; e += 128) {
            const int tok = e >> 5, c = tile * 32 + (e & 31);
            v_s[tok][e & 31] = tok < cnt && c < p.vdim
                ? silu_exact(to_float(proj[(long long)(row0 + c0 + tok) * p.ld + p.v_at + (long long)h * p.vdim + c])) : 0.0f;
        }
        __syncthreads();
        for (int tok = 0; tok < cnt; tok++) {
            const float v = v_s[tok][vc];
            float o = 0.0f;
#pragma unroll
            for (int i = 0; i < DPT; i++) {
                s[i] = fmaf(decay, s[i], k_s[tok][i * 4 + part] * v);
                o = fmaf(s[i], q_s[tok][i * 4 + part], o);
            }
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            if (part == 0 && col < p.vdim)
                p.out[(long long)(row0 + c0 + tok) * p.n_heads * p.vdim + (long long)h * p.vdim + col] = o;
        }
    }
#pragma unroll
    for (int i = 0; i < DPT; i++) {
        const int d = i * 4 + part;
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
    dim3 grid((vdim + 31) / 32, n_heads, n_seqs);
    cudaStream_t s = (cudaStream_t)stream;
#define LS_LAUNCH(T)                                                                    \
    do {                                                                                \
        if (dim <= 16) abk_launch(lightning_scan_kernel<T, 4>, grid, dim3(128), 0, s, p);       \
        else if (dim <= 32) abk_launch(lightning_scan_kernel<T, 8>, grid, dim3(128), 0, s, p);  \
        else if (dim <= 64) abk_launch(lightning_scan_kernel<T, 16>, grid, dim3(128), 0, s, p); \
        else if (dim <= 128) abk_launch(lightning_scan_kernel<T, 32>, grid, dim3(128), 0, s, p);\
        else abk_launch(lightning_scan_kernel<T, 64>, grid, dim3(128), 0, s, p);                \
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
