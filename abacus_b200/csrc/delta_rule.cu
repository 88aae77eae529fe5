// The gated delta rule with a decay per key channel, as a recurrent mixer: the short causal convolution in
// front of it, the recurrence over a per-sequence state, and the gated per-head norm behind it.
//
// Per head, with a state S [key, value] in float32 that starts at zero and is carried from token to token:
//     S <- diag(g) S;   e = b (v - S^T k);   S <- S + k e^T;   o = S^T q
// q and k are unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q also times key^-1/2; b = sigmoid(.) per head;
// g = exp(-exp(A) * softplus(a + bias)) per head and key channel. Everything that enters the recurrence is
// float32; q, k and v come from the convolution in the model's storage type.
//
// A value column of S never meets another: column j needs S[:, j], v_j and the token's q, k, g, b. So a thread
// keeps (a part of) one column in registers and walks the sequence's tokens in order, and a prompt of any length
// and a decode step are the same kernel. The state is stored [head, value, key], so a column is one contiguous run.
#define ABK_DEFINE_ERROR
#include "common.cuh"

#define CONV_MAX_TAPS 8

// ------------------------------------------------------------------ short convolution + SiLU
// out[t, c] = silu(sum_j w[c, j] * in[position(t) - (taps - 1 - j), c]); inputs before the sequence's start are
// zero, inputs before this step's rows come from the slot's tail [taps - 1, channels] (the last inputs of the
// steps before). in: the first `channels` columns of rows of `ld` elements.
struct ShortConv {
    const void *in;
    long long ld;
    void *out;          // [tokens, channels]
    const float *w;     // [channels, taps]
    const float *tail;  // [slots, taps - 1, channels]
    const int *token_seq, *token_pos, *seq_slot, *seq_pos0;
    int channels, taps, n_tokens;
};

template <typename T> __global__ void __launch_bounds__(128) short_conv_kernel(ShortConv p) {
    pdl_wait();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= p.channels) return;
    T *out = (T *)p.out + (long long)t * p.channels + c;
    const int seq = p.token_seq[t];
    if (seq < 0) {
        *out = from_float<T>(0.0f);
        return;
    }
    const int pos = p.token_pos[t], pos0 = p.seq_pos0[seq], taps = p.taps;
    const float *w = p.w + (long long)c * taps;
    const float *tail = p.tail + (long long)p.seq_slot[seq] * (taps - 1) * p.channels + c;
    float acc = 0.0f;
    for (int j = 0; j < taps; j++) {
        const int back = taps - 1 - j, at = pos - back;
        float v = 0.0f;
        if (at >= pos0) v = to_float(((const T *)p.in)[(long long)(t - back) * p.ld + c]);
        else if (at >= 0) v = tail[(long long)(at - (pos0 - (taps - 1))) * p.channels];
        acc = fmaf(w[j], v, acc);
    }
    *out = from_float<T>(acc / (1.0f + expf(-acc)));
}

// The same with VEC channels a thread (16 bytes of the storage type), for channel counts and row pitches that are
// multiples of VEC with everything 16-byte aligned; a block has CONV_TOKENS tokens, its weights read once.
#define CONV_TOKENS 4
template <typename T, int VEC> struct ConvVector;
template <> struct ConvVector<__nv_bfloat16, 8> {
    static __device__ __forceinline__ void load(const __nv_bfloat16 *p, float *v) {
        const uint4 raw = *(const uint4 *)p;
        const __nv_bfloat162 *h = (const __nv_bfloat162 *)&raw;
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const float2 f = __bfloat1622float2(h[u]);
            v[2 * u] = f.x, v[2 * u + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16 *p, const float *v) {
        uint4 raw;
        __nv_bfloat162 *h = (__nv_bfloat162 *)&raw;
#pragma unroll
        for (int u = 0; u < 4; u++) h[u] = __floats2bfloat162_rn(v[2 * u], v[2 * u + 1]);
        *(uint4 *)p = raw;
    }
};
template <> struct ConvVector<float, 4> {
    static __device__ __forceinline__ void load(const float *p, float *v) {
        const float4 f = *(const float4 *)p;
        v[0] = f.x, v[1] = f.y, v[2] = f.z, v[3] = f.w;
    }
    static __device__ __forceinline__ void store(float *p, const float *v) { *(float4 *)p = make_float4(v[0], v[1], v[2], v[3]); }
};

template <typename T, int VEC> __global__ void __launch_bounds__(128) short_conv_vec_kernel(ShortConv p) {
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * VEC, taps = p.taps;
    float w[VEC][CONV_MAX_TAPS];
    if (c < p.channels) {
#pragma unroll
        for (int u = 0; u < VEC; u++)
#pragma unroll
            for (int j = 0; j < CONV_MAX_TAPS; j++) w[u][j] = j < taps ? p.w[(long long)(c + u) * taps + j] : 0.0f;  // weights: ahead of the wait
    }
    pdl_wait();
    if (c >= p.channels) return;
    for (int t = blockIdx.x * CONV_TOKENS; t < min(p.n_tokens, (blockIdx.x + 1) * CONV_TOKENS); t++) {
        T *out = (T *)p.out + (long long)t * p.channels + c;
        const int seq = p.token_seq[t];
        float acc[VEC];
#pragma unroll
        for (int u = 0; u < VEC; u++) acc[u] = 0.0f;
        if (seq >= 0) {
            const int pos = p.token_pos[t], pos0 = p.seq_pos0[seq];
            const float *tail = p.tail + (long long)p.seq_slot[seq] * (taps - 1) * p.channels + c;
#pragma unroll
            for (int j = 0; j < CONV_MAX_TAPS; j++) {
                if (j < taps) {
                    const int back = taps - 1 - j, at = pos - back;
                    float v[VEC];
                    if (at >= pos0) ConvVector<T, VEC>::load((const T *)p.in + (long long)(t - back) * p.ld + c, v);
                    else if (at >= 0) {
#pragma unroll
                        for (int u = 0; u < VEC; u++) v[u] = tail[(long long)(at - (pos0 - (taps - 1))) * p.channels + u];
                    } else {
#pragma unroll
                        for (int u = 0; u < VEC; u++) v[u] = 0.0f;
                    }
#pragma unroll
                    for (int u = 0; u < VEC; u++) acc[u] = fmaf(w[u][j], v[u], acc[u]);
                }
            }
#pragma unroll
            for (int u = 0; u < VEC; u++) acc[u] = acc[u] / (1.0f + expf(-acc[u]));
        }
        ConvVector<T, VEC>::store(out, acc);
    }
}

extern "C" int abk_short_conv(const void *in, long long ld, void *out, int dtype, const float *w, const float *tail,
                              const int *token_seq, const int *token_pos, const int *seq_slot, const int *seq_pos0,
                              int n_tokens, int channels, int taps, void *stream) {
    if (n_tokens <= 0 || channels <= 0) return 0;
    if (taps < 1 || taps > CONV_MAX_TAPS) ABK_REFUSE("short convolution: %d taps, the kernel takes 1 to %d", taps, CONV_MAX_TAPS);
    ShortConv p;
    p.in = in, p.ld = ld, p.out = out, p.w = w, p.tail = tail, p.token_seq = token_seq, p.token_pos = token_pos;
    p.seq_slot = seq_slot, p.seq_pos0 = seq_pos0, p.channels = channels, p.taps = taps, p.n_tokens = n_tokens;
    dim3 grid(n_tokens, (channels + 127) / 128);
    if (grid.y > 65535) ABK_REFUSE("short convolution: %d channels are more than a grid takes", channels);
    cudaStream_t s = (cudaStream_t)stream;
    const int vec = dtype == ABK_BF16 ? 8 : 4;
    if (channels % vec == 0 && ld % vec == 0 && !(((uintptr_t)in | (uintptr_t)out) & 15)) {
        dim3 tiles((n_tokens + CONV_TOKENS - 1) / CONV_TOKENS, (channels / vec + 127) / 128);
        if (dtype == ABK_BF16) abk_launch(short_conv_vec_kernel<__nv_bfloat16, 8>, tiles, dim3(128), 0, s, p);
        else abk_launch(short_conv_vec_kernel<float, 4>, tiles, dim3(128), 0, s, p);
        return ABK_LAUNCH_RESULT();
    }
    if (dtype == ABK_BF16) abk_launch(short_conv_kernel<__nv_bfloat16>, grid, dim3(128), 0, s, p);
    else abk_launch(short_conv_kernel<float>, grid, dim3(128), 0, s, p);
    return ABK_LAUNCH_RESULT();
}

// The tails after the step: for every sequence and channel the last taps - 1 inputs, from this step's rows and,
// where the step brought fewer, from the old tail moved up. One thread reads all it needs before it writes.
template <typename T>
__global__ void short_conv_tail_kernel(const T *in, long long ld, float *tail, const int *seq_start, const int *seq_slot,
                                       const int *seq_pos0, int n_seqs, int channels, int taps) {
    pdl_wait();
    const int i = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels || i >= n_seqs) return;
    const int row0 = seq_start[i], n = seq_start[i + 1] - row0;
    if (n <= 0) return;
    float *mine = tail + (long long)seq_slot[i] * (taps - 1) * channels + c;
    float keep[CONV_MAX_TAPS];
    for (int a = 0; a < taps - 1; a++) {
        const int back = taps - 1 - a;  // this place holds the input `back` tokens before the next one
        if (back <= n) keep[a] = to_float(in[(long long)(row0 + n - back) * ld + c]);
        else keep[a] = seq_pos0[i] + n - back >= 0 ? mine[(long long)(a + n) * channels] : 0.0f;
    }
    for (int a = 0; a < taps - 1; a++) mine[(long long)a * channels] = keep[a];
}

extern "C" int abk_short_conv_tail(const void *in, long long ld, int dtype, float *tail, const int *seq_start,
                                   const int *seq_slot, const int *seq_pos0, int n_seqs, int channels, int taps,
                                   void *stream) {
    if (n_seqs <= 0 || channels <= 0 || taps <= 1) return 0;
    if (taps > CONV_MAX_TAPS) ABK_REFUSE("short convolution: %d taps, the kernel takes 1 to %d", taps, CONV_MAX_TAPS);
    if (n_seqs > 65535) ABK_REFUSE("short convolution: %d sequences are more than a grid takes", n_seqs);
    dim3 grid((channels + 127) / 128, n_seqs);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == ABK_BF16)
        abk_launch(short_conv_tail_kernel<__nv_bfloat16>, grid, dim3(128), 0, s, (const __nv_bfloat16 *)in, ld, tail,
                   seq_start, seq_slot, seq_pos0, n_seqs, channels, taps);
    else
        abk_launch(short_conv_tail_kernel<float>, grid, dim3(128), 0, s, (const float *)in, ld, tail, seq_start, seq_slot,
                   seq_pos0, n_seqs, channels, taps);
    return ABK_LAUNCH_RESULT();
}

// ------------------------------------------------------------------ the recurrence
// A thread keeps KR key channels of one value column in registers (KR = 32, 64 or 128: all of a column where the
// key size allows, else the column's channels are dealt to 2, 4 or 8 neighbouring lanes that meet by shuffles), so
// the lanes of a warp are different columns and read a token's q, k and g from shared memory at one address (a
// broadcast). A block has 128 / lanes-per-column columns of one (sequence, head); a chunk of 16 tokens is prepared
// together (unit vectors, decays, write strengths: a warp a token), then walked in order. The state comes in and
// goes out through shared memory, so that global memory is read and written in whole lines.
#define SCAN_CHUNK 16   // tokens prepared together
#define SCAN_THREADS 128

struct DeltaScan {
    const void *qkv;        // [tokens, ld_qkv]: q heads (kv_heads x key), k heads, v heads (heads x value), after the convolution
    long long ld_qkv;
    const float *decay_in;  // [tokens, heads * key]: a, before bias and softplus
    const void *beta_in;    // row t, head h at beta_in[t * ld_beta + h], before the sigmoid
    long long ld_beta;
    const float *a_log;     // [heads]
    const float *dt_bias;   // [heads * key]
    float *state;           // [slots, heads, value, key]
    float *out;             // [tokens, heads * value]
    const int *seq_start, *seq_slot;
    int heads, kv_heads, key, value;
    int parts;              // lanes to a column: 1, 2, 4 or 8; parts * KR >= key
    float q_scale;          // key^-1/2
};

__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

template <typename T, int KR> __global__ void __launch_bounds__(SCAN_THREADS) delta_scan_kernel(DeltaScan p) {
    extern __shared__ float smem[];
    const int parts = p.parts, kp = parts * KR;         // padded key size
    const int cols = SCAN_THREADS / parts;              // columns of this block
    float *k_s = smem;                                  // [chunk][kp]
    float *q_s = k_s + SCAN_CHUNK * kp;
    float *g_s = q_s + SCAN_CHUNK * kp;
    float *v_s = g_s + SCAN_CHUNK * kp;                 // [chunk][cols]
    float *b_s = v_s + SCAN_CHUNK * cols;               // [chunk]
    float *stage = b_s + SCAN_CHUNK;                    // [warps][32 * 33]: 32 floats of each lane, a line at a time
    const int seq = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31, n_warps = SCAN_THREADS / 32;
    const int col = blockIdx.z * cols + tid / parts, part = tid % parts;
    const int K = p.key, V = p.value;
    const int kvh = h / (p.heads / p.kv_heads);
    const float decay_rate = expf(p.a_log[h]);  // a weight: ahead of the wait
    pdl_wait();
    const int row0 = p.seq_start[seq], n = p.seq_start[seq + 1] - row0;
    if (n <= 0) return;
    const bool live = col < V;
    float *head_state = p.state + ((long long)p.seq_slot[seq] * p.heads + h) * V * K;
    float *mine_stage = stage + warp * 32 * 33;
    // lane j of this warp owns channels [part_j * KR, + KR) of column col_j
    const int warp_col0 = blockIdx.z * cols + (warp * 32) / parts;
    float S[KR];
#pragma unroll
    for (int c = 0; c < KR / 32; c++) {
        for (int j = 0; j < 32; j++) {
            const int cj = warp_col0 + j / parts, ch = (j % parts) * KR + c * 32 + lane;
            mine_stage[j * 33 + lane] = cj < V && ch < K ? head_state[(long long)cj * K + ch] : 0.0f;
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 32; i++) S[c * 32 + i] = mine_stage[lane * 33 + i];
        __syncwarp();
    }

    for (int base = 0; base < n; base += SCAN_CHUNK) {
        const int count = n - base < SCAN_CHUNK ? n - base : SCAN_CHUNK;
        __syncthreads();  // the chunk before is done with
        // a warp prepares a token: unit vectors, decays, the write strength
        for (int c = warp; c < count; c += n_warps) {
            const long long row = row0 + base + c;
            const T *qr = (const T *)p.qkv + row * p.ld_qkv + (long long)kvh * K;
            const T *kr = qr + (long long)p.kv_heads * K;
            float qq = 0.0f, kk = 0.0f;
            for (int i = lane; i < kp; i += 32) {
                float qv = i < K ? to_float(qr[i]) : 0.0f, kv = i < K ? to_float(kr[i]) : 0.0f;
                q_s[c * kp + i] = qv, k_s[c * kp + i] = kv;
                qq = fmaf(qv, qv, qq), kk = fmaf(kv, kv, kk);
                float g = 0.0f;
                if (i < K)
                    g = expf(-decay_rate * softplus_f(p.decay_in[row * p.heads * K + (long long)h * K + i] + p.dt_bias[h * K + i]));
                g_s[c * kp + i] = g;
            }
            qq = warp_sum(qq), kk = warp_sum(kk);
            const float qn = p.q_scale / sqrtf(qq + 1e-6f), kn = 1.0f / sqrtf(kk + 1e-6f);
            for (int i = lane; i < kp; i += 32) q_s[c * kp + i] *= qn, k_s[c * kp + i] *= kn;
            if (lane == 0) {
                float z = to_float(((const T *)p.beta_in)[row * p.ld_beta + h]);
                b_s[c] = 1.0f / (1.0f + expf(-z));
            }
        }
        for (int e = tid; e < count * cols; e += SCAN_THREADS) {
            const int c = e / cols, j = blockIdx.z * cols + e % cols;
            const T *vr = (const T *)p.qkv + (long long)(row0 + base + c) * p.ld_qkv + 2LL * p.kv_heads * K + (long long)h * V;
            v_s[e] = j < V ? to_float(vr[j]) : 0.0f;
        }
        __syncthreads();
        for (int c = 0; c < count; c++) {
            const float4 *k4 = (const float4 *)(k_s + c * kp + part * KR);
            const float4 *q4 = (const float4 *)(q_s + c * kp + part * KR);
            const float4 *g4 = (const float4 *)(g_s + c * kp + part * KR);
            float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
            for (int i = 0; i < KR / 4; i++) {
                const float4 g = g4[i], k = k4[i];
                S[4 * i] *= g.x, S[4 * i + 1] *= g.y, S[4 * i + 2] *= g.z, S[4 * i + 3] *= g.w;
                s0 = fmaf(S[4 * i], k.x, s0), s1 = fmaf(S[4 * i + 1], k.y, s1);
                s2 = fmaf(S[4 * i + 2], k.z, s2), s3 = fmaf(S[4 * i + 3], k.w, s3);
            }
            float seen = (s0 + s1) + (s2 + s3);
            for (int o = 1; o < parts; o <<= 1) seen += __shfl_xor_sync(0xffffffffu, seen, o);
            const float e = b_s[c] * (v_s[c * cols + tid / parts] - seen);
            s0 = s1 = s2 = s3 = 0.0f;
#pragma unroll
            for (int i = 0; i < KR / 4; i++) {
                const float4 k = k4[i], q = q4[i];
                S[4 * i] = fmaf(k.x, e, S[4 * i]), S[4 * i + 1] = fmaf(k.y, e, S[4 * i + 1]);
                S[4 * i + 2] = fmaf(k.z, e, S[4 * i + 2]), S[4 * i + 3] = fmaf(k.w, e, S[4 * i + 3]);
                s0 = fmaf(S[4 * i], q.x, s0), s1 = fmaf(S[4 * i + 1], q.y, s1);
                s2 = fmaf(S[4 * i + 2], q.z, s2), s3 = fmaf(S[4 * i + 3], q.w, s3);
            }
            float read = (s0 + s1) + (s2 + s3);
            for (int o = 1; o < parts; o <<= 1) read += __shfl_xor_sync(0xffffffffu, read, o);
            if (live && part == 0) p.out[(long long)(row0 + base + c) * p.heads * V + (long long)h * V + col] = read;
        }
    }
#pragma unroll
    for (int c = 0; c < KR / 32; c++) {
#pragma unroll
        for (int i = 0; i < 32; i++) mine_stage[lane * 33 + i] = S[c * 32 + i];
        __syncwarp();
        for (int j = 0; j < 32; j++) {
            const int cj = warp_col0 + j / parts, ch = (j % parts) * KR + c * 32 + lane;
            if (cj < V && ch < K) head_state[(long long)cj * K + ch] = mine_stage[j * 33 + lane];
        }
        __syncwarp();
    }
}

template <typename T, int KR>
static int delta_scan_launch(DeltaScan &p, int n_seqs, cudaStream_t s) {
    int parts = 1;
    while (parts * KR < p.key) parts *= 2;
    p.parts = parts;
    const int cols = SCAN_THREADS / parts;
    const size_t smem = (size_t)(3 * SCAN_CHUNK * parts * KR + SCAN_CHUNK * cols + SCAN_CHUNK + (SCAN_THREADS / 32) * 32 * 33) * 4;
    dim3 grid(n_seqs, p.heads, (p.value + cols - 1) / cols);
    if (smem > 48 * 1024) {
        cudaError_t e = abk_allow_shared_memory((const void *)delta_scan_kernel<T, KR>, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    abk_launch(delta_scan_kernel<T, KR>, grid, dim3(SCAN_THREADS), smem, s, p);
    return ABK_LAUNCH_RESULT();
}

extern "C" int abk_delta_scan(const void *qkv, long long ld_qkv, int dtype, const float *decay_in, const void *beta_in,
                              long long ld_beta, const float *a_log, const float *dt_bias, float *state, float *out,
                              const int *seq_start, const int *seq_slot, int n_seqs, int heads, int kv_heads, int key,
                              int value, void *stream) {
    if (n_seqs <= 0) return 0;
    if (key < 1 || key > 256) ABK_REFUSE("delta rule: key size %d, the kernel takes 1 to 256", key);
    if (kv_heads < 1 || heads % kv_heads) ABK_REFUSE("delta rule: %d heads do not divide into %d key heads", heads, kv_heads);
    if (heads > 65535 || value > 65535 * 16) ABK_REFUSE("delta rule: %d heads of %d values are more than a grid takes", heads, value);
    DeltaScan p;
    p.qkv = qkv, p.ld_qkv = ld_qkv, p.decay_in = decay_in, p.beta_in = beta_in, p.ld_beta = ld_beta, p.a_log = a_log;
    p.dt_bias = dt_bias, p.state = state, p.out = out, p.seq_start = seq_start, p.seq_slot = seq_slot;
    p.heads = heads, p.kv_heads = kv_heads, p.key = key, p.value = value;
    p.q_scale = 1.0f / sqrtf((float)key);
    cudaStream_t s = (cudaStream_t)stream;
    const bool bf = dtype == ABK_BF16;
    if (key <= 32) return bf ? delta_scan_launch<__nv_bfloat16, 32>(p, n_seqs, s) : delta_scan_launch<float, 32>(p, n_seqs, s);
    if (key <= 64) return bf ? delta_scan_launch<__nv_bfloat16, 64>(p, n_seqs, s) : delta_scan_launch<float, 64>(p, n_seqs, s);
    return bf ? delta_scan_launch<__nv_bfloat16, 128>(p, n_seqs, s) : delta_scan_launch<float, 128>(p, n_seqs, s);
}

// ------------------------------------------------------------------ gated per-head norm
// out[t, h, :] = o[t, h, :] / sqrt(mean(o^2) + eps) * w * sigmoid(gate[t, h, :]); one warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128) gated_head_norm_kernel(const float *o, const float *gate, const float *w, T *out,
                                                              long long n_heads_total, int value, float eps) {
    pdl_wait();
    const long long head = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (head >= n_heads_total) return;
    const float *src = o + head * value, *gs = gate + head * value;
    float ss = 0.0f;
    for (int j = lane; j < value; j += 32) ss = fmaf(src[j], src[j], ss);
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)value + eps);
    for (int j = lane; j < value; j += 32)
        out[head * value + j] = from_float<T>(src[j] * scale * w[j] * (1.0f / (1.0f + expf(-gs[j]))));
}

extern "C" int abk_gated_head_norm(const float *o, const float *gate, const float *w, void *out, int dtype, int n_tokens,
                                   int heads, int value, float eps, void *stream) {
    const long long total = (long long)n_tokens * heads;
    if (total <= 0) return 0;
    const long long blocks = (total + 3) / 4;
    if (blocks > 0x7fffffffLL) ABK_REFUSE("gated norm: %lld heads are more than a grid takes", total);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == ABK_BF16)
        abk_launch(gated_head_norm_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(128), 0, s, o, gate, w,
                   (__nv_bfloat16 *)out, total, value, eps);
    else
        abk_launch(gated_head_norm_kernel<float>, dim3((unsigned)blocks), dim3(128), 0, s, o, gate, w, (float *)out, total,
                   value, eps);
    return ABK_LAUNCH_RESULT();
}
