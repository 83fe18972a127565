// The gated delta rule with a decay per key channel, as a recurrent mixer: the short causal convolution in
// front of it, the recurrence over a per-sequence state, and the gated per-head norm behind it.
//
// Per head, with a state S [key, value] in float32 that starts at zero and is carried from token to token:
//     S <- diag(g) S;   e = b (v - S^T k);   S <- S + k e^T;   o = S^T q
// q and k are unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q also times key^-1/2; b = sigmoid(.) per head;
// g = exp(-exp(A) * softplus(a + bias)) per head and key channel (or, per_head, one for all of a head's channels).
// The convolution may also stand alone, without its SiLU (plain). Everything that enters the recurrence is
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
    int tokens_per_block;  // of the vector kernel: 4 for long steps (its weights read once for four tokens), 1 for short ones
    float *new_tail;       // a step of one token a sequence: the kernel leaves the slot's new tail itself (the thread that
                           // read a channel's old tail writes its new one); null: short_conv_tail does it
    int plain;             // 1: the sum as it is, no SiLU behind it
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
    float *left = p.new_tail ? p.new_tail + (long long)p.seq_slot[seq] * (taps - 1) * p.channels + c : nullptr;
    for (int j = 0; j < taps; j++) {
        const int back = taps - 1 - j, at = pos - back;
        float v = 0.0f;
        if (at >= pos0) v = to_float(((const T *)p.in)[(long long)(t - back) * p.ld + c]);
        else if (at >= 0) v = tail[(long long)(at - (pos0 - (taps - 1))) * p.channels];
        if (left && j > 0) left[(long long)(j - 1) * p.channels] = v;  // the input `back` tokens ago is back + 1 ago next time
        acc = fmaf(w[j], v, acc);
    }
    *out = from_float<T>(p.plain ? acc : acc / (1.0f + expf(-acc)));
}

// The same with VEC channels a thread (16 bytes of the storage type), for channel counts and row pitches that are
// multiples of VEC with everything 16-byte aligned, for 2 to 4 taps; a block has CONV_TOKENS tokens, its weights
// read once, as vectors.
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

template <typename T, int VEC, int TAPS> __global__ void __launch_bounds__(128) short_conv_vec_kernel(ShortConv p) {
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
    constexpr int taps = TAPS;
    float w[VEC * TAPS];  // this thread's weights lie together: VEC channels of TAPS taps, a multiple of 16 bytes
    if (c < p.channels) {
#pragma unroll
        for (int i = 0; i < VEC * TAPS / 4; i++) {
            const float4 f = *(const float4 *)(p.w + (long long)c * TAPS + 4 * i);  // weights: ahead of the wait
            w[4 * i] = f.x, w[4 * i + 1] = f.y, w[4 * i + 2] = f.z, w[4 * i + 3] = f.w;
        }
    }
    pdl_wait();
    if (c >= p.channels) return;
    for (int t = blockIdx.x * p.tokens_per_block; t < min(p.n_tokens, (blockIdx.x + 1) * p.tokens_per_block); t++) {
        T *out = (T *)p.out + (long long)t * p.channels + c;
        const int seq = p.token_seq[t];
        float acc[VEC];
#pragma unroll
        for (int u = 0; u < VEC; u++) acc[u] = 0.0f;
        if (seq >= 0) {
            const int pos = p.token_pos[t], pos0 = p.seq_pos0[seq];
            const float *tail = p.tail + (long long)p.seq_slot[seq] * (taps - 1) * p.channels + c;
#pragma unroll
            for (int j = 0; j < TAPS; j++) {
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
                if (p.new_tail && j > 0) {  // the input `back` tokens ago is back + 1 ago next time
                    float *left = p.new_tail + (long long)p.seq_slot[seq] * (taps - 1) * p.channels + (long long)(j - 1) * p.channels + c;
#pragma unroll
                    for (int u = 0; u < VEC; u++) left[u] = v[u];
                }
#pragma unroll
                for (int u = 0; u < VEC; u++) acc[u] = fmaf(w[u * TAPS + j], v[u], acc[u]);
            }
#pragma unroll
            for (int u = 0; u < VEC; u++) acc[u] = p.plain ? acc[u] : acc[u] / (1.0f + expf(-acc[u]));
        }
        ConvVector<T, VEC>::store(out, acc);
    }
}

// update_tail: every sequence of the step brings one token, and the kernel leaves the slots' new tails itself.
extern "C" int abk_short_conv(const void *in, long long ld, void *out, int dtype, const float *w, float *tail,
                              const int *token_seq, const int *token_pos, const int *seq_slot, const int *seq_pos0,
                              int n_tokens, int channels, int taps, int update_tail, int plain, void *stream) {
    if (n_tokens <= 0 || channels <= 0) return 0;
    if (taps < 1 || taps > CONV_MAX_TAPS) ABK_REFUSE("short convolution: %d taps, the kernel takes 1 to %d", taps, CONV_MAX_TAPS);
    ShortConv p;
    p.in = in, p.ld = ld, p.out = out, p.w = w, p.tail = tail, p.token_seq = token_seq, p.token_pos = token_pos;
    p.seq_slot = seq_slot, p.seq_pos0 = seq_pos0, p.channels = channels, p.taps = taps, p.n_tokens = n_tokens;
    p.tokens_per_block = 1, p.plain = plain;
    p.new_tail = update_tail && taps > 1 ? tail : nullptr;
    dim3 grid(n_tokens, (channels + 127) / 128);
    if (grid.y > 65535) ABK_REFUSE("short convolution: %d channels are more than a grid takes", channels);
    cudaStream_t s = (cudaStream_t)stream;
    const int vec = dtype == ABK_BF16 ? 8 : 4;
    if (channels % vec == 0 && ld % vec == 0 && taps >= 2 && taps <= 4 && !(((uintptr_t)in | (uintptr_t)out | (uintptr_t)w) & 15)) {
        p.tokens_per_block = n_tokens >= 1024 ? CONV_TOKENS : 1;
        dim3 tiles((n_tokens + p.tokens_per_block - 1) / p.tokens_per_block, (channels / vec + 127) / 128);
#define CONV_LAUNCH(TAPS)                                                                                          \
    if (dtype == ABK_BF16) abk_launch(short_conv_vec_kernel<__nv_bfloat16, 8, TAPS>, tiles, dim3(128), 0, s, p); \
    else abk_launch(short_conv_vec_kernel<float, 4, TAPS>, tiles, dim3(128), 0, s, p);
        if (taps == 2) { CONV_LAUNCH(2) } else if (taps == 3) { CONV_LAUNCH(3) } else { CONV_LAUNCH(4) }
#undef CONV_LAUNCH
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
// Two kernels. The first prepares every (token, head) in parallel, a warp each: the unit vectors q and k (q times
// key^-1/2), the decays g, the value row and the write strength b, as one float32 record
//     [ k | q | g | v (vp) | b, 0, 0, 0 ]     vp = the value size padded to a multiple of 4
// in which k, q and g each lie as `parts` runs of 32 channels with 4 floats of padding behind each run (zeros
// beyond the key size; parts = 1, 2, 4 or 8).
// The second walks each sequence's tokens in order (see delta_scan_kernel): the records of 8 tokens come in by
// cp.async while the 8 before them are walked. The state comes in and goes out through shared memory, so that global
// memory is read and written in whole lines.
#define SCAN_ROWS 32    // key channels a thread keeps
#define SCAN_RUN 36     // a run of 32 channels with its padding
#define SCAN_CHUNK 8    // tokens in a stage

static inline int delta_parts(int key) { return key <= 32 ? 1 : key <= 64 ? 2 : key <= 128 ? 4 : 8; }
static inline int delta_record_floats(int key, int value) { return 3 * delta_parts(key) * SCAN_RUN + ((value + 3) & ~3) + 4; }

struct DeltaPrepare {
    const void *qkv;        // [tokens, ld_qkv]: q heads (kv_heads x key), k heads, v heads (heads x value), after the convolution
    long long ld_qkv;
    const void *decay_in;   // row t at decay_in + t * ld_decay, heads * key float32: a, before bias and softplus; with
    long long ld_decay;     // per_head: one a per head, `heads` of them in the storage type, and dt_bias [heads]
    int per_head;
    const void *beta_in;    // row t, head h at beta_in[t * ld_beta + h], before the sigmoid
    long long ld_beta;
    const float *a_log;     // [heads]
    const float *dt_bias;   // [heads * key]
    float *records;         // [tokens, heads, record]
    const int *token_seq;
    long long pairs;        // tokens * heads
    int heads, kv_heads, key, value, parts, record;
    float q_scale;          // key^-1/2
};

__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

template <typename T> __global__ void __launch_bounds__(128) delta_prepare_kernel(DeltaPrepare p) {
    const long long pair = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    pdl_wait();
    if (pair >= p.pairs) return;
    const long long row = pair / p.heads;
    const int h = (int)(pair - row * p.heads), K = p.key, V = p.value, region = p.parts * SCAN_RUN;
    float *rec = p.records + pair * p.record;
    if (p.token_seq[row] < 0) return;  // padding: its record is never read
    const int kvh = h / (p.heads / p.kv_heads);
    const T *qr = (const T *)p.qkv + row * p.ld_qkv + (long long)kvh * K;
    const T *kr = qr + (long long)p.kv_heads * K;
    const T *vr = (const T *)p.qkv + row * p.ld_qkv + 2LL * p.kv_heads * K + (long long)h * V;
    const float rate = expf(p.a_log[h]);
    float head_decay = 0.0f;  // one decay for all of the head's key channels
    if (p.per_head)
        head_decay = expf(-rate * softplus_f(to_float(((const T *)p.decay_in)[row * p.ld_decay + h]) + p.dt_bias[h]));
    const float *channel_decay = (const float *)p.decay_in + row * p.ld_decay + (long long)h * K;
    float qq = 0.0f, kk = 0.0f;
    for (int i = lane; i < K; i += 32) {
        const float qv = to_float(qr[i]), kv = to_float(kr[i]);
        qq = fmaf(qv, qv, qq), kk = fmaf(kv, kv, kk);
    }
    qq = warp_sum(qq), kk = warp_sum(kk);
    const float qn = p.q_scale / sqrtf(qq + 1e-6f), kn = 1.0f / sqrtf(kk + 1e-6f);
    for (int at = lane; at < region; at += 32) {  // a place within a region: run at / 36, channel at % 36 of it
        const int i = (at / SCAN_RUN) * SCAN_ROWS + at % SCAN_RUN;
        const bool real = at % SCAN_RUN < SCAN_ROWS && i < K;
        rec[at] = real ? to_float(kr[i]) * kn : 0.0f;
        rec[region + at] = real ? to_float(qr[i]) * qn : 0.0f;
        rec[2 * region + at] = !real ? 0.0f : p.per_head ? head_decay : expf(-rate * softplus_f(channel_decay[i] + p.dt_bias[h * K + i]));
    }
    const int vp = p.record - 3 * region - 4;
    for (int j = lane; j < vp; j += 32) rec[3 * region + j] = j < V ? to_float(vr[j]) : 0.0f;
    if (lane < 4) {
        const float z = to_float(((const T *)p.beta_in)[row * p.ld_beta + h]);
        rec[3 * region + vp + lane] = lane == 0 ? 1.0f / (1.0f + expf(-z)) : 0.0f;
    }
}

struct DeltaScan {
    const float *records;   // [tokens, heads, record]
    float *state;           // [slots, heads, value, key]
    float *out;             // [tokens, heads * value]
    const int *seq_start, *seq_slot;
    int heads, key, value, parts, record;
    int col_warps;          // warps side by side along the columns (each 64 columns): a block has parts * col_warps warps
};

__device__ __forceinline__ void scan_copy_16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

// A warp has one run of 32 key channels (its part) of 64 value columns, a lane two neighbouring columns: 64 state
// values in registers. All lanes of a warp read the token's k, q and g of the warp's run at one address. The sums
// over the key channels meet across the block's warps through shared memory, two barriers a token.
// MAX_THREADS: the most threads a block has (128, 256 or 512): the fewer, the more registers a thread may use.
template <int MAX_THREADS> __global__ void __launch_bounds__(MAX_THREADS) delta_scan_kernel(DeltaScan p) {
    extern __shared__ __align__(16) float smem[];  // records [2][SCAN_CHUNK][R] (before and after the walk: the
                                                   // state's lines, [warps][32 * 33]), then the partial sums
    const int parts = p.parts, region = parts * SCAN_RUN, R = p.record, cw = p.col_warps;
    const int n_warps = parts * cw, n_threads = n_warps * 32;
    const int seq = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int part = warp % parts, col_warp = warp / parts;
    const int block_cols = cw * 64, col0 = blockIdx.z * block_cols;          // this block's columns
    const int local = col_warp * 64 + 2 * lane, col = col0 + local;          // this lane's two columns: col, col + 1
    const int K = p.key, V = p.value, vp = R - 3 * region - 4;
    size_t front = (size_t)2 * SCAN_CHUNK * R;
    if (front < (size_t)n_warps * 32 * 33) front = (size_t)n_warps * 32 * 33;
    float *sums = smem + ((front + 3) & ~(size_t)3);  // [2 (token parity)][2 (seen, read)][parts][block_cols]
    pdl_wait();
    const int row0 = p.seq_start[seq], n = p.seq_start[seq + 1] - row0;
    if (n <= 0) return;
    float *head_state = p.state + ((long long)p.seq_slot[seq] * p.heads + h) * V * K;
    float *mine_stage = smem + warp * 32 * 33;  // 32 floats of each of 32 columns, a line at a time
    float S0[SCAN_ROWS], S1[SCAN_ROWS];
#pragma unroll
    for (int half = 0; half < 2; half++) {  // the warp's even columns, then its odd ones
#pragma unroll 8
        for (int j = 0; j < 32; j++) {
            const int cj = col0 + col_warp * 64 + 2 * j + half, ch = part * SCAN_ROWS + lane;
            mine_stage[j * 33 + lane] = cj < V && ch < K ? head_state[(long long)cj * K + ch] : 0.0f;
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < SCAN_ROWS; i++) {
            if (half == 0) S0[i] = mine_stage[lane * 33 + i];
            else S1[i] = mine_stage[lane * 33 + i];
        }
        __syncwarp();
    }
    __syncthreads();  // the records come into the same memory

    const uint32_t chunk_s = (uint32_t)__cvta_generic_to_shared(smem);
    auto fetch = [&](int base, int stage_index) {  // the records of tokens [base, base + count) of this head
        const int count = n - base < SCAN_CHUNK ? n - base : SCAN_CHUNK;
        const int per = R / 4;
        for (int e = tid; e < count * per; e += n_threads) {
            const int c = e / per, q = e - c * per;
            scan_copy_16(chunk_s + ((stage_index * SCAN_CHUNK + c) * R + q * 4) * 4,
                         p.records + ((long long)(row0 + base + c) * p.heads + h) * R + q * 4);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch(0, 0);
    int token = 0;
    for (int base = 0, it = 0; base < n; base += SCAN_CHUNK, it++) {
        const int count = n - base < SCAN_CHUNK ? n - base : SCAN_CHUNK;
        if (base + SCAN_CHUNK < n) {  // the next tokens into the other stage (its readers passed the barrier below)
            fetch(base + SCAN_CHUNK, (it + 1) & 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float *records = smem + (it & 1) * SCAN_CHUNK * R;
        for (int c = 0; c < count; c++, token++) {
            const float *rec = records + c * R;
            const float4 *k4 = (const float4 *)(rec + part * SCAN_RUN);
            const float4 *q4 = (const float4 *)(rec + region + part * SCAN_RUN);
            const float4 *g4 = (const float4 *)(rec + 2 * region + part * SCAN_RUN);
            float *seen_s = sums + (size_t)(token & 1) * 2 * parts * block_cols, *read_s = seen_s + parts * block_cols;
            float a0 = 0.0f, a1 = 0.0f, b0 = 0.0f, b1 = 0.0f;
#pragma unroll
            for (int i = 0; i < SCAN_ROWS / 4; i++) {
                const float4 g = g4[i], k = k4[i];
                S0[4 * i] *= g.x, S0[4 * i + 1] *= g.y, S0[4 * i + 2] *= g.z, S0[4 * i + 3] *= g.w;
                S1[4 * i] *= g.x, S1[4 * i + 1] *= g.y, S1[4 * i + 2] *= g.z, S1[4 * i + 3] *= g.w;
                a0 = fmaf(S0[4 * i], k.x, a0), a1 = fmaf(S0[4 * i + 1], k.y, a1);
                a0 = fmaf(S0[4 * i + 2], k.z, a0), a1 = fmaf(S0[4 * i + 3], k.w, a1);
                b0 = fmaf(S1[4 * i], k.x, b0), b1 = fmaf(S1[4 * i + 1], k.y, b1);
                b0 = fmaf(S1[4 * i + 2], k.z, b0), b1 = fmaf(S1[4 * i + 3], k.w, b1);
            }
            *(float2 *)(seen_s + part * block_cols + local) = make_float2(a0 + a1, b0 + b1);
            __syncthreads();
            float seen0 = 0.0f, seen1 = 0.0f;
            for (int o = 0; o < parts; o++) {
                const float2 t = *(const float2 *)(seen_s + o * block_cols + local);
                seen0 += t.x, seen1 += t.y;
            }
            const float beta = rec[3 * region + vp];
            const float e0 = beta * (rec[3 * region + (col < V ? col : 0)] - seen0);
            const float e1 = beta * (rec[3 * region + (col + 1 < V ? col + 1 : 0)] - seen1);
            a0 = a1 = b0 = b1 = 0.0f;
#pragma unroll
            for (int i = 0; i < SCAN_ROWS / 4; i++) {
                const float4 k = k4[i], q = q4[i];
                S0[4 * i] = fmaf(k.x, e0, S0[4 * i]), S0[4 * i + 1] = fmaf(k.y, e0, S0[4 * i + 1]);
                S0[4 * i + 2] = fmaf(k.z, e0, S0[4 * i + 2]), S0[4 * i + 3] = fmaf(k.w, e0, S0[4 * i + 3]);
                S1[4 * i] = fmaf(k.x, e1, S1[4 * i]), S1[4 * i + 1] = fmaf(k.y, e1, S1[4 * i + 1]);
                S1[4 * i + 2] = fmaf(k.z, e1, S1[4 * i + 2]), S1[4 * i + 3] = fmaf(k.w, e1, S1[4 * i + 3]);
                a0 = fmaf(S0[4 * i], q.x, a0), a1 = fmaf(S0[4 * i + 1], q.y, a1);
                a0 = fmaf(S0[4 * i + 2], q.z, a0), a1 = fmaf(S0[4 * i + 3], q.w, a1);
                b0 = fmaf(S1[4 * i], q.x, b0), b1 = fmaf(S1[4 * i + 1], q.y, b1);
                b0 = fmaf(S1[4 * i + 2], q.z, b0), b1 = fmaf(S1[4 * i + 3], q.w, b1);
            }
            *(float2 *)(read_s + part * block_cols + local) = make_float2(a0 + a1, b0 + b1);
            __syncthreads();
            if (part == 0) {  // the warps of the first run add up what the token reads
                float r0 = 0.0f, r1 = 0.0f;
                for (int o = 0; o < parts; o++) {
                    const float2 t = *(const float2 *)(read_s + o * block_cols + local);
                    r0 += t.x, r1 += t.y;
                }
                float *dst = p.out + (long long)(row0 + base + c) * p.heads * V + (long long)h * V;
                if (col < V) dst[col] = r0;
                if (col + 1 < V) dst[col + 1] = r1;
            }
        }
        __syncthreads();  // the stage is filled again by the iteration after next (and, at the end, by the state)
    }
#pragma unroll
    for (int half = 0; half < 2; half++) {
#pragma unroll
        for (int i = 0; i < SCAN_ROWS; i++) mine_stage[lane * 33 + i] = half == 0 ? S0[i] : S1[i];
        __syncwarp();
#pragma unroll 8
        for (int j = 0; j < 32; j++) {
            const int cj = col0 + col_warp * 64 + 2 * j + half, ch = part * SCAN_ROWS + lane;
            if (cj < V && ch < K) head_state[(long long)cj * K + ch] = mine_stage[j * 33 + lane];
        }
        __syncwarp();
    }
}

// Floats of scratch memory the recurrence needs for n_tokens tokens (its records).
extern "C" long long abk_delta_scan_scratch(int n_tokens, int heads, int key, int value) {
    return (long long)n_tokens * heads * delta_record_floats(key, value);
}

extern "C" int abk_delta_scan(const void *qkv, long long ld_qkv, int dtype, const void *decay_in, long long ld_decay, int per_head, const void *beta_in,
                              long long ld_beta, const float *a_log, const float *dt_bias, float *state, float *out,
                              const int *token_seq, const int *seq_start, const int *seq_slot, int n_tokens, int n_seqs,
                              int heads, int kv_heads, int key, int value, float *records, long long records_floats,
                              void *stream) {
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (key < 1 || key > 256) ABK_REFUSE("delta rule: key size %d, the kernel takes 1 to 256", key);
    if (kv_heads < 1 || heads % kv_heads) ABK_REFUSE("delta rule: %d heads do not divide into %d key heads", heads, kv_heads);
    if (heads > 65535 || value > 65535 * 16) ABK_REFUSE("delta rule: %d heads of %d values are more than a grid takes", heads, value);
    const int parts = delta_parts(key), record = delta_record_floats(key, value);
    if ((long long)n_tokens * heads * record > records_floats || ((uintptr_t)records & 15))
        ABK_REFUSE("delta rule: the scratch memory holds %lld floats, the step needs %lld (16-byte aligned)", records_floats,
                   (long long)n_tokens * heads * record);
    // 64 columns a warp; two warps side by side where they fit a block and the step has (sequence, head) pairs enough
    // to fill the GPU without the halves of a head going to different SMs
    const int col_warps = parts <= 4 && value > 64 && (long long)n_seqs * heads * ((value + 63) / 64) > 2LL * abk_sm_count() ? 2 : 1;
    const int n_warps = parts * col_warps, block_cols = 64 * col_warps;
    size_t front = (size_t)2 * SCAN_CHUNK * record;
    if (front < (size_t)n_warps * 32 * 33) front = (size_t)n_warps * 32 * 33;
    const size_t smem = (((front + 3) & ~(size_t)3) + (size_t)4 * parts * block_cols) * 4;
    if (smem > 220 * 1024) ABK_REFUSE("delta rule: heads of %d x %d need more shared memory than an SM has", key, value);
    cudaStream_t s = (cudaStream_t)stream;
    DeltaPrepare q;
    q.qkv = qkv, q.ld_qkv = ld_qkv, q.decay_in = decay_in, q.ld_decay = ld_decay, q.per_head = per_head, q.beta_in = beta_in, q.ld_beta = ld_beta, q.a_log = a_log;
    q.dt_bias = dt_bias, q.records = records, q.token_seq = token_seq, q.pairs = (long long)n_tokens * heads;
    q.heads = heads, q.kv_heads = kv_heads, q.key = key, q.value = value, q.parts = parts, q.record = record;
    q.q_scale = 1.0f / sqrtf((float)key);
    const long long blocks = (q.pairs + 3) / 4;
    if (blocks > 0x7fffffffLL) ABK_REFUSE("delta rule: %lld (token, head) pairs are more than a grid takes", q.pairs);
    if (dtype == ABK_BF16) abk_launch(delta_prepare_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(128), 0, s, q);
    else abk_launch(delta_prepare_kernel<float>, dim3((unsigned)blocks), dim3(128), 0, s, q);
    int rc = ABK_LAUNCH_RESULT();
    if (rc) return rc;
    DeltaScan p;
    p.records = records, p.state = state, p.out = out, p.seq_start = seq_start, p.seq_slot = seq_slot;
    p.heads = heads, p.key = key, p.value = value, p.parts = parts, p.record = record;
    p.col_warps = col_warps;
    dim3 grid(n_seqs, heads, (value + block_cols - 1) / block_cols);
#define SCAN_LAUNCH(MAXT)                                                                                  \
    do {                                                                                                   \
        if (smem > 48 * 1024) {                                                                            \
            cudaError_t e = abk_allow_shared_memory((const void *)delta_scan_kernel<MAXT>, (int)smem);     \
            if (e != cudaSuccess) return (int)e;                                                           \
        }                                                                                                  \
        abk_launch(delta_scan_kernel<MAXT>, grid, dim3(n_warps * 32), smem, s, p);                         \
    } while (0)
    if (n_warps <= 4) SCAN_LAUNCH(128);
    else if (n_warps <= 8) SCAN_LAUNCH(256);
    else SCAN_LAUNCH(512);
#undef SCAN_LAUNCH
    return ABK_LAUNCH_RESULT();
}

// ------------------------------------------------------------------ one decay a head, prompts: in chunks
// With one decay g_t for all of a head's key channels the recurrence of a chunk of DC_TOKENS tokens that starts from S0
// unrolls, G_t the product of the chunk's decays up to t and r(t, s) = G_t / G_s:
//     u_t = b_t (v_t - G_t S0^T k_t - sum over s < t of r(t, s) (k_s . k_t) u_s)
//     o_t = G_t S0^T q_t + sum over s <= t of r(t, s) (k_s . q_t) u_s        S_end = G_end S0 + sum_s r(end, s) k_s u_s^T
// The first line is a triangular system (I + M) U = diag(b) (V - diag(G) K S0), M(t, s) = b_t r(t, s) (k_t . k_s) for
// s < t, whose matrix knows neither the state nor the values. delta_chunk_tables makes T = (I + M)^-1 diag(b) and
// Q(t, s) = r(t, s) (q_t . k_s) for every chunk and head side by side; delta_chunk_scan walks a sequence's chunks for one
// head and DC_VT value columns (the columns of a state do not meet) with four products a chunk:
//     [K; Q] S0,   U = T (V - diag(G) K S0),   O = diag(G) Q S0 + Q U,   S_end = G_end S0 + K^T diag(r(end, .)) U.
// Float32 throughout; the same numbers as token by token, summed in another order. A decay below e^-80 counts as e^-80.
#define DC_TOKENS 64
#define DC_VT 16
#define DC_P (DC_TOKENS + 1)

struct DeltaChunks {
    DeltaScan s;
    float *work;   // per (chunk, head): one table [64][64] (Q on and below the diagonal, T below its diagonal transposed
    int n_seqs, max_chunks;   // above it), the logarithms of G [64], T's diagonal [64] (the write strengths)
};
#define DC_WORK (DC_TOKENS * DC_TOKENS + 2 * DC_TOKENS)

__device__ __forceinline__ bool dc_locate(const DeltaChunks &p, int chunk, int &t0, int &nt) {
    for (int q = 0; q < p.n_seqs; q++) {
        const int first = p.s.seq_start[q], n = p.s.seq_start[q + 1] - first;
        const int chunks = (n + DC_TOKENS - 1) / DC_TOKENS;
        if (chunk < chunks) {
            t0 = first + chunk * DC_TOKENS, nt = min(DC_TOKENS, n - chunk * DC_TOKENS);
            return true;
        }
        chunk -= chunks;
    }
    return false;
}

// 16 bytes from global to shared memory, or 16 bytes of zeros.
__device__ __forceinline__ void dc_copy_16(float *dst, const float *src, bool real) {
    const int bytes = real ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(bytes) : "memory");
}

__global__ void __launch_bounds__(256) delta_chunk_tables_kernel(DeltaChunks p) {
    extern __shared__ __align__(16) float dc_smem[];
    const int h = blockIdx.y, parts = p.s.parts, region = parts * SCAN_RUN, RP = 2 * region + 4, vp = p.s.record - 3 * region - 4;
    float *kq = dc_smem;                      // [64][RP]: k's runs, then q's, as in the records (see delta_chunk_scan)
    float *m = kq + DC_TOKENS * RP;           // [64][65]: M, strictly below the diagonal
    float *x = m + DC_TOKENS * DC_P;          // [64][65]: T
    float *lg = x + DC_TOKENS * DC_P, *beta = lg + DC_TOKENS;
    pdl_wait();
    int t0, nt;
    if (!dc_locate(p, blockIdx.x, t0, nt)) return;
    const int row_pieces = 2 * region / 4;
    for (int e = threadIdx.x; e < DC_TOKENS * row_pieces; e += 256) {
        const int t = e / row_pieces, c = e - t * row_pieces;
        const float *rec = p.s.records + ((long long)(t0 + min(t, nt - 1)) * p.s.heads + h) * p.s.record;
        dc_copy_16(kq + t * RP + 4 * c, rec + 4 * c, t < nt);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    if (threadIdx.x < DC_TOKENS) {
        const float *rec = p.s.records + ((long long)(t0 + min((int)threadIdx.x, nt - 1)) * p.s.heads + h) * p.s.record;
        lg[threadIdx.x] = threadIdx.x < nt ? fmaxf(logf(rec[2 * region]), -80.0f) : 0.0f;
        beta[threadIdx.x] = threadIdx.x < nt ? rec[3 * region + vp] : 0.0f;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0) {
        float sum = 0.0f;
        for (int t = 0; t < DC_TOKENS; t++) sum += lg[t], lg[t] = sum;   // (beyond nt: the last real one's)
    }
    __syncthreads();
    float *work = p.work + ((long long)blockIdx.x * p.s.heads + h) * DC_WORK;
    // a thread: one row t and every fourth column s
    const int t = threadIdx.x >> 2, sg = threadIdx.x & 3;
    for (int j = 0; j < DC_TOKENS / 4; j++) {
        const int c = sg + 4 * j;
        float kk = 0.0f, qk = 0.0f;
        if (c <= t && t < nt) {
            const float *kt = kq + t * RP, *kc = kq + c * RP;
            for (int r = 0; r < parts; r++) {
#pragma unroll
                for (int i = r * SCAN_RUN; i < r * SCAN_RUN + SCAN_ROWS; i += 4) {
                    const float4 a = *(const float4 *)(kc + i), b = *(const float4 *)(kt + i), q = *(const float4 *)(kt + region + i);
                    kk = fmaf(b.w, a.w, fmaf(b.z, a.z, fmaf(b.y, a.y, fmaf(b.x, a.x, kk))));
                    qk = fmaf(q.w, a.w, fmaf(q.z, a.z, fmaf(q.y, a.y, fmaf(q.x, a.x, qk))));
                }
            }
        }
        const float r = c <= t && t < nt ? expf(lg[t] - lg[c]) : 0.0f;
        m[t * DC_P + c] = c < t ? beta[t] * r * kk : 0.0f;
        if (c <= t) work[t * DC_TOKENS + c] = r * qk;
    }
    __syncthreads();
    // (I + M) X = diag(b): a thread a column, down its rows
    if (threadIdx.x < DC_TOKENS) {
        const int j = threadIdx.x;
        for (int r = 0; r < DC_TOKENS; r++) {
            float v = r == j ? beta[j] : 0.0f;
            if (r > j) {
                float acc = 0.0f;
                for (int c = j; c < r; c++) acc = fmaf(m[r * DC_P + c], x[c * DC_P + j], acc);
                v = -acc;
            }
            x[r * DC_P + j] = r >= j ? v : 0.0f;
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < DC_TOKENS * DC_TOKENS; e += 256) {  // T below its diagonal, transposed, above the table's
        const int r = e / DC_TOKENS, c = e % DC_TOKENS;
        if (c > r) work[e] = x[c * DC_P + r];
    }
    if (threadIdx.x < DC_TOKENS) {
        work[DC_TOKENS * DC_TOKENS + threadIdx.x] = lg[threadIdx.x];
        work[DC_TOKENS * DC_TOKENS + DC_TOKENS + threadIdx.x] = beta[threadIdx.x];
    }
}

// The rows of k and q lie in shared memory as in their records: runs of 32 channels with 4 floats of padding (zeros
// beyond the key size), k's runs and then q's, a row every 2 * region + 4 floats; so a chunk comes in as 16-byte copies
// that are all in flight together. Channel c of run r is at r * SCAN_RUN + c; the state's columns lie the same way,
// [run][32][DC_VT], rows beyond the key size zero.
#define DC_TP (DC_TOKENS + 4)   // a row of T or Q in shared memory
__global__ void __launch_bounds__(256) delta_chunk_scan_kernel(DeltaChunks p) {
    extern __shared__ __align__(16) float dc_smem[];
    const int K = p.s.key, V = p.s.value, h = blockIdx.y, seq = blockIdx.x, v0 = blockIdx.z * DC_VT;
    const int parts = p.s.parts, region = parts * SCAN_RUN, RP = 2 * region + 4, vp = p.s.record - 3 * region - 4;
    float *st = dc_smem;                          // [parts * 32][DC_VT]: the state's columns
    float *rs = st + parts * SCAN_ROWS * DC_VT;   // [64][DC_VT]: V, then V - diag(G) K S0
    float *us = rs + DC_TOKENS * DC_VT;           // [64][DC_VT]: U
    float *os = us + DC_TOKENS * DC_VT;           // [64][DC_VT]: diag(G) Q S0
    float *tq = os + DC_TOKENS * DC_VT;           // [64][DC_TP]: Q on and below the diagonal, T transposed above it
    float *lg = tq + DC_TOKENS * DC_TP;           // [64], then T's diagonal [64]
    float *td = lg + DC_TOKENS;
    float *kq = td + DC_TOKENS;                   // [64][RP]: k's runs, then q's
    pdl_wait();
    const int first = p.s.seq_start[seq], n = p.s.seq_start[seq + 1] - first;
    if (n <= 0) return;  // the sequence brings no token: its state stays as it is
    int chunk = 0;
    for (int q = 0; q < seq; q++) chunk += (p.s.seq_start[q + 1] - p.s.seq_start[q] + DC_TOKENS - 1) / DC_TOKENS;
    float *state = p.s.state + ((long long)p.s.seq_slot[seq] * p.s.heads + h) * V * K;
    for (int e = threadIdx.x; e < parts * SCAN_ROWS * DC_VT; e += 256) {
        const int c = e / (parts * SCAN_ROWS), i = e - c * (parts * SCAN_ROWS);
        st[i * DC_VT + c] = v0 + c < V && i < K ? state[(long long)(v0 + c) * K + i] : 0.0f;
    }
    const int row_pieces = 2 * region / 4;
    for (int t0 = first; t0 < first + n; t0 += DC_TOKENS, chunk++) {
        const int nt = min(DC_TOKENS, first + n - t0);
        const float *work = p.work + ((long long)chunk * p.s.heads + h) * DC_WORK;
        __syncthreads();  // the chunk before has been read
        for (int e = threadIdx.x; e < DC_TOKENS * row_pieces; e += 256) {
            const int t = e / row_pieces, c = e - t * row_pieces;
            const float *rec = p.s.records + ((long long)(t0 + min(t, nt - 1)) * p.s.heads + h) * p.s.record;
            dc_copy_16(kq + t * RP + 4 * c, rec + 4 * c, t < nt);
        }
        for (int e = threadIdx.x; e < DC_TOKENS * (DC_TOKENS / 4); e += 256) {
            const int r = e / (DC_TOKENS / 4), c = e - r * (DC_TOKENS / 4);
            dc_copy_16(tq + r * DC_TP + 4 * c, work + r * DC_TOKENS + 4 * c, true);
        }
        if (threadIdx.x < 2 * DC_TOKENS / 4) dc_copy_16(lg + 4 * threadIdx.x, work + DC_TOKENS * DC_TOKENS + 4 * threadIdx.x, true);
        {   // the values' columns: a row is DC_VT / 4 pieces, zeros beyond the record's values and the chunk's tokens
            const int t = threadIdx.x >> 2, c = (threadIdx.x & 3) * 4;
            const float *rec = p.s.records + ((long long)(t0 + min(t, nt - 1)) * p.s.heads + h) * p.s.record;
            dc_copy_16(rs + t * DC_VT + c, rec + 3 * region + min(v0 + c, vp - 4), t < nt && v0 + c < vp);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        {   // [K; Q] S0: a thread one of the 128 rows and 8 columns
            const int row = threadIdx.x >> 1, cg = (threadIdx.x & 1) * 8, t = row & (DC_TOKENS - 1);
            const float *a = kq + t * RP + (row < DC_TOKENS ? 0 : region);
            float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
            for (int r = 0; r < parts; r++) {
                const float *ar = a + r * SCAN_RUN, *sr = st + r * SCAN_ROWS * DC_VT + cg;
#pragma unroll 8
                for (int i = 0; i < SCAN_ROWS; i++) {
                    const float w = ar[i];
                    const float4 s0 = *(const float4 *)(sr + i * DC_VT), s1 = *(const float4 *)(sr + i * DC_VT + 4);
                    acc[0] = fmaf(w, s0.x, acc[0]), acc[1] = fmaf(w, s0.y, acc[1]), acc[2] = fmaf(w, s0.z, acc[2]), acc[3] = fmaf(w, s0.w, acc[3]);
                    acc[4] = fmaf(w, s1.x, acc[4]), acc[5] = fmaf(w, s1.y, acc[5]), acc[6] = fmaf(w, s1.z, acc[6]), acc[7] = fmaf(w, s1.w, acc[7]);
                }
            }
            const float G = expf(lg[t]);
#pragma unroll
            for (int u = 0; u < 8; u++) {
                if (row < DC_TOKENS) rs[t * DC_VT + cg + u] -= G * acc[u];
                else os[t * DC_VT + cg + u] = G * acc[u];
            }
        }
        __syncthreads();
        const int t = threadIdx.x >> 2, c4 = (threadIdx.x & 3) * 4;   // a thread: one token and 4 columns
        {   // U = T R
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            for (int c = 0; c <= t; c++) {
                const float w = c < t ? tq[c * DC_TP + t] : td[t];
                const float4 r = *(const float4 *)(rs + c * DC_VT + c4);
                acc[0] = fmaf(w, r.x, acc[0]), acc[1] = fmaf(w, r.y, acc[1]), acc[2] = fmaf(w, r.z, acc[2]), acc[3] = fmaf(w, r.w, acc[3]);
            }
            *(float4 *)(us + t * DC_VT + c4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        }
        __syncthreads();
        {   // O = diag(G) Q S0 + Q U
            float4 o = *(const float4 *)(os + t * DC_VT + c4);
            for (int c = 0; c <= t; c++) {
                const float w = tq[t * DC_TP + c];
                const float4 u = *(const float4 *)(us + c * DC_VT + c4);
                o.x = fmaf(w, u.x, o.x), o.y = fmaf(w, u.y, o.y), o.z = fmaf(w, u.z, o.z), o.w = fmaf(w, u.w, o.w);
            }
            if (t < nt) {
                float *out = p.s.out + (long long)(t0 + t) * p.s.heads * V + (long long)h * V + v0 + c4;
                if (v0 + c4 < V) out[0] = o.x;
                if (v0 + c4 + 1 < V) out[1] = o.y;
                if (v0 + c4 + 2 < V) out[2] = o.z;
                if (v0 + c4 + 3 < V) out[3] = o.w;
            }
        }
        // S_end = G_end S0 + K^T diag(r(end, .)) U: a thread a key channel and 8 columns (its own elements of the state)
        const float lg_end = lg[nt - 1], G_end = expf(lg_end);
        for (int i = threadIdx.x >> 1; i < parts * SCAN_ROWS; i += 128) {
            const int cg = (threadIdx.x & 1) * 8, at = (i / SCAN_ROWS) * SCAN_RUN + i % SCAN_ROWS;
            float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
            for (int c = 0; c < nt; c++) {
                const float w = kq[c * RP + at] * expf(lg_end - lg[c]);
                const float4 u0 = *(const float4 *)(us + c * DC_VT + cg), u1 = *(const float4 *)(us + c * DC_VT + cg + 4);
                acc[0] = fmaf(w, u0.x, acc[0]), acc[1] = fmaf(w, u0.y, acc[1]), acc[2] = fmaf(w, u0.z, acc[2]), acc[3] = fmaf(w, u0.w, acc[3]);
                acc[4] = fmaf(w, u1.x, acc[4]), acc[5] = fmaf(w, u1.y, acc[5]), acc[6] = fmaf(w, u1.z, acc[6]), acc[7] = fmaf(w, u1.w, acc[7]);
            }
#pragma unroll
            for (int u = 0; u < 8; u++) st[i * DC_VT + cg + u] = fmaf(G_end, st[i * DC_VT + cg + u], acc[u]);
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < K * DC_VT; e += 256) {
        const int c = e / K, i = e - c * K;
        if (v0 + c < V) state[(long long)(v0 + c) * K + i] = st[i * DC_VT + c];
    }
}

// The delta rule with one decay a head over a step that brings prompts, in chunks of 64 tokens: the preparation of
// abk_delta_scan, then the chunks' tables side by side, then the sequences' chunks in order. work: float32 scratch of at
// least max_chunks * heads * (64 * 64 + 2 * 64), max_chunks >= ceil(tokens / 64) + sequences.
extern "C" int abk_delta_chunks(const void *qkv, long long ld_qkv, int dtype, const void *decay_in, long long ld_decay,
                                const void *beta_in, long long ld_beta, const float *a_log, const float *dt_bias, float *state,
                                float *out, const int *token_seq, const int *seq_start, const int *seq_slot, int n_tokens,
                                int n_seqs, int heads, int kv_heads, int key, int value, float *records,
                                long long records_floats, int max_chunks, float *work, long long work_floats, void *stream) {
    if (n_seqs <= 0 || n_tokens <= 0 || max_chunks <= 0) return 0;
    if (key < 1 || key > 256) ABK_REFUSE("delta rule: key size %d, the kernel takes 1 to 256", key);
    if (kv_heads < 1 || heads % kv_heads) ABK_REFUSE("delta rule: %d heads do not divide into %d key heads", heads, kv_heads);
    if (heads > 65535 || n_seqs > 65535 || value > 65535 * DC_VT) ABK_REFUSE("delta rule: %d heads of %d values, %d sequences are more than a grid takes", heads, value, n_seqs);
    const int parts = delta_parts(key), record = delta_record_floats(key, value);
    if ((long long)n_tokens * heads * record > records_floats || ((uintptr_t)records & 15))
        ABK_REFUSE("delta rule: the scratch memory holds %lld floats, the step needs %lld (16-byte aligned)", records_floats,
                   (long long)n_tokens * heads * record);
    if ((long long)max_chunks * heads * DC_WORK > work_floats || ((uintptr_t)work & 15))
        ABK_REFUSE("delta rule: the chunks' scratch memory holds %lld floats, the step needs %lld (16-byte aligned)", work_floats,
                   (long long)max_chunks * heads * DC_WORK);
    cudaStream_t s = (cudaStream_t)stream;
    DeltaPrepare q;
    q.qkv = qkv, q.ld_qkv = ld_qkv, q.decay_in = decay_in, q.ld_decay = ld_decay, q.per_head = 1, q.beta_in = beta_in, q.ld_beta = ld_beta, q.a_log = a_log;
    q.dt_bias = dt_bias, q.records = records, q.token_seq = token_seq, q.pairs = (long long)n_tokens * heads;
    q.heads = heads, q.kv_heads = kv_heads, q.key = key, q.value = value, q.parts = parts, q.record = record;
    q.q_scale = 1.0f / sqrtf((float)key);
    const long long blocks = (q.pairs + 3) / 4;
    if (blocks > 0x7fffffffLL) ABK_REFUSE("delta rule: %lld (token, head) pairs are more than a grid takes", q.pairs);
    if (dtype == ABK_BF16) abk_launch(delta_prepare_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(128), 0, s, q);
    else abk_launch(delta_prepare_kernel<float>, dim3((unsigned)blocks), dim3(128), 0, s, q);
    int rc = ABK_LAUNCH_RESULT();
    if (rc) return rc;
    DeltaChunks p;
    p.s.records = records, p.s.state = state, p.s.out = out, p.s.seq_start = seq_start, p.s.seq_slot = seq_slot;
    p.s.heads = heads, p.s.key = key, p.s.value = value, p.s.parts = parts, p.s.record = record, p.s.col_warps = 1;
    p.work = work, p.n_seqs = n_seqs, p.max_chunks = max_chunks;
    const size_t smem_t = (size_t)(DC_TOKENS * (2 * parts * SCAN_RUN + 4) + 2 * DC_TOKENS * DC_P + 2 * DC_TOKENS) * sizeof(float);
    const size_t smem_s = (size_t)(parts * SCAN_ROWS * DC_VT + 3 * DC_TOKENS * DC_VT + DC_TOKENS * DC_TP + 2 * DC_TOKENS +
                                   DC_TOKENS * (2 * parts * SCAN_RUN + 4)) * sizeof(float);
    // Two CTAs of the walk fit an SM (heads of 128 channels: 111 KB each), which a step of many sequences needs; a step
    // whose CTAs are fewer than the SMs asks for more than half an SM's shared memory instead, so that each CTA has an SM
    // to itself (measured, one prompt of 2,048 tokens, 64 CTAs: 3.03 ms a step of four layers against 3.37 when the
    // scheduler may pair them)
    size_t smem_walk = smem_s;
    if ((long long)n_seqs * heads * ((value + DC_VT - 1) / DC_VT) <= abk_sm_count() && smem_walk < 116 * 1024) smem_walk = 116 * 1024;
    cudaError_t e = abk_allow_shared_memory((const void *)delta_chunk_tables_kernel, (int)smem_t);
    if (e == cudaSuccess) e = abk_allow_shared_memory((const void *)delta_chunk_scan_kernel, (int)smem_walk);
    if (e != cudaSuccess) return (int)e;
    abk_launch(delta_chunk_tables_kernel, dim3(max_chunks, heads), dim3(256), smem_t, s, p);
    abk_launch(delta_chunk_scan_kernel, dim3(n_seqs, heads, (value + DC_VT - 1) / DC_VT), dim3(256), smem_walk, s, p);
    return ABK_LAUNCH_RESULT();
}

// ------------------------------------------------------------------ gated per-head norm
// out[t, h, :] = o[t, h, :] / sqrt(mean(o^2) + eps) * w * act(gate[t, h, :]); one warp per (token, head). A token's
// gates lie at gate + t * ld_gate, float32 or (TG) in the storage type. act: sigmoid, or (silu) z sigmoid(z). w: [value],
// shared by the heads, or (w_per_head) [heads * value].
template <typename T, typename TG>
__global__ void __launch_bounds__(128) gated_head_norm_kernel(const float *o, const TG *gate, long long ld_gate, int heads,
                                                              const float *w, T *out, long long n_heads_total, int value,
                                                              float eps, int silu, int w_per_head) {
    pdl_wait();
    const long long head = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (head >= n_heads_total) return;
    const float *src = o + head * value;
    const TG *gs = gate + (head / heads) * ld_gate + (head % heads) * value;
    if (w_per_head) w += (head % heads) * value;
    float ss = 0.0f;
    for (int j = lane; j < value; j += 32) ss = fmaf(src[j], src[j], ss);
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)value + eps);
    for (int j = lane; j < value; j += 32) {
        const float z = to_float(gs[j]), sg = 1.0f / (1.0f + expf(-z));
        out[head * value + j] = from_float<T>(src[j] * scale * w[j] * (silu ? z * sg : sg));
    }
}

extern "C" int abk_gated_head_norm(const float *o, const void *gate, long long ld_gate, int gate_stored, const float *w, void *out,
                                   int dtype, int n_tokens, int heads, int value, float eps, int silu, int w_per_head,
                                   void *stream) {
    const long long total = (long long)n_tokens * heads;
    if (total <= 0) return 0;
    const long long blocks = (total + 3) / 4;
    if (blocks > 0x7fffffffLL) ABK_REFUSE("gated norm: %lld heads are more than a grid takes", total);
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
    if (dtype == ABK_BF16 && gate_stored)
        abk_launch(gated_head_norm_kernel<bf, bf>, dim3((unsigned)blocks), dim3(128), 0, s, o, (const bf *)gate, ld_gate, heads, w,
                   (bf *)out, total, value, eps, silu, w_per_head);
    else if (dtype == ABK_BF16)
        abk_launch(gated_head_norm_kernel<bf, float>, dim3((unsigned)blocks), dim3(128), 0, s, o, (const float *)gate, ld_gate, heads, w,
                   (bf *)out, total, value, eps, silu, w_per_head);
    else
        abk_launch(gated_head_norm_kernel<float, float>, dim3((unsigned)blocks), dim3(128), 0, s, o, (const float *)gate, ld_gate, heads, w,
                   (float *)out, total, value, eps, silu, w_per_head);
    return ABK_LAUNCH_RESULT();
}
