// Time mixing with a decay per head, key channel and token ("wkv"): a recurrent mixer whose state is one [key, value]
// matrix per head and the token before,
//     o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t,    S_t = diag(w_t) S_(t-1) + k_t v_t^T,    w_t = exp(-exp(z_t + w0)),
// float32, zero at a sequence's start and carried from step to step in the sequence's slot.
//
//   token_shift       per token the blends m_s = x + (x' - x) * mu_s of a row with the row before it (the sequence's
//                     last row of the step before, kept in its slot, for a step's first row; zeros at the start), one
//                     plane of the output per s. In a step of one token a sequence it also leaves the new last row.
//   token_shift_keep  the last row of every sequence of a step of prompts, into its slot.
//   wkv_scan          a CTA walks one sequence's tokens for one head and 16 (32 for heads of up to 32 channels) value
//                     columns. Its threads are those columns x 4, 8 or 16 parts of the key channels, so a thread keeps 4
//                     to 16 state values in registers; the parts' partial outputs of a column meet by shuffles, four
//                     tokens at a time. Rows come 16 (8 for heads beyond 128 channels) tokens at a time: asked for a
//                     chunk ahead into registers, the decay made from its pre-activation on the way into shared memory,
//                     read from there as 16-byte pieces. A sequence that brings no token to the step is left alone.
#define ABK_DEFINE_ERROR
#include "common.cuh"

// ---------------------------------------------------------------- the blends with the token before
struct TokenShift {
    const void *x;       // [tokens][d], as stored
    float *last;         // [slots][d]: the last row a sequence brought
    const float *mu;     // [blends][d]
    void *out;           // [blends][plane]: blend s of row t at out + s * plane + t * d
    long long plane;
    int d, blends, update;
    const int *token_seq, *seq_start, *seq_slot;
};

// A thread has one column (a CTA 128 of them: blockIdx.y counts the runs of columns), so that no load waits for a store.
template <typename T> __global__ void __launch_bounds__(128) token_shift_kernel(TokenShift p) {
    const int t = blockIdx.x, j = blockIdx.y * 128 + threadIdx.x;
    pdl_wait();
    const int seq = p.token_seq[t];
    if (seq < 0 || j >= p.d) return;
    const bool first = t == p.seq_start[seq];
    float *last = p.last + (long long)p.seq_slot[seq] * p.d;
    const T *x = (const T *)p.x + (long long)t * p.d;
    T *out = (T *)p.out + (long long)t * p.d;
    const float h = to_float(x[j]);
    const float before = first ? last[j] : to_float(x[j - p.d]);
    const float diff = before - h;
    for (int s = 0; s < p.blends; s++) out[s * p.plane + j] = from_float<T>(fmaf(diff, __ldg(p.mu + (long long)s * p.d + j), h));
    if (p.update) last[j] = h;  // (a step of one token a sequence: this row is the sequence's only one)
}

// The same for bfloat16 rows of a multiple of 8 columns and up to 8 blends: a thread has 8 consecutive columns, read
// and written as 16-byte pieces, every load on its way before the first store.
template <int BLENDS> __global__ void __launch_bounds__(128) token_shift_bf16x8_kernel(TokenShift p) {
    const int t = blockIdx.x, j = (blockIdx.y * 128 + threadIdx.x) * 8;
    pdl_wait();
    const int seq = p.token_seq[t];
    if (seq < 0 || j >= p.d) return;
    const bool first = t == p.seq_start[seq];
    float *last = p.last + (long long)p.seq_slot[seq] * p.d + j;
    const __nv_bfloat16 *x = (const __nv_bfloat16 *)p.x + (long long)t * p.d + j;
    const uint4 raw = *(const uint4 *)x;
    float h[8], before[8];
    const uint32_t in[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const float2 f = __bfloat1622float2(*(const __nv_bfloat162 *)&in[e]);
        h[2 * e] = f.x, h[2 * e + 1] = f.y;
    }
    if (first) {
        const float4 a = *(const float4 *)last, b = *(const float4 *)(last + 4);
        before[0] = a.x, before[1] = a.y, before[2] = a.z, before[3] = a.w, before[4] = b.x, before[5] = b.y, before[6] = b.z, before[7] = b.w;
    } else {
        const uint4 r = *(const uint4 *)(x - p.d);
        const uint32_t pw[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const float2 f = __bfloat1622float2(*(const __nv_bfloat162 *)&pw[e]);
            before[2 * e] = f.x, before[2 * e + 1] = f.y;
        }
    }
    float4 m[BLENDS][2];
#pragma unroll
    for (int s = 0; s < BLENDS; s++)
        if (s < p.blends) m[s][0] = __ldg((const float4 *)(p.mu + (long long)s * p.d + j)), m[s][1] = __ldg((const float4 *)(p.mu + (long long)s * p.d + j + 4));
    __nv_bfloat16 *out = (__nv_bfloat16 *)p.out + (long long)t * p.d + j;
#pragma unroll
    for (int s = 0; s < BLENDS; s++) {
        if (s >= p.blends) break;
        const float mu[8] = {m[s][0].x, m[s][0].y, m[s][0].z, m[s][0].w, m[s][1].x, m[s][1].y, m[s][1].z, m[s][1].w};
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const __nv_bfloat162 h2 = __floats2bfloat162_rn(fmaf(before[2 * e] - h[2 * e], mu[2 * e], h[2 * e]),
                                                            fmaf(before[2 * e + 1] - h[2 * e + 1], mu[2 * e + 1], h[2 * e + 1]));
            w[e] = *(const uint32_t *)&h2;
        }
        *(uint4 *)(out + s * p.plane) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    if (p.update) {
        *(float4 *)last = make_float4(h[0], h[1], h[2], h[3]);
        *(float4 *)(last + 4) = make_float4(h[4], h[5], h[6], h[7]);
    }
}

template <typename T>
__global__ void __launch_bounds__(128) token_shift_keep_kernel(const T *x, float *last, int d, const int *seq_start,
                                                               const int *seq_slot) {
    const int seq = blockIdx.x;
    pdl_wait();
    const int row0 = seq_start[seq], n = seq_start[seq + 1] - row0;
    if (n <= 0) return;
    const T *src = x + (long long)(row0 + n - 1) * d;
    float *dst = last + (long long)seq_slot[seq] * d;
    for (int j = threadIdx.x; j < d; j += 128) dst[j] = to_float(src[j]);
}

extern "C" int abk_token_shift(const void *x, int dtype, int n_tokens, int d, const float *mu, int blends, float *last, void *out,
                               long long plane, int update, const int *token_seq, const int *seq_start, const int *seq_slot,
                               void *stream) {
    if (n_tokens <= 0) return 0;
    if (blends < 1 || d < 1 || plane < (long long)n_tokens * d) ABK_REFUSE("token_shift: %d blends of %d columns", blends, d);
    TokenShift p;
    p.x = x, p.last = last, p.mu = mu, p.out = out, p.plane = plane, p.d = d, p.blends = blends, p.update = update;
    p.token_seq = token_seq, p.seq_start = seq_start, p.seq_slot = seq_slot;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == ABK_BF16 && d % 8 == 0 && blends <= 8 && plane % 8 == 0 && ((uintptr_t)x | (uintptr_t)out | (uintptr_t)mu | (uintptr_t)last) % 16 == 0)
        abk_launch(token_shift_bf16x8_kernel<8>, dim3(n_tokens, (d / 8 + 127) / 128), dim3(128), 0, s, p);
    else if (dtype == ABK_BF16) abk_launch(token_shift_kernel<__nv_bfloat16>, dim3(n_tokens, (d + 127) / 128), dim3(128), 0, s, p);
    else abk_launch(token_shift_kernel<float>, dim3(n_tokens, (d + 127) / 128), dim3(128), 0, s, p);
    return ABK_LAUNCH_RESULT();
}

extern "C" int abk_token_shift_keep(const void *x, int dtype, int d, float *last, const int *seq_start, const int *seq_slot,
                                    int n_seqs, void *stream) {
    if (n_seqs <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == ABK_BF16)
        abk_launch(token_shift_keep_kernel<__nv_bfloat16>, dim3(n_seqs), dim3(128), 0, s, (const __nv_bfloat16 *)x, last, d, seq_start, seq_slot);
    else
        abk_launch(token_shift_keep_kernel<float>, dim3(n_seqs), dim3(128), 0, s, (const float *)x, last, d, seq_start, seq_slot);
    return ABK_LAUNCH_RESULT();
}

// ---------------------------------------------------------------- the activation inside the decay's pair of matrices
// dst = tanh(src) over `cols` columns of n rows (rows of any pitch): src float32 (a product's sums) or as stored, dst as
// stored (the second product's input).
template <typename TS, typename T>
__global__ void __launch_bounds__(256) tanh_rows_kernel(const TS *src, long long lds, T *dst, long long ldd, int cols, long long total) {
    pdl_wait();
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= total) return;
    const long long t = i / cols;
    const int j = (int)(i - t * cols);
    dst[t * ldd + j] = from_float<T>(tanhf(to_float(src[t * lds + j])));
}

extern "C" int abk_tanh_rows(const void *src, long long lds, int src_dtype, void *dst, long long ldd, int dtype, int n, int cols,
                             void *stream) {
    const long long total = (long long)n * cols;
    if (total <= 0) return 0;
    const dim3 grid((unsigned)((total + 255) / 256));
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
    if (dtype == ABK_BF16 && src_dtype == ABK_BF16)
        abk_launch(tanh_rows_kernel<bf, bf>, grid, dim3(256), 0, s, (const bf *)src, lds, (bf *)dst, ldd, cols, total);
    else if (dtype == ABK_BF16)
        abk_launch(tanh_rows_kernel<float, bf>, grid, dim3(256), 0, s, (const float *)src, lds, (bf *)dst, ldd, cols, total);
    else if (src_dtype == ABK_F32)
        abk_launch(tanh_rows_kernel<float, float>, grid, dim3(256), 0, s, (const float *)src, lds, (float *)dst, ldd, cols, total);
    else
        ABK_REFUSE("tanh_rows: bfloat16 into float32 is not built");
    return ABK_LAUNCH_RESULT();
}

// ---------------------------------------------------------------- the recurrence
struct WkvScan {
    const void *proj;    // row t at proj + t * ld: r head h at r_at + h * dim, k at k_at + h * dim, v at v_at + h * dim
    long long ld;
    int r_at, k_at, v_at;
    int n_heads, dim;
    const float *pre;    // [tokens][heads * dim]: the decay's pre-activation z
    const float *w0;     // [heads * dim]
    const float *bonus;  // [heads * dim]
    float *state;        // [slots][heads][dim][dim] (key, value)
    float *out;          // [tokens][heads * dim]
    const int *seq_start, *seq_slot;
    // A step of prompts runs in segments of `chunk` tokens, all at once (blockIdx.z counts the step's segments, sequence
    // after sequence): phase 1 walks each segment from an empty state and leaves its sum and the product of its decays,
    // wkv_segment_prefix turns the sums into the states at the segments' starts (and leaves the last in the slot), phase 2
    // walks each segment again from its start state for the outputs. chunk 0 (phase 0): a CTA walks a whole sequence.
    int chunk, phase, n_seqs;
    float *sums;         // [segments][heads][dim][dim]
    float *prods;        // [segments][heads][dim]
};

// The segment blockIdx.z names: its sequence, its first row and its rows (0: none). Sequences are walked in order.
__device__ __forceinline__ void wkv_segment(const int *seq_start, int n_seqs, int chunk, int z, int &seq, int &row0, int &n) {
    n = 0;
    int first = 0;
    for (seq = 0; seq < n_seqs; seq++) {
        const int start = seq_start[seq], len = seq_start[seq + 1] - start, count = (len + chunk - 1) / chunk;
        if (z < first + count) {
            const int c = z - first;
            row0 = start + c * chunk, n = len - c * chunk < chunk ? len - c * chunk : chunk;
            return;
        }
        first += count;
    }
}

// N tokens of one thread's share: r, k, w point at the thread's channels of the first token (tokens `pitch` floats
// apart), v at its column's value (tokens `v_pitch` apart); the column's output goes to out if `writes`.
// SUMS: the state alone moves (a segment's own sum): no r, no output.
template <int DPT, int PARTS, int N, bool SUMS>
__device__ __forceinline__ void wkv_tokens(float *s, const float *u, const float *r, const float *k, const float *w, int pitch,
                                           const float *v, int v_pitch, bool writes, float *out, long long out_pitch) {
    if constexpr (SUMS) {
        float vv[N];
#pragma unroll
        for (int n = 0; n < N; n++) vv[n] = v[n * v_pitch];
#pragma unroll
        for (int i = 0; i < DPT / 4; i++) {
            float4 kk[N], ww[N];
#pragma unroll
            for (int n = 0; n < N; n++) kk[n] = *(const float4 *)(k + n * pitch + 4 * i), ww[n] = *(const float4 *)(w + n * pitch + 4 * i);
#pragma unroll
            for (int n = 0; n < N; n++) {
                s[4 * i] = fmaf(ww[n].x, s[4 * i], kk[n].x * vv[n]), s[4 * i + 1] = fmaf(ww[n].y, s[4 * i + 1], kk[n].y * vv[n]);
                s[4 * i + 2] = fmaf(ww[n].z, s[4 * i + 2], kk[n].z * vv[n]), s[4 * i + 3] = fmaf(ww[n].w, s[4 * i + 3], kk[n].w * vv[n]);
            }
        }
        return;
    }
    float vv[N], o[N];
#pragma unroll
    for (int n = 0; n < N; n++) vv[n] = v[n * v_pitch], o[n] = 0.0f;
#pragma unroll
    for (int i = 0; i < DPT / 4; i++) {
        float4 kk[N], rr[N], ww[N];
#pragma unroll
        for (int n = 0; n < N; n++) {
            kk[n] = *(const float4 *)(k + n * pitch + 4 * i), rr[n] = *(const float4 *)(r + n * pitch + 4 * i);
            ww[n] = *(const float4 *)(w + n * pitch + 4 * i);
        }
#pragma unroll
        for (int n = 0; n < N; n++) {
            const float a0 = kk[n].x * vv[n], a1 = kk[n].y * vv[n], a2 = kk[n].z * vv[n], a3 = kk[n].w * vv[n];
            o[n] = fmaf(rr[n].x, fmaf(u[4 * i], a0, s[4 * i]), o[n]);
            o[n] = fmaf(rr[n].y, fmaf(u[4 * i + 1], a1, s[4 * i + 1]), o[n]);
            o[n] = fmaf(rr[n].z, fmaf(u[4 * i + 2], a2, s[4 * i + 2]), o[n]);
            o[n] = fmaf(rr[n].w, fmaf(u[4 * i + 3], a3, s[4 * i + 3]), o[n]);
            s[4 * i] = fmaf(ww[n].x, s[4 * i], a0), s[4 * i + 1] = fmaf(ww[n].y, s[4 * i + 1], a1);
            s[4 * i + 2] = fmaf(ww[n].z, s[4 * i + 2], a2), s[4 * i + 3] = fmaf(ww[n].w, s[4 * i + 3], a3);
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

// DPT key channels a thread, PARTS threads a value column (DPT * PARTS >= dim); a CTA has COLS columns and stages TOK
// tokens at a time.
// The decay from its pre-activation: to the last bit where the model is float32; where the model's operands are bfloat16
// numbers, by the special-function unit (a few units in the last place of float32, in float32 arithmetic).
template <typename T> __device__ __forceinline__ float wkv_decay(float z) { return expf(-expf(z)); }
template <> __device__ __forceinline__ float wkv_decay<__nv_bfloat16>(float z) { return __expf(-__expf(z)); }

template <typename T, int DPT, int PARTS, int COLS, int TOK, bool SUMS>
__global__ void __launch_bounds__(PARTS * COLS, 2) wkv_scan_kernel(WkvScan p) {
    constexpr int DP = DPT * PARTS;             // key channels, padded
    constexpr int PITCH = PARTS * (DPT + 4);    // a token's channels in shared memory: a part's run, then 4 floats of
    constexpr int THREADS = PARTS * COLS;       // padding, so that the parts' 16-byte reads meet no bank twice
    constexpr int PER = TOK * DP / THREADS;     // elements of r (of k, of the decay) a thread stages a chunk
    constexpr int PER_V = (TOK * COLS + THREADS - 1) / THREADS;
    __shared__ __align__(16) float r_s[TOK][PITCH], k_s[TOK][PITCH], w_s[TOK][PITCH];
    __shared__ float v_s[TOK][COLS];
    const int tile = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, part = tid % PARTS, vc = tid / PARTS;
    const int col = tile * COLS + vc;
    float u[DPT];
#pragma unroll
    for (int i = 0; i < DPT; i++) {
        const int d = part * DPT + i;
        u[i] = d < p.dim ? p.bonus[(long long)h * p.dim + d] : 0.0f;
    }
    pdl_wait();
    int seq = blockIdx.z, row0, n;
    if (p.chunk > 0) wkv_segment(p.seq_start, p.n_seqs, p.chunk, blockIdx.z, seq, row0, n);
    else row0 = p.seq_start[seq], n = p.seq_start[seq + 1] - row0;
    if (n <= 0) return;  // (a sequence of the step's padding: its slot is someone else's)
    float *state = p.phase == 0 ? p.state + ((long long)p.seq_slot[seq] * p.n_heads + h) * p.dim * p.dim
                                : p.sums + ((long long)blockIdx.z * p.n_heads + h) * p.dim * p.dim;
    float s[DPT];
#pragma unroll
    for (int i = 0; i < DPT; i++) {
        const int d = part * DPT + i;
        s[i] = p.phase != 1 && d < p.dim && col < p.dim ? state[(long long)d * p.dim + col] : 0.0f;
    }
    float decayed = 1.0f;  // phase 1: the product of this thread's staged decays (one channel, its share of the tokens)
    const T *proj = (const T *)p.proj;
    const long long hk = (long long)p.n_heads * p.dim;
    // A chunk's rows are asked for a chunk ahead and kept as they come: nothing is done to a loaded value before the
    // chunk is staged (an instruction that needs it would hold the warp until the load is back), so the loads' way from
    // memory lies under the chunk before. A thread stages one channel (THREADS is a multiple of the padded channels).
    static_assert(THREADS % DP == 0, "a thread stages one channel");
    T rr[PER], rk[PER], rv[PER_V];
    float rz[PER];
    const int my_d = tid % DP, my_ch = h * p.dim + (my_d < p.dim ? my_d : 0);
    const float my_w0 = p.w0[my_ch];
    auto fetch = [&](int c0) {
        const int cnt = n - c0 < TOK ? n - c0 : TOK;
#pragma unroll
        for (int it = 0; it < PER; it++) {
            // (every load is made, from a place that exists, and dropped where it is not wanted: loads that hang on no
            // branch are all in flight together)
            if (it * THREADS >= cnt * DP) break;  // (the same for every thread: the chunk has no such token)
            const int tok = (tid + it * THREADS) / DP;
            const long long row = row0 + c0 + (tok < cnt ? tok : cnt - 1);
            const T *r = proj + row * p.ld + my_ch;
            if (!SUMS) rr[it] = r[p.r_at];
            rk[it] = r[p.k_at], rz[it] = p.pre[row * hk + my_ch];
        }
#pragma unroll
        for (int it = 0; it < PER_V; it++) {
            if (it * THREADS >= cnt * COLS) break;
            const int e = tid + it * THREADS, tok = e / COLS, c = tile * COLS + e % COLS;
            rv[it] = proj[(long long)(row0 + c0 + (tok < cnt ? tok : cnt - 1)) * p.ld + p.v_at + (long long)h * p.dim + (c < p.dim ? c : 0)];
        }
    };
    fetch(0);
    for (int c0 = 0; c0 < n; c0 += TOK) {
        const int cnt = n - c0 < TOK ? n - c0 : TOK;
        __syncthreads();  // the chunk before is done with
#pragma unroll
        for (int it = 0; it < PER; it++) {
            if (it * THREADS >= cnt * DP) break;
            const int tok = (tid + it * THREADS) / DP, at = (my_d / DPT) * (DPT + 4) + my_d % DPT;
            const bool in = tok < cnt && my_d < p.dim;
            const float w = wkv_decay<T>(rz[it] + my_w0);
            if (!SUMS) r_s[tok][at] = in ? to_float(rr[it]) : 0.0f;
            k_s[tok][at] = in ? to_float(rk[it]) : 0.0f, w_s[tok][at] = w;
            if (in) decayed *= w;
        }
#pragma unroll
        for (int it = 0; it < PER_V; it++) {
            const int e = tid + it * THREADS;
            if (e < cnt * COLS) v_s[e / COLS][e % COLS] = tile * COLS + e % COLS < p.dim ? to_float(rv[it]) : 0.0f;
        }
        __syncthreads();
        if (c0 + TOK < n) fetch(c0 + TOK);
        // four tokens at a time: their reads from shared memory and their shuffles overlap, and only the state's own
        // multiply-adds follow one another
        const int at = part * (DPT + 4);
        float *out = p.out + (long long)(row0 + c0) * hk + (long long)h * p.dim + col;
        const bool writes = part == 0 && col < p.dim && p.phase != 1;
        int tok = 0;
        for (; tok + 4 <= cnt; tok += 4)
            wkv_tokens<DPT, PARTS, 4, SUMS>(s, u, &r_s[tok][at], &k_s[tok][at], &w_s[tok][at], PITCH, &v_s[tok][vc], COLS, writes, out + tok * hk, hk);
        for (; tok < cnt; tok++)
            wkv_tokens<DPT, PARTS, 1, SUMS>(s, u, &r_s[tok][at], &k_s[tok][at], &w_s[tok][at], PITCH, &v_s[tok][vc], COLS, writes, out + tok * hk, hk);
    }
    if (p.phase == 2) return;  // (the states between segments are wkv_segment_prefix's)
#pragma unroll
    for (int i = 0; i < DPT; i++) {
        const int d = part * DPT + i;
        if (d < p.dim && col < p.dim) state[(long long)d * p.dim + col] = s[i];
    }
    if (p.phase == 1 && tile == 0) {
        // every thread staged the decays of one channel: the shares of a channel meet through shared memory
        __syncthreads();
        float *share = &r_s[0][0];
        share[tid] = decayed;
        __syncthreads();
        if (tid < DP && tid < p.dim) {
            float all = 1.0f;
            for (int o = tid; o < THREADS; o += DP) all *= share[o];
            p.prods[((long long)blockIdx.z * p.n_heads + h) * p.dim + tid] = all;
        }
    }
}

// The states at the segments' starts from the segments' own sums: along a sequence S <- prod * S + sum, the state before
// each segment left where its sum was, the last in the sequence's slot. A thread an element of the state; four segments'
// loads are on their way together.
__global__ void __launch_bounds__(256) wkv_segment_prefix_kernel(float *sums, const float *prods, float *state, const int *seq_start,
                                                                 const int *seq_slot, int n_heads, int dim, int chunk) {
    const int e = blockIdx.x * 256 + threadIdx.x, h = blockIdx.y, seq = blockIdx.z;
    pdl_wait();
    const int len = seq_start[seq + 1] - seq_start[seq];
    if (len <= 0 || e >= dim * dim) return;
    int first = 0;
    for (int q = 0; q < seq; q++) first += (seq_start[q + 1] - seq_start[q] + chunk - 1) / chunk;
    const int count = (len + chunk - 1) / chunk, d = e / dim;
    float *slot = state + ((long long)seq_slot[seq] * n_heads + h) * dim * dim + e;
    float S = *slot;
    for (int c0 = 0; c0 < count; c0 += 4) {
        float u[4], pr[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const long long at = (long long)(first + (c0 + i < count ? c0 + i : count - 1)) * n_heads + h;
            u[i] = sums[at * dim * dim + e], pr[i] = prods[at * dim + d];
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if (c0 + i >= count) break;
            sums[((long long)(first + c0 + i) * n_heads + h) * dim * dim + e] = S;
            S = fmaf(pr[i], S, u[i]);
        }
    }
    *slot = S;
}

extern "C" int abk_wkv_scan(const void *proj, long long ld, int dtype, int r_at, int k_at, int v_at, int n_heads, int dim,
                            const float *pre, const float *w0, const float *bonus, float *state, float *out,
                            const int *seq_start, const int *seq_slot, int n_seqs, int chunk, int segments, float *sums,
                            float *prods, void *stream) {
    if (n_seqs <= 0) return 0;
    if (dim < 1 || dim > 256) ABK_REFUSE("wkv_scan: %d key channels a head are not 1 to 256", dim);
    if (n_heads < 1 || n_heads > 65535 || n_seqs > 65535) ABK_REFUSE("wkv_scan: %d heads, %d sequences", n_heads, n_seqs);
    WkvScan p;
    p.proj = proj, p.ld = ld, p.r_at = r_at, p.k_at = k_at, p.v_at = v_at, p.n_heads = n_heads, p.dim = dim;
    p.pre = pre, p.w0 = w0, p.bonus = bonus, p.state = state, p.out = out, p.seq_start = seq_start, p.seq_slot = seq_slot;
    p.chunk = chunk, p.phase = 0, p.n_seqs = n_seqs, p.sums = sums, p.prods = prods;
    if (chunk < 0 || (chunk > 0 && (segments < 1 || segments > 65535 || !sums || !prods)))
        ABK_REFUSE("wkv_scan: %d segments of %d tokens", segments, chunk);
    cudaStream_t s = (cudaStream_t)stream;
    const int cols = dim <= 32 ? 32 : 16;  // value columns a CTA has
    dim3 grid((dim + cols - 1) / cols, n_heads, chunk > 0 ? segments : n_seqs);
#define WS_LAUNCH(T, SUMS)                                                                                  \
    do {                                                                                                    \
        if (dim <= 16) abk_launch(wkv_scan_kernel<T, 4, 4, 32, 16, SUMS>, grid, dim3(128), 0, s, p);        \
        else if (dim <= 32) abk_launch(wkv_scan_kernel<T, 8, 4, 32, 16, SUMS>, grid, dim3(128), 0, s, p);   \
        else if (dim <= 64) abk_launch(wkv_scan_kernel<T, 8, 8, 16, 16, SUMS>, grid, dim3(128), 0, s, p);   \
        else if (dim <= 128) abk_launch(wkv_scan_kernel<T, 8, 16, 16, 16, SUMS>, grid, dim3(256), 0, s, p); \
        else abk_launch(wkv_scan_kernel<T, 16, 16, 16, 8, SUMS>, grid, dim3(256), 0, s, p);                 \
    } while (0)
    if (chunk > 0) {  // the segments' sums, the states between them, the segments' outputs
        p.phase = 1;
        if (dtype == ABK_BF16) WS_LAUNCH(__nv_bfloat16, true);
        else WS_LAUNCH(float, true);
        int rc = ABK_LAUNCH_RESULT();
        if (rc) return rc;
        abk_launch(wkv_segment_prefix_kernel, dim3((dim * dim + 255) / 256, n_heads, n_seqs), dim3(256), 0, s, sums, prods, state,
                   seq_start, seq_slot, n_heads, dim, chunk);
        rc = ABK_LAUNCH_RESULT();
        if (rc) return rc;
        p.phase = 2;
    }
    if (dtype == ABK_BF16) WS_LAUNCH(__nv_bfloat16, false);
    else WS_LAUNCH(float, false);
#undef WS_LAUNCH
    return ABK_LAUNCH_RESULT();
}
