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

template <typename T> __global__ void __launch_bounds__(128) token_shift_kernel(TokenShift p) {
    const int t = blockIdx.x;
    pdl_wait();
    const int seq = p.token_seq[t];
    if (seq < 0) return;
    const bool first = t == p.seq_start[seq];
    float *last = p.last + (long long)p.seq_slot[seq] * p.d;
    const T *x = (const T *)p.x + (long long)t * p.d;
    T *out = (T *)p.out + (long long)t * p.d;
    for (int j = threadIdx.x; j < p.d; j += 128) {
        const float h = to_float(x[j]);
        const float before = first ? last[j] : to_float(x[j - p.d]);
        const float diff = before - h;
        for (int s = 0; s < p.blends; s++) out[s * p.plane + j] = from_float<T>(fmaf(diff, p.mu[(long long)s * p.d + j], h));
        if (p.update) last[j] = h;  // (a step of one token a sequence: this row is the sequence's only one)
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
    if (dtype == ABK_BF16) abk_launch(token_shift_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(128), 0, s, p);
    else abk_launch(token_shift_kernel<float>, dim3(n_tokens), dim3(128), 0, s, p);
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
// dst = tanh(src): src float32 (the first product's sums), dst as stored (the second product's input).
template <typename T> __global__ void __launch_bounds__(256) tanh_rows_kernel(const float *src, T *dst, long long total) {
    pdl_wait();
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i < total) dst[i] = from_float<T>(tanhf(src[i]));
}

extern "C" int abk_tanh_rows(const float *src, void *dst, int dtype, long long total, void *stream) {
    if (total <= 0) return 0;
    const dim3 grid((unsigned)((total + 255) / 256));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == ABK_BF16) abk_launch(tanh_rows_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, src, (__nv_bfloat16 *)dst, total);
    else abk_launch(tanh_rows_kernel<float>, grid, dim3(256), 0, s, src, (float *)dst, total);
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
};

// N tokens of one thread's share: r, k, w point at the thread's channels of the first token (tokens `pitch` floats
// apart), v at its column's value (tokens `v_pitch` apart); the column's output goes to out if `writes`.
template <int DPT, int PARTS, int N>
__device__ __forceinline__ void wkv_tokens(float *s, const float *u, const float *r, const float *k, const float *w, int pitch,
                                           const float *v, int v_pitch, bool writes, float *out, long long out_pitch) {
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
template <typename T, int DPT, int PARTS, int COLS, int TOK>
__global__ void __launch_bounds__(PARTS * COLS, 2) wkv_scan_kernel(WkvScan p) {
    constexpr int DP = DPT * PARTS;             // key channels, padded
    constexpr int PITCH = PARTS * (DPT + 4);    // a token's channels in shared memory: a part's run, then 4 floats of
    constexpr int THREADS = PARTS * COLS;       // padding, so that the parts' 16-byte reads meet no bank twice
    constexpr int PER = TOK * DP / THREADS;     // elements of r (of k, of the decay) a thread stages a chunk
    constexpr int PER_V = (TOK * COLS + THREADS - 1) / THREADS;
    __shared__ __align__(16) float r_s[TOK][PITCH], k_s[TOK][PITCH], w_s[TOK][PITCH];
    __shared__ float v_s[TOK][COLS];
    const int tile = blockIdx.x, h = blockIdx.y, seq = blockIdx.z, tid = threadIdx.x, part = tid % PARTS, vc = tid / PARTS;
    const int col = tile * COLS + vc;
    float u[DPT];
#pragma unroll
    for (int i = 0; i < DPT; i++) {
        const int d = part * DPT + i;
        u[i] = d < p.dim ? p.bonus[(long long)h * p.dim + d] : 0.0f;
    }
    pdl_wait();
    const int row0 = p.seq_start[seq], n = p.seq_start[seq + 1] - row0;
    if (n <= 0) return;  // (a sequence of the step's padding: its slot is someone else's)
    float *state = p.state + ((long long)p.seq_slot[seq] * p.n_heads + h) * p.dim * p.dim;
    float s[DPT];
#pragma unroll
    for (int i = 0; i < DPT; i++) {
        const int d = part * DPT + i;
        s[i] = d < p.dim && col < p.dim ? state[(long long)d * p.dim + col] : 0.0f;
    }
    const T *proj = (const T *)p.proj;
    const long long hk = (long long)p.n_heads * p.dim;
    float rr[PER], rk[PER], rw[PER], rv[PER_V];
    auto fetch = [&](int c0) {
        const int cnt = n - c0 < TOK ? n - c0 : TOK;
#pragma unroll
        for (int it = 0; it < PER; it++) {
            // (every load is made, from a place that exists, and dropped where it is not wanted: loads that hang on no
            // branch are all in flight together)
            if (it * THREADS >= cnt * DP) break;  // (the same for every thread: the chunk has no such token)
            const int e = tid + it * THREADS, tok = e / DP, d = e % DP;
            const bool in = tok < cnt && d < p.dim;
            const long long row = row0 + c0 + (tok < cnt ? tok : cnt - 1);
            const int ch = h * p.dim + (d < p.dim ? d : 0);
            const T *r = proj + row * p.ld + ch;
            const float rv_ = to_float(r[p.r_at]), kv_ = to_float(r[p.k_at]);
            const float z = p.pre[row * hk + ch] + p.w0[ch];
            rr[it] = in ? rv_ : 0.0f, rk[it] = in ? kv_ : 0.0f, rw[it] = in ? z : 0.0f;
        }
#pragma unroll
        for (int it = 0; it < PER_V; it++) {
            if (it * THREADS >= cnt * COLS) break;
            const int e = tid + it * THREADS, tok = e / COLS, c = tile * COLS + e % COLS;
            const float v = to_float(proj[(long long)(row0 + c0 + (tok < cnt ? tok : cnt - 1)) * p.ld + p.v_at + (long long)h * p.dim +
                                          (c < p.dim ? c : 0)]);
            rv[it] = tok < cnt && c < p.dim ? v : 0.0f;
        }
    };
    fetch(0);
    for (int c0 = 0; c0 < n; c0 += TOK) {
        const int cnt = n - c0 < TOK ? n - c0 : TOK;
        __syncthreads();  // the chunk before is done with
#pragma unroll
        for (int it = 0; it < PER; it++) {
            if (it * THREADS >= cnt * DP) break;
            const int e = tid + it * THREADS, tok = e / DP, d = e % DP, at = (d / DPT) * (DPT + 4) + d % DPT;
            r_s[tok][at] = rr[it], k_s[tok][at] = rk[it], w_s[tok][at] = expf(-expf(rw[it]));
        }
#pragma unroll
        for (int it = 0; it < PER_V; it++) {
            const int e = tid + it * THREADS;
            if (e < cnt * COLS) v_s[e / COLS][e % COLS] = rv[it];
        }
        __syncthreads();
        if (c0 + TOK < n) fetch(c0 + TOK);
        // four tokens at a time: their reads from shared memory and their shuffles overlap, and only the state's own
        // multiply-adds follow one another
        const int at = part * (DPT + 4);
        float *out = p.out + (long long)(row0 + c0) * hk + (long long)h * p.dim + col;
        const bool writes = part == 0 && col < p.dim;
        int tok = 0;
        for (; tok + 4 <= cnt; tok += 4)
            wkv_tokens<DPT, PARTS, 4>(s, u, &r_s[tok][at], &k_s[tok][at], &w_s[tok][at], PITCH, &v_s[tok][vc], COLS, writes, out + tok * hk, hk);
        for (; tok < cnt; tok++)
            wkv_tokens<DPT, PARTS, 1>(s, u, &r_s[tok][at], &k_s[tok][at], &w_s[tok][at], PITCH, &v_s[tok][vc], COLS, writes, out + tok * hk, hk);
    }
#pragma unroll
    for (int i = 0; i < DPT; i++) {
        const int d = part * DPT + i;
        if (d < p.dim && col < p.dim) state[(long long)d * p.dim + col] = s[i];
    }
}

extern "C" int abk_wkv_scan(const void *proj, long long ld, int dtype, int r_at, int k_at, int v_at, int n_heads, int dim,
                            const float *pre, const float *w0, const float *bonus, float *state, float *out,
                            const int *seq_start, const int *seq_slot, int n_seqs, void *stream) {
    if (n_seqs <= 0) return 0;
    if (dim < 1 || dim > 256) ABK_REFUSE("wkv_scan: %d key channels a head are not 1 to 256", dim);
    if (n_heads < 1 || n_heads > 65535 || n_seqs > 65535) ABK_REFUSE("wkv_scan: %d heads, %d sequences", n_heads, n_seqs);
    WkvScan p;
    p.proj = proj, p.ld = ld, p.r_at = r_at, p.k_at = k_at, p.v_at = v_at, p.n_heads = n_heads, p.dim = dim;
    p.pre = pre, p.w0 = w0, p.bonus = bonus, p.state = state, p.out = out, p.seq_start = seq_start, p.seq_slot = seq_slot;
    cudaStream_t s = (cudaStream_t)stream;
    const int cols = dim <= 32 ? 32 : 16;  // value columns a CTA has
    dim3 grid((dim + cols - 1) / cols, n_heads, n_seqs);
#define WS_LAUNCH(T)                                                                                  \
    do {                                                                                              \
        if (dim <= 16) abk_launch(wkv_scan_kernel<T, 4, 4, 32, 16>, grid, dim3(128), 0, s, p);        \
        else if (dim <= 32) abk_launch(wkv_scan_kernel<T, 8, 4, 32, 16>, grid, dim3(128), 0, s, p);   \
        else if (dim <= 64) abk_launch(wkv_scan_kernel<T, 8, 8, 16, 16>, grid, dim3(128), 0, s, p);   \
        else if (dim <= 128) abk_launch(wkv_scan_kernel<T, 8, 16, 16, 16>, grid, dim3(256), 0, s, p); \
        else abk_launch(wkv_scan_kernel<T, 16, 16, 16, 8>, grid, dim3(256), 0, s, p);                 \
    } while (0)
    if (dtype == ABK_BF16) WS_LAUNCH(__nv_bfloat16);
    else WS_LAUNCH(float);
#undef WS_LAUNCH
    return ABK_LAUNCH_RESULT();
}
