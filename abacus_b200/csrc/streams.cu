// A residual stream kept as several copies ("streams") with learned connections between them, and the
// embedding that starts them. All arithmetic is float32; only the normed output may be bfloat16.
//
// The streams of a token lie together: X [tokens, s, d] float32. A branch (a mixer or a feed-forward) with
// connection (a [s], M [s, s], c [s]) and multiplier m reads u = sum_s a[s] X[s] and, once its output y is
// there, the streams become X'[t] = sum_s M[s, t] X[s] + m c[t] y for every t at once. What runs between two
// branches is one kernel here: it applies the write of the branch before (if any), stores the new streams,
// reads for the branch after and norms what it read, out = w * u / sqrt(mean(u^2) + eps). With a = 1 and a
// list of rows it is the model's end: the sum of the streams of the wanted rows, normed.
// With one stream, a = M = c = 1, this is the residual sum with a multiplier, x += m y.
#define ABK_DEFINE_ERROR
#include "common.cuh"

#define STREAMS_MAX 8

__device__ __forceinline__ void store4(float *p, float a, float b, float c, float d) { *(float4 *)p = make_float4(a, b, c, d); }
__device__ __forceinline__ void store4(__nv_bfloat16 *p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    *(uint2 *)p = make_uint2(*(uint32_t *)&lo, *(uint32_t *)&hi);
}

struct StreamsStep {
    float *x;             // [tokens, s, d]
    const float *y;       // [tokens, d] or null: no write pending
    const float *mix;     // [s, s] indexed [from, to] (used with y)
    const float *leave;   // [s] (used with y)
    float mult;
    const float *enter;   // [s]: the read
    const float *w;       // [d] the norm's weight as it multiplies, or null: out = u, not normed
    float eps;
    void *out;            // [rows, d]
    const int *rows;      // null: every row, and the new streams are stored; else output row r is made from row
                          // rows[r] and x is left as it is
    int s, d;
};

template <typename TO> __global__ void __launch_bounds__(256) streams_step_kernel(StreamsStep p) {
    extern __shared__ float u_s[];  // [d]
    __shared__ float scratch[33];
    __shared__ float mix_s[STREAMS_MAX * STREAMS_MAX], leave_s[STREAMS_MAX], enter_s[STREAMS_MAX];
    const int s = p.s, d = p.d;
    // the connections are weights: they may be read ahead of the wait
    if (threadIdx.x < s * s && p.y) mix_s[threadIdx.x] = p.mix[threadIdx.x];
    if (threadIdx.x < s) {
        leave_s[threadIdx.x] = p.y ? p.mult * p.leave[threadIdx.x] : 0.0f;
        enter_s[threadIdx.x] = p.enter[threadIdx.x];
    }
    pdl_wait();
    __syncthreads();
    const int r = blockIdx.x;
    const long long src = p.rows ? p.rows[r] : r;
    float *xr = p.x + src * s * d;
    const float *yr = p.y ? p.y + src * d : nullptr;
    const bool store = yr && !p.rows;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        float old[STREAMS_MAX], now[STREAMS_MAX];
#pragma unroll
        for (int a = 0; a < STREAMS_MAX; a++)
            if (a < s) old[a] = xr[(long long)a * d + j];
        float u = 0.0f;
        if (yr) {
            const float yv = yr[j];
#pragma unroll
            for (int t = 0; t < STREAMS_MAX; t++) {
                if (t < s) {
                    float acc = 0.0f;
#pragma unroll
                    for (int a = 0; a < STREAMS_MAX; a++)
                        if (a < s) acc = fmaf(mix_s[a * s + t], old[a], acc);
                    now[t] = fmaf(leave_s[t], yv, acc);
                    if (store) xr[(long long)t * d + j] = now[t];
                }
            }
        } else {
#pragma unroll
            for (int t = 0; t < STREAMS_MAX; t++)
                if (t < s) now[t] = old[t];
        }
#pragma unroll
        for (int t = 0; t < STREAMS_MAX; t++)
            if (t < s) u = fmaf(enter_s[t], now[t], u);
        u_s[j] = u;
        ss += u * u;
    }
    TO *o = (TO *)p.out + (long long)r * d;
    if (!p.w) {  // the read itself
        for (int j = threadIdx.x; j < d; j += blockDim.x) o[j] = from_float<TO>(u_s[j]);
        return;
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)d + p.eps);
    for (int j = threadIdx.x; j < d; j += blockDim.x) o[j] = from_float<TO>(p.w[j] * (u_s[j] * scale));
}

// The same for widths that are multiples of 4 with everything 16-byte aligned: four columns a thread, read and
// written as one vector per stream, all of a thread's loads in flight together.
template <typename TO> __global__ void __launch_bounds__(256) streams_step_vec_kernel(StreamsStep p) {
    extern __shared__ float u_s[];  // [d]
    __shared__ float scratch[33];
    __shared__ float mix_s[STREAMS_MAX * STREAMS_MAX], leave_s[STREAMS_MAX], enter_s[STREAMS_MAX];
    const int s = p.s, d = p.d;
    if (threadIdx.x < s * s && p.y) mix_s[threadIdx.x] = p.mix[threadIdx.x];
    if (threadIdx.x < s) {
        leave_s[threadIdx.x] = p.y ? p.mult * p.leave[threadIdx.x] : 0.0f;
        enter_s[threadIdx.x] = p.enter[threadIdx.x];
    }
    // a row that the block covers in one turn (width up to 4 x threads): the norm's weights come in ahead of the wait
    // and what was read stays in registers
    const bool one_turn = d <= 4 * (int)blockDim.x;
    float4 w_early = make_float4(1.0f, 1.0f, 1.0f, 1.0f), u_kept = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (one_turn && p.w && 4 * (int)threadIdx.x < d) w_early = *(const float4 *)(p.w + 4 * threadIdx.x);
    pdl_wait();
    __syncthreads();
    const int r = blockIdx.x;
    const long long src = p.rows ? p.rows[r] : r;
    float *xr = p.x + src * s * d;
    const float *yr = p.y ? p.y + src * d : nullptr;
    const bool store = yr && !p.rows;
    float ss = 0.0f;
    for (int j = 4 * threadIdx.x; j < d; j += 4 * blockDim.x) {
        float4 old[STREAMS_MAX];
#pragma unroll
        for (int a = 0; a < STREAMS_MAX; a++)
            if (a < s) old[a] = *(const float4 *)(xr + (long long)a * d + j);
        float4 u = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (yr) {
            const float4 yv = *(const float4 *)(yr + j);
#pragma unroll
            for (int t = 0; t < STREAMS_MAX; t++) {
                if (t < s) {
                    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                    for (int a = 0; a < STREAMS_MAX; a++) {
                        if (a < s) {
                            const float m = mix_s[a * s + t];
                            acc.x = fmaf(m, old[a].x, acc.x), acc.y = fmaf(m, old[a].y, acc.y);
                            acc.z = fmaf(m, old[a].z, acc.z), acc.w = fmaf(m, old[a].w, acc.w);
                        }
                    }
                    const float lv = leave_s[t], e = enter_s[t];
                    acc.x = fmaf(lv, yv.x, acc.x), acc.y = fmaf(lv, yv.y, acc.y);
                    acc.z = fmaf(lv, yv.z, acc.z), acc.w = fmaf(lv, yv.w, acc.w);
                    if (store) *(float4 *)(xr + (long long)t * d + j) = acc;
                    u.x = fmaf(e, acc.x, u.x), u.y = fmaf(e, acc.y, u.y), u.z = fmaf(e, acc.z, u.z), u.w = fmaf(e, acc.w, u.w);
                }
            }
        } else {
#pragma unroll
            for (int t = 0; t < STREAMS_MAX; t++) {
                if (t < s) {
                    const float e = enter_s[t];
                    u.x = fmaf(e, old[t].x, u.x), u.y = fmaf(e, old[t].y, u.y);
                    u.z = fmaf(e, old[t].z, u.z), u.w = fmaf(e, old[t].w, u.w);
                }
            }
        }
        if (one_turn) u_kept = u;
        else *(float4 *)(u_s + j) = u;
        ss += u.x * u.x + u.y * u.y + u.z * u.z + u.w * u.w;
    }
    TO *o = (TO *)p.out + (long long)r * d;
    float scale = 1.0f;
    if (p.w) {
        ss = block_sum(ss, scratch);
        scale = 1.0f / sqrtf(ss / (float)d + p.eps);
    }
    for (int j = 4 * threadIdx.x; j < d; j += 4 * blockDim.x) {  // a thread reads back what it wrote itself
        const float4 u = one_turn ? u_kept : *(const float4 *)(u_s + j);
        float4 w = w_early;
        if (p.w && !one_turn) w = *(const float4 *)(p.w + j);
        if (p.w) store4(o + j, w.x * (u.x * scale), w.y * (u.y * scale), w.z * (u.z * scale), w.w * (u.w * scale));
        else store4(o + j, u.x, u.y, u.z, u.w);
    }
}

extern "C" int abk_streams_step(float *x, const float *y, const float *mix, const float *leave, float mult,
                                const float *enter, const float *w, float eps, void *out, int out_dtype,
                                const int *rows, int n_rows, int s, int d, void *stream) {
    if (n_rows <= 0) return 0;
    if (s < 1 || s > STREAMS_MAX) ABK_REFUSE("streams: %d streams, the kernel takes 1 to %d", s, STREAMS_MAX);
    if (d < 1 || d > 12288) ABK_REFUSE("streams: width %d is more than a row in shared memory (12288)", d);
    StreamsStep p;
    p.x = x, p.y = y, p.mix = mix, p.leave = leave, p.mult = mult, p.enter = enter, p.w = w, p.eps = eps;
    p.out = out, p.rows = rows, p.s = s, p.d = d;
    cudaStream_t st = (cudaStream_t)stream;
    if (d % 4 == 0 && !(((uintptr_t)x | (uintptr_t)y | (uintptr_t)w | (uintptr_t)out) & 15)) {
        int lanes = (d / 4 + 31) / 32 * 32;
        lanes = lanes > 256 ? 256 : lanes;
        if (out_dtype == ABK_BF16)
            abk_launch(streams_step_vec_kernel<__nv_bfloat16>, dim3(n_rows), dim3(lanes), (size_t)d * 4, st, p);
        else
            abk_launch(streams_step_vec_kernel<float>, dim3(n_rows), dim3(lanes), (size_t)d * 4, st, p);
        return ABK_LAUNCH_RESULT();
    }
    const int threads = d >= 1024 ? 256 : 128;
    if (out_dtype == ABK_BF16)
        abk_launch(streams_step_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), (size_t)d * 4, st, p);
    else
        abk_launch(streams_step_kernel<float>, dim3(n_rows), dim3(threads), (size_t)d * 4, st, p);
    return ABK_LAUNCH_RESULT();
}

// ------------------------------------------------------------------ embedding with a scale and a hashed pair table
// x[t, a, :] = float(table[tok]) * scale + float(pairs[row]) for every stream a, where
// row = (prev * mul_prev + tok * mul_cur) mod buckets and prev is the token before in the same sequence: the row
// above in this step, or, for a sequence's first row of the step, the token its slot remembers. A sequence's first
// token takes row `buckets`, the table's last. pairs null: no pair table.
struct EmbedPairs {
    const int *tokens, *token_seq, *token_pos, *seq_slot, *seq_pos0;
    const void *table, *pairs;
    const int *remembered;  // [slots]
    float *x;
    float scale;
    int d, vocab, s;
    long long buckets, mul_prev, mul_cur;
    int *status;
};

template <typename TW> __global__ void embed_pairs_kernel(EmbedPairs p) {
    pdl_wait();
    const int t = blockIdx.x, d = p.d;
    const int seq = p.token_seq[t];
    float *out = p.x + (long long)t * p.s * d;
    if (seq < 0) {  // padding
        for (int j = threadIdx.x; j < p.s * d; j += blockDim.x) out[j] = 0.0f;
        return;
    }
    const int tok = p.tokens[t], pos = p.token_pos[t];
    bool bad = tok < 0 || tok >= p.vocab;
    long long row = p.buckets;
    if (p.pairs && pos > 0) {
        int prev = pos > p.seq_pos0[seq] ? p.tokens[t - 1] : p.remembered[p.seq_slot[seq]];
        if (prev < 0 || prev >= p.vocab) bad = true, prev = 0;
        row = ((long long)prev * p.mul_prev + (long long)(bad ? 0 : tok) * p.mul_cur) % p.buckets;
    }
    if (bad && threadIdx.x == 0) atomicOr(p.status, 1);
    const TW *e = (const TW *)p.table + (long long)(bad ? 0 : tok) * d;
    const TW *b = p.pairs ? (const TW *)p.pairs + row * d : nullptr;
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        float v = bad ? 0.0f : to_float(e[j]) * p.scale;
        if (b && !bad) v += to_float(b[j]);
        for (int a = 0; a < p.s; a++) out[(long long)a * d + j] = v;
    }
}

extern "C" int abk_embed_pairs(const int *tokens, const int *token_seq, const int *token_pos, const int *seq_slot,
                               const int *seq_pos0, const void *table, const void *pairs, int table_dtype,
                               const int *remembered, float *x, float scale, int n_tokens, int d, int vocab, int s,
                               long long buckets, long long mul_prev, long long mul_cur, int *status, void *stream) {
    if (n_tokens <= 0) return 0;
    if (pairs && buckets < 1) ABK_REFUSE("embedding: a pair table of %lld buckets", buckets);
    EmbedPairs p;
    p.tokens = tokens, p.token_seq = token_seq, p.token_pos = token_pos, p.seq_slot = seq_slot, p.seq_pos0 = seq_pos0;
    p.table = table, p.pairs = pairs, p.remembered = remembered, p.x = x, p.scale = scale, p.d = d, p.vocab = vocab;
    p.s = s, p.buckets = buckets, p.mul_prev = mul_prev, p.mul_cur = mul_cur, p.status = status;
    const int threads = d >= 1024 ? 256 : 128;
    cudaStream_t st = (cudaStream_t)stream;
    if (table_dtype == ABK_BF16)
        abk_launch(embed_pairs_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, st, p);
    else
        abk_launch(embed_pairs_kernel<float>, dim3(n_tokens), dim3(threads), 0, st, p);
    return ABK_LAUNCH_RESULT();
}

// Every sequence of the step leaves its last token with its slot (a kernel of its own: the embedding above reads
// what the step before left while other rows of the same sequence are still looked up).
__global__ void remember_tokens_kernel(const int *tokens, const int *seq_start, const int *seq_slot, int n_seqs,
                                       int *remembered) {
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_seqs) return;
    const int a = seq_start[i], b = seq_start[i + 1];
    if (b > a) remembered[seq_slot[i]] = tokens[b - 1];
}

extern "C" int abk_remember_tokens(const int *tokens, const int *seq_start, const int *seq_slot, int n_seqs,
                                   int *remembered, void *stream) {
    if (n_seqs <= 0) return 0;
    abk_launch(remember_tokens_kernel, dim3((n_seqs + 127) / 128), dim3(128), 0, (cudaStream_t)stream, tokens, seq_start,
               seq_slot, n_seqs, remembered);
    return ABK_LAUNCH_RESULT();
}

// ------------------------------------------------------------------ learned positions, a stream that is joined again
// x[t, a] = table[token] + positions[position] for every stream a: an embedding with a learned vector per position (not
// scaled). `keep` (or null) gets a copy [tokens, d]: what a later layer adds to the stream again (rejoin).
struct EmbedPositions {
    const int *tokens, *token_seq, *token_pos;
    const void *table, *positions;
    float *x, *keep;
    int d, vocab, n_positions, s;
    int *status;
};

template <typename TW> __global__ void embed_positions_kernel(EmbedPositions p) {
    pdl_wait();
    const int t = blockIdx.x, d = p.d;
    const int seq = p.token_seq[t];
    float *out = p.x + (long long)t * p.s * d;
    float *keep = p.keep ? p.keep + (long long)t * d : nullptr;
    const int tok = seq < 0 ? 0 : p.tokens[t], pos = seq < 0 ? 0 : p.token_pos[t];
    const bool bad = tok < 0 || tok >= p.vocab || pos < 0 || pos >= p.n_positions;
    if (seq >= 0 && bad && threadIdx.x == 0) atomicOr(p.status, 1);
    const TW *e = (const TW *)p.table + (long long)(bad ? 0 : tok) * d;
    const TW *w = (const TW *)p.positions + (long long)(bad ? 0 : pos) * d;
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        const float v = seq < 0 || bad ? 0.0f : to_float(e[j]) + to_float(w[j]);
        for (int a = 0; a < p.s; a++) out[(long long)a * d + j] = v;
        if (keep) keep[j] = v;
    }
}

extern "C" int abk_embed_positions(const int *tokens, const int *token_seq, const int *token_pos, const void *table,
                                   const void *positions, int table_dtype, float *x, float *keep, int n_tokens, int d,
                                   int vocab, int n_positions, int s, int *status, void *stream) {
    if (n_tokens <= 0) return 0;
    EmbedPositions p;
    p.tokens = tokens, p.token_seq = token_seq, p.token_pos = token_pos, p.table = table, p.positions = positions;
    p.x = x, p.keep = keep, p.d = d, p.vocab = vocab, p.n_positions = n_positions, p.s = s, p.status = status;
    const int threads = d >= 1024 ? 256 : 128;
    cudaStream_t st = (cudaStream_t)stream;
    if (table_dtype == ABK_BF16)
        abk_launch(embed_positions_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, st, p);
    else
        abk_launch(embed_positions_kernel<float>, dim3(n_tokens), dim3(threads), 0, st, p);
    return ABK_LAUNCH_RESULT();
}

// x[t, a] += kept[t] for every stream a (x float32 [tokens, s, d], kept float32 [tokens, d]).
__global__ void __launch_bounds__(256) rejoin_kernel(float *x, const float *kept, long long total, int s, int d) {
    pdl_wait();
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= total) return;
    const long long t = i / ((long long)s * d);
    x[i] += kept[t * d + i % d];
}

extern "C" int abk_rejoin(float *x, const float *kept, int n_tokens, int s, int d, void *stream) {
    const long long total = (long long)n_tokens * s * d;
    if (total <= 0) return 0;
    abk_launch(rejoin_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, x, kept, total, s, d);
    return ABK_LAUNCH_RESULT();
}

// out[t] = share * (wa * a[t] / rms(a[t]) + wb * b[t] / rms(b[t])): two branches that ran side by side, each normed over
// the width with a weight of its own, then joined. All float32; a block a row.
__global__ void __launch_bounds__(128) normed_pair_kernel(const float *a, const float *b, const float *wa, const float *wb,
                                                          float *out, int d, float eps, float share) {
    __shared__ float scratch[33];
    pdl_wait();
    const long long t = blockIdx.x;
    const float *ar = a + t * d, *br = b + t * d;
    float sa = 0.0f, sb = 0.0f;
    for (int j = threadIdx.x; j < d; j += 128) sa = fmaf(ar[j], ar[j], sa), sb = fmaf(br[j], br[j], sb);
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    const float ra = 1.0f / sqrtf(sa / (float)d + eps), rb = 1.0f / sqrtf(sb / (float)d + eps);
    for (int j = threadIdx.x; j < d; j += 128) out[t * d + j] = share * (ar[j] * ra * wa[j] + br[j] * rb * wb[j]);
}

extern "C" int abk_normed_pair(const float *a, const float *b, const float *wa, const float *wb, float *out, int n_tokens,
                               int d, float eps, float share, void *stream) {
    if (n_tokens <= 0 || d <= 0) return 0;
    abk_launch(normed_pair_kernel, dim3(n_tokens), dim3(128), 0, (cudaStream_t)stream, a, b, wa, wb, out, d, eps, share);
    return ABK_LAUNCH_RESULT();
}

// ------------------------------------------------------------------ a stream made anew from itself and the embedding
// Before a pass over a run of layers the stream becomes Win [x; x0] + step: `stream_beside` writes the branch still
// pending (x += y, one stream) and lays the row [x | x0] out in the product's type; `add_vector` adds the pass's vector
// to the product's result.
template <typename T>
__global__ void __launch_bounds__(256) stream_beside_kernel(float *x, const float *y, const float *x0, T *out, int d, long long total) {
    pdl_wait();
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= total) return;
    const long long t = i / d;
    const int j = (int)(i - t * d);
    float v = x[i];
    if (y) {
        v += y[i];
        x[i] = v;
    }
    out[t * 2 * d + j] = from_float<T>(v);
    out[t * 2 * d + d + j] = from_float<T>(x0[i]);
}

extern "C" int abk_stream_beside(float *x, const float *y, const float *x0, void *out, int dtype, int n_tokens, int d, void *stream) {
    const long long total = (long long)n_tokens * d;
    if (total <= 0) return 0;
    const dim3 grid((unsigned)((total + 255) / 256));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == ABK_BF16) abk_launch(stream_beside_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, x, y, x0, (__nv_bfloat16 *)out, d, total);
    else abk_launch(stream_beside_kernel<float>, grid, dim3(256), 0, s, x, y, x0, (float *)out, d, total);
    return ABK_LAUNCH_RESULT();
}

__global__ void __launch_bounds__(256) add_vector_kernel(float *x, const float *v, int d, long long total) {
    pdl_wait();
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i < total) x[i] += v[i % d];
}

extern "C" int abk_add_vector(float *x, const float *v, int n_tokens, int d, void *stream) {
    const long long total = (long long)n_tokens * d;
    if (total <= 0) return 0;
    abk_launch(add_vector_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, x, v, d, total);
    return ABK_LAUNCH_RESULT();
}
