// Causal grouped-query attention over the paged cache, for any head size up to 256 that is a
// multiple of 8, any number of heads and groups, with or without a window. One block per
// (token, query head); float32 arithmetic with an online softmax over tiles of 128 keys (in the
// bfloat16 instantiation the probabilities are rounded to bfloat16 for the second product, as in
// the tensor-core kernels, and summed unrounded; a model that wants them in float32 says so).
// Options: values of another size than keys; a window that also keeps a sequence's first keys (key j is
// seen from i when j <= i and (i - j < window or j < keep_first)); a sink, a learned score per head that
// joins the softmax's denominator once, unscaled, without a key or a value; chunks (key j is seen from i only when
// both lie in the same run of `chunk` positions, counted from the sequence's first); capped scores
// (s <- cap * tanh(s / cap), after the scale).
// It serves prefill and decode alike and is the kernel every size falls back to; the float32
// path of the model uses nothing else for attention.
//
// Formula (src/model.c:197-211): s_j = (q . k_j) * scale for the keys the token may see,
// p = softmax(s), out = sum_j p_j v_j; query head h reads kv head h / (Hq / Hkv).
// The result for a token depends only on its own position and keys: tiles start at the first
// visible key, never at a batch-dependent place.
#define ABK_DEFINE_ERROR
#include "common.cuh"

#define ATT_THREADS 128
#define ATT_MAX_HEAD_DIM 640
#define ATT_COLS (ATT_MAX_HEAD_DIM / ATT_THREADS)  // value columns a thread may have

struct AttnGeneric {
    const void *q;      // row t, head h at q + (t * q_row + h * head_dim)
    long long q_row;    // elements between rows of q
    void *out;          // [tokens, n_heads * head_dim]
    int n_heads, n_kv_heads, head_dim;
    int v_dim;          // size of a value head (out is [tokens, n_heads * v_dim])
    float scale;
    int window;         // 0: all earlier keys
    int keep_first;     // with a window: the sequence's first keep_first keys are seen too
    const float *sink;  // [n_heads] or null
    const int *token_seq, *token_pos, *seq_slot, *seq_start, *seq_pos0;
    // keys and values either in the paged cache ...
    const void *k_pool, *v_pool;
    PagedCache cache;
    // ... or in the rows of this step (k_step null: use the cache): position j of sequence s is
    // row seq_start[s] + j - seq_pos0[s]
    const void *k_step, *v_step;
    long long kv_row;   // elements between rows of k_step / v_step
    PagedCache v_cache; // the values' pool has pages of v_dim
    int values_in_keys; // a value is the first v_dim elements of its key (one pool, one row per token)
    int vector_rows;    // key rows are whole 16-byte pieces at 16-byte places (else they are read an element at a time)
    int chunk;          // > 0: only the keys of the token's own run of `chunk` positions are seen
    float softcap;      // > 0: s <- softcap * tanh(s / softcap)
};

template <typename T> __device__ __forceinline__ float dot_row_plain(const float *q, const T *k, int hd) {
    float acc = 0.0f;
    for (int i = 0; i < hd; i++) acc = fmaf(q[i], to_float(k[i]), acc);
    return acc;
}

template <typename T> __device__ __forceinline__ float dot_row(const float *q, const T *k, int hd);
template <> __device__ __forceinline__ float dot_row<float>(const float *q, const float *k, int hd) {
    float acc = 0.0f;
    for (int i = 0; i < hd; i += 4) {
        float4 v = *(const float4 *)(k + i);
        acc = fmaf(q[i], v.x, acc), acc = fmaf(q[i + 1], v.y, acc);
        acc = fmaf(q[i + 2], v.z, acc), acc = fmaf(q[i + 3], v.w, acc);
    }
    return acc;
}
template <> __device__ __forceinline__ float dot_row<__nv_bfloat16>(const float *q, const __nv_bfloat16 *k, int hd) {
    float acc = 0.0f;
    for (int i = 0; i < hd; i += 8) {
        uint4 raw = *(const uint4 *)(k + i);
        const __nv_bfloat162 *h = (const __nv_bfloat162 *)&raw;
#pragma unroll
        for (int u = 0; u < 4; u++) {
            float2 f = __bfloat1622float2(h[u]);
            acc = fmaf(q[i + 2 * u], f.x, acc), acc = fmaf(q[i + 2 * u + 1], f.y, acc);
        }
    }
    return acc;
}

// ROUNDED_P: the probabilities are a stored tensor in the model's type (bfloat16) for the second product.
template <typename T, bool ROUNDED_P>
__global__ void __launch_bounds__(ATT_THREADS) attention_generic_kernel(AttnGeneric p) {
    __shared__ float q_s[ATT_MAX_HEAD_DIM];
    __shared__ float p_s[ATT_THREADS];
    __shared__ long long v_off[ATT_THREADS];
    __shared__ float scratch[33];
    int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, hd = p.head_dim, vd = p.v_dim;
    int seq = p.token_seq[t];
    T *out = (T *)p.out + ((long long)t * p.n_heads + h) * vd;
    if (seq < 0) {  // padding
        for (int d = tid; d < vd; d += ATT_THREADS) out[d] = from_float<T>(0.0f);
        return;
    }
    int pos = p.token_pos[t], slot = p.seq_slot[seq];
    int kvh = h / (p.n_heads / p.n_kv_heads);
    int lo = p.window > 0 && pos - p.window + 1 > 0 ? pos - p.window + 1 : 0;
    if (p.chunk > 0 && pos / p.chunk * p.chunk > lo) lo = pos / p.chunk * p.chunk;
    // the sequence's first keys that the window no longer reaches: positions [0, first_end)
    int first_end = p.keep_first < lo ? p.keep_first : lo;
    const T *q = (const T *)p.q + (long long)t * p.q_row + (long long)h * hd;
    for (int d = tid; d < hd; d += ATT_THREADS) q_s[d] = to_float(q[d]);
    __syncthreads();

    float m = -INFINITY, l = 0.0f, acc[ATT_COLS];
#pragma unroll
    for (int u = 0; u < ATT_COLS; u++) acc[u] = 0.0f;
    if (p.sink) m = p.sink[h], l = 1.0f;  // a key with this score and no value (never with ROUNDED_P)
    // two runs of keys: the kept first ones, then the window (or everything up to the token)
    for (int run = first_end > 0 ? 0 : 1; run < 2; run++)
    for (int base = run ? lo : 0, end = run ? pos : first_end - 1; base <= end; base += ATT_THREADS) {
        int j = base + tid;
        bool valid = j <= end;
        float s = -INFINITY;
        if (valid) {
            const T *k;
            long long vo;
            if (p.k_step) {
                long long row = (long long)p.seq_start[seq] + j - p.seq_pos0[seq];
                vo = row * p.kv_row + (long long)kvh * (p.values_in_keys ? hd : vd);
                k = (const T *)p.k_step + row * p.kv_row + (long long)kvh * hd;
            } else {
                int page = cache_page(p.cache, slot, j);
                vo = cache_offset(p.v_cache, page, kvh, p.n_kv_heads, j, p.values_in_keys ? hd : vd);
                k = (const T *)p.k_pool + cache_offset(p.cache, page, kvh, p.n_kv_heads, j, hd);
            }
            v_off[tid] = vo;
            s = (p.vector_rows ? dot_row<T>(q_s, k, hd) : dot_row_plain<T>(q_s, k, hd)) * p.scale;
            if (p.softcap > 0.0f) s = p.softcap * tanhf(s / p.softcap);
            if (ROUNDED_P) s *= 1.4426950408889634f;
        }
        float m_new, pj, corr;
        if (ROUNDED_P) {
            // in units of log2, against the maximum rounded up to a whole number: a probability is then the same
            // bits times a power of two whatever tile it is in, and rounds to the same bfloat16 in every kernel
            m_new = fmaxf(m, ceilf(block_max(s, scratch)));
            pj = valid ? exp2f(s - m_new) : 0.0f;
            corr = exp2f(m - m_new);  // 0 on the first tile (m = -inf)
        } else {
            m_new = fmaxf(m, block_max(s, scratch));
            pj = valid ? expf(s - m_new) : 0.0f;
            corr = expf(m - m_new);
        }
        // the probabilities of the second product are a stored tensor: bfloat16 where the model's are (the
        // tensor-core kernels must round them, so every kernel does); the row's sum is of the unrounded ones
        p_s[tid] = ROUNDED_P ? to_float(from_float<T>(pj)) : pj;
        l = l * corr + block_sum(pj, scratch);  // the barrier inside also publishes p_s and v_off
        m = m_new;
        int n_valid = end - base + 1 < ATT_THREADS ? end - base + 1 : ATT_THREADS;
        const T *v_base = (const T *)(p.k_step ? p.v_step : p.v_pool);
#pragma unroll
        for (int u = 0; u < ATT_COLS; u++) acc[u] *= corr;
        if (tid < vd) {
            for (int jj = 0; jj < n_valid; jj++) {
                const T *v = v_base + v_off[jj];
                acc[0] = fmaf(p_s[jj], to_float(v[tid]), acc[0]);
#pragma unroll
                for (int u = 1; u < ATT_COLS; u++)
                    if (tid + u * ATT_THREADS < vd) acc[u] = fmaf(p_s[jj], to_float(v[tid + u * ATT_THREADS]), acc[u]);
            }
        }
        __syncthreads();  // p_s and v_off are rewritten by the next tile
    }
#pragma unroll
    for (int u = 0; u < ATT_COLS; u++)
        if (tid + u * ATT_THREADS < vd) out[tid + u * ATT_THREADS] = from_float<T>(acc[u] / l);
}

static int attention_general(int values_in_keys, const void *q, long long q_row, void *out, int dtype, int n_tokens, int n_heads,
                                     int n_kv_heads, int head_dim, float scale, int window, const int *token_seq,
                                     const int *token_pos, const int *seq_slot, const int *seq_start,
                                     const int *seq_pos0, const void *k_pool, const void *v_pool,
                                     const int *page_table, int table_width, int ring_pages, int tokens_per_page,
                                     const void *k_step, const void *v_step, long long kv_row, int v_dim,
                                     int keep_first, int pinned_pages, const float *sink, int exact_weights,
                                     void *stream, int chunk = 0, float softcap = 0.0f) {
    if (n_tokens <= 0) return 0;
    if (v_dim <= 0) v_dim = head_dim;
    if (chunk < 0 || softcap < 0.0f) ABK_REFUSE("attention: a chunk of %d positions, a score cap of %g", chunk, softcap);
    if (v_dim > ATT_MAX_HEAD_DIM) ABK_REFUSE("attention: value size %d is more than %d", v_dim, ATT_MAX_HEAD_DIM);
    if (keep_first < 0 || (keep_first > 0 && window <= 0)) keep_first = 0;
    if (sink && !exact_weights && dtype == ABK_BF16)
        ABK_REFUSE("attention: a sink goes with softmax weights in float32 (exact_weights)");
    if (head_dim > ATT_MAX_HEAD_DIM || head_dim < 1)
        ABK_REFUSE("attention: head_dim %d is not 1 to %d", head_dim, ATT_MAX_HEAD_DIM);
    if (n_kv_heads < 1 || n_heads % n_kv_heads)
        ABK_REFUSE("attention: %d query heads do not divide into %d kv heads", n_heads, n_kv_heads);
    if (n_heads > 65535) ABK_REFUSE("attention: %d heads are more than a grid takes", n_heads);
    AttnGeneric p;
    p.q = q, p.q_row = q_row, p.out = out, p.n_heads = n_heads, p.n_kv_heads = n_kv_heads, p.head_dim = head_dim;
    p.scale = scale, p.window = window, p.token_seq = token_seq, p.token_pos = token_pos, p.seq_slot = seq_slot;
    p.seq_start = seq_start, p.seq_pos0 = seq_pos0, p.k_pool = k_pool, p.v_pool = v_pool;
    p.cache.page_table = page_table, p.cache.table_width = table_width, p.cache.ring_pages = ring_pages;
    p.cache.tokens_per_page = tokens_per_page;
    p.cache.pinned_pages = pinned_pages;
    p.v_cache = p.cache;
    p.k_step = k_step, p.v_step = v_step, p.kv_row = kv_row;
    p.v_dim = v_dim, p.keep_first = keep_first, p.sink = sink, p.values_in_keys = values_in_keys;
    p.chunk = chunk, p.softcap = softcap;
    if (values_in_keys && v_dim > head_dim) ABK_REFUSE("attention: values of %d inside keys of %d", v_dim, head_dim);
    const int esize = dtype == ABK_BF16 ? 2 : 4;
    p.vector_rows = (head_dim * esize) % 16 == 0 && (kv_row * esize) % 16 == 0 &&
                    !(((uintptr_t)k_pool | (uintptr_t)k_step) & 15);
    dim3 grid(n_tokens, n_heads);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == ABK_BF16 && !exact_weights)
        attention_generic_kernel<__nv_bfloat16, true><<<grid, ATT_THREADS, 0, s>>>(p);
    else if (dtype == ABK_BF16)
        attention_generic_kernel<__nv_bfloat16, false><<<grid, ATT_THREADS, 0, s>>>(p);
    else
        attention_generic_kernel<float, false><<<grid, ATT_THREADS, 0, s>>>(p);
    return ABK_LAUNCH_RESULT();
}

extern "C" int abk_attention_general(const void *q, long long q_row, void *out, int dtype, int n_tokens, int n_heads,
                                     int n_kv_heads, int head_dim, float scale, int window, const int *token_seq,
                                     const int *token_pos, const int *seq_slot, const int *seq_start,
                                     const int *seq_pos0, const void *k_pool, const void *v_pool,
                                     const int *page_table, int table_width, int ring_pages, int tokens_per_page,
                                     const void *k_step, const void *v_step, long long kv_row, int v_dim,
                                     int keep_first, int pinned_pages, const float *sink, int exact_weights,
                                     void *stream) {
    return attention_general(0, q, q_row, out, dtype, n_tokens, n_heads, n_kv_heads, head_dim, scale, window, token_seq,
                             token_pos, seq_slot, seq_start, seq_pos0, k_pool, v_pool, page_table, table_width, ring_pages,
                             tokens_per_page, k_step, v_step, kv_row, v_dim, keep_first, pinned_pages, sink, exact_weights,
                             stream);
}

// The general form with chunks and capped scores.
extern "C" int abk_attention_chunked(const void *q, long long q_row, void *out, int dtype, int n_tokens, int n_heads,
                                     int n_kv_heads, int head_dim, float scale, int window, const int *token_seq,
                                     const int *token_pos, const int *seq_slot, const int *seq_start,
                                     const int *seq_pos0, const void *k_pool, const void *v_pool,
                                     const int *page_table, int table_width, int ring_pages, int tokens_per_page,
                                     const void *k_step, const void *v_step, long long kv_row, int v_dim,
                                     int keep_first, int pinned_pages, const float *sink, int exact_weights, int chunk,
                                     float softcap, void *stream) {
    return attention_general(0, q, q_row, out, dtype, n_tokens, n_heads, n_kv_heads, head_dim, scale, window, token_seq,
                             token_pos, seq_slot, seq_start, seq_pos0, k_pool, v_pool, page_table, table_width, ring_pages,
                             tokens_per_page, k_step, v_step, kv_row, v_dim, keep_first, pinned_pages, sink, exact_weights,
                             stream, chunk, softcap);
}

// Keys that carry their values: a value is the first v_dim elements of its key row (one pool; with keys from the
// step's rows, one row). What attention over shared latent rows needs (csrc/latent.cu).
extern "C" int abk_attention_values_in_keys(const void *q, long long q_row, void *out, int dtype, int n_tokens, int n_heads,
                                            int n_kv_heads, int head_dim, float scale, const int *token_seq,
                                            const int *token_pos, const int *seq_slot, const int *seq_start,
                                            const int *seq_pos0, const void *k_pool, const int *page_table,
                                            int table_width, int tokens_per_page, int v_dim, const float *sink,
                                            int exact_weights, void *stream) {
    return attention_general(1, q, q_row, out, dtype, n_tokens, n_heads, n_kv_heads, head_dim, scale, 0, token_seq,
                             token_pos, seq_slot, seq_start, seq_pos0, k_pool, k_pool, page_table, table_width, 0,
                             tokens_per_page, nullptr, nullptr, 0, v_dim, 0, 0, sink, exact_weights, stream);
}

// The same without the options: values as large as keys, no kept first keys, no sink, probabilities in the model's type.
extern "C" int abk_attention_generic(const void *q, long long q_row, void *out, int dtype, int n_tokens, int n_heads,
                                     int n_kv_heads, int head_dim, float scale, int window, const int *token_seq,
                                     const int *token_pos, const int *seq_slot, const int *seq_start,
                                     const int *seq_pos0, const void *k_pool, const void *v_pool,
                                     const int *page_table, int table_width, int ring_pages, int tokens_per_page,
                                     const void *k_step, const void *v_step, long long kv_row, void *stream) {
    return abk_attention_general(q, q_row, out, dtype, n_tokens, n_heads, n_kv_heads, head_dim, scale, window, token_seq,
                                 token_pos, seq_slot, seq_start, seq_pos0, k_pool, v_pool, page_table, table_width,
                                 ring_pages, tokens_per_page, k_step, v_step, kv_row, head_dim, 0, 0, nullptr, 0, stream);
}
