// Decode attention (one new token per sequence) over the paged cache with the general options (a window that also
// keeps the first keys, a sink, values of another size than keys, float32 softmax weights), split along the keys so
// that a handful of rows fills the GPU: a CTA takes 128 of a row's visible keys for all query heads of one kv head
// (each key and value row is read once for the group), and leaves, per head, the maximum, the sum and the
// unnormalised weighted values of its keys; a second kernel folds a row's parts, the sink among them.
//
//   key j is seen from position i when j <= i and (window == 0 or i - j < window or j < keep_first)
//                                             and (chunk == 0 or j / chunk == i / chunk)
//   p_j = exp(z_j - M) / (exp(sink - M) + sum_j exp(z_j - M)),  z_j = scale * (q . k_j),  out = sum_j p_j v_j
//   (with a cap c of the scores, z_j = c tanh(scale * (q . k_j) / c))
//
// A row's visible keys are numbered: first the kept first keys the window no longer reaches, then the window's
// (or all). Part t has numbers [128 t, 128 t + 128). All arithmetic is float32.
#define ABK_DEFINE_ERROR
#include "common.cuh"

#define AS_THREADS 128
#define AS_MAX_GROUP 16
#define AS_MAX_DIM 256

struct AttnSplit {
    const void *q;       // row t, head h at q + t * q_row + h * head_dim
    long long q_row;
    float *parts;        // [tokens, heads, n_parts, v_dim + 2]: weighted values, then maximum and sum
    void *out;           // [tokens, heads * v_dim]
    int n_heads, n_kv_heads, head_dim, v_dim;
    float scale;
    float softcap;       // > 0: z <- softcap * tanh(z / softcap), after the scale
    int window, keep_first;
    int chunk;           // > 0: key j is seen from i only if j / chunk == i / chunk
    const float *sink;
    const int *token_seq, *token_pos, *seq_slot;
    const void *k_pool, *v_pool;
    PagedCache cache, v_cache;
    int n_parts;
    int values_in_keys;  // a value is the first v_dim elements of its key row (one pool)
    int one_kv;          // the cache has one kv head; n_kv_heads counts runs of query heads that a CTA takes together
    const void *gate;    // null, or a gate per token and head (of q's type, at gate + t * ldg + h): the head's output is
    long long ldg;       // multiplied by its sigmoid where the parts are folded
};

// (first key of the window, number of kept first keys before it, number of visible keys) of a token at pos
__device__ __forceinline__ void visible_keys(const AttnSplit &p, int pos, int &lo, int &kept, int &total) {
    lo = p.window > 0 && pos - p.window + 1 > 0 ? pos - p.window + 1 : 0;
    kept = p.keep_first < lo ? p.keep_first : lo;
    if (p.chunk > 0) {  // the token's chunk starts no earlier than any kept first key that lies outside it
        const int first = pos / p.chunk * p.chunk;
        if (first > lo) lo = first;
        if (first > 0) kept = 0;
    }
    total = kept + pos - lo + 1;
}

// The score of a product q . k: scaled, then capped where the layer caps its scores.
__device__ __forceinline__ float score_of(const AttnSplit &p, float dot) {
    const float z = dot * p.scale;
    return p.softcap > 0.0f ? p.softcap * tanhf(z / p.softcap) : z;
}

// q (float32, 16-byte aligned, the same for every thread: a broadcast) . k (this thread's key row)
template <typename T> __device__ __forceinline__ float dot_q(const float *q, const T *k, int hd);
template <> __device__ __forceinline__ float dot_q<float>(const float *q, const float *k, int hd) {
    float acc = 0.0f;
    for (int i = 0; i < hd; i += 4) {
        const float4 v = *(const float4 *)(k + i), w = *(const float4 *)(q + i);
        acc = fmaf(w.x, v.x, acc), acc = fmaf(w.y, v.y, acc), acc = fmaf(w.z, v.z, acc), acc = fmaf(w.w, v.w, acc);
    }
    return acc;
}
template <> __device__ __forceinline__ float dot_q<__nv_bfloat16>(const float *q, const __nv_bfloat16 *k, int hd) {
    float a0 = 0.0f, a1 = 0.0f;
    for (int i = 0; i < hd; i += 8) {
        const uint4 raw = *(const uint4 *)(k + i);
        const float4 w0 = *(const float4 *)(q + i), w1 = *(const float4 *)(q + i + 4);
        const __nv_bfloat162 *h = (const __nv_bfloat162 *)&raw;
        const float2 f0 = __bfloat1622float2(h[0]), f1 = __bfloat1622float2(h[1]), f2 = __bfloat1622float2(h[2]),
                     f3 = __bfloat1622float2(h[3]);
        a0 = fmaf(w0.x, f0.x, a0), a1 = fmaf(w0.y, f0.y, a1), a0 = fmaf(w0.z, f1.x, a0), a1 = fmaf(w0.w, f1.y, a1);
        a0 = fmaf(w1.x, f2.x, a0), a1 = fmaf(w1.y, f2.y, a1), a0 = fmaf(w1.z, f3.x, a0), a1 = fmaf(w1.w, f3.y, a1);
    }
    return a0 + a1;
}

// STAGED: the part's 128 key rows come into shared memory by cp.async, all at once (padded by 16 bytes so that a thread
// reading its own row meets no bank conflict), and once the scores are made the 128 value rows into the same memory,
// under the softmax; else each thread reads global memory.
// GMAX: the group's size rounded up to 1, 2, 4, 8 or 16 (what the loops over its heads are unrolled to).
__device__ __forceinline__ void as_mma_bf16(float *c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// A float32 number as three bfloat16 numbers that add up to it (its 24 bits), each pair packed for one operand register.
__device__ __forceinline__ void as_split3(float x, float y, uint32_t &hi, uint32_t &mid, uint32_t &lo) {
    const __nv_bfloat16 xh = __float2bfloat16_rn(x), yh = __float2bfloat16_rn(y);
    const float xr = x - __bfloat162float(xh), yr = y - __bfloat162float(yh);
    const __nv_bfloat16 xm = __float2bfloat16_rn(xr), ym = __float2bfloat16_rn(yr);
    const __nv_bfloat16 xl = __float2bfloat16_rn(xr - __bfloat162float(xm)), yl = __float2bfloat16_rn(yr - __bfloat162float(ym));
    hi = (uint32_t)__bfloat16_as_ushort(xh) | ((uint32_t)__bfloat16_as_ushort(yh) << 16);
    mid = (uint32_t)__bfloat16_as_ushort(xm) | ((uint32_t)__bfloat16_as_ushort(ym) << 16);
    lo = (uint32_t)__bfloat16_as_ushort(xl) | ((uint32_t)__bfloat16_as_ushort(yl) << 16);
}

// TC (bfloat16, STAGED, keys that carry their values, head_dim a multiple of 16, values a multiple of 8 up to 256): both
// products on the warp-level tensor cores, the group's heads as the 16 rows of a tile. Scores: q from global memory
// as the row operand, the staged key rows as the column operand, float32 sums. Weighted values: the float32 weights
// as three bfloat16 parts that hold their 24 bits, each multiplied with the same value fragment, so that the weights
// stay float32 in effect.
template <typename T, bool STAGED, int GMAX, bool TC = false> __global__ void __launch_bounds__(AS_THREADS) attention_split_kernel(AttnSplit p) {
    extern __shared__ __align__(16) float as_smem[];
    const int group = p.n_heads / p.n_kv_heads, hd = p.head_dim, vd = p.v_dim;
    float *q_s = as_smem;                      // [group][hd]
    float *p_s = q_s + group * hd;             // [group][128]
    float *red = p_s + group * AS_THREADS;     // [4][group] maxima, then sums
    const int k_pitch = hd * (int)sizeof(T) + 16;
    uint8_t *k_s = (uint8_t *)(red + ((4 * group + 3) & ~3));  // [128][k_pitch]
    uint8_t *v_s = k_s;                                        // [128][vd], once the keys are done with
    __shared__ long long k_off[AS_THREADS], v_off[AS_THREADS];
    const int t = blockIdx.x, kvh = blockIdx.y, part = blockIdx.z, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_wait();
    const int seq = p.token_seq[t];
    if (seq < 0) return;
    const int pos = p.token_pos[t], slot = p.seq_slot[seq];
    int lo, kept, total;
    visible_keys(p, pos, lo, kept, total);
    if (part * AS_THREADS >= total) return;  // the fold knows how many parts a row has
    const int n_valid = total - part * AS_THREADS < AS_THREADS ? total - part * AS_THREADS : AS_THREADS;
    const int number = part * AS_THREADS + tid;
    const bool valid = number < total;
    if (valid) {
        const int j = number < kept ? number : lo + number - kept;
        const int page = cache_page(p.cache, slot, j);
        const int ckv = p.one_kv ? 0 : kvh, cn = p.one_kv ? 1 : p.n_kv_heads;
        v_off[tid] = cache_offset(p.v_cache, page, ckv, cn, j, p.values_in_keys ? hd : vd);
        k_off[tid] = cache_offset(p.cache, page, ckv, cn, j, hd);
    }
    const T *q = (const T *)p.q + (long long)t * p.q_row + (long long)kvh * group * hd;
    for (int e = tid; e < group * hd; e += AS_THREADS) q_s[e] = to_float(q[e]);
    __syncthreads();
    if (STAGED) {
        const uint32_t k_dst = (uint32_t)__cvta_generic_to_shared(k_s);
        const int k_chunks = hd * (int)sizeof(T) / 16;
        for (int e = tid; e < n_valid * k_chunks; e += AS_THREADS) {
            const int r = e / k_chunks, c = e - r * k_chunks;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(k_dst + r * k_pitch + c * 16),
                         "l"((const uint8_t *)((const T *)p.k_pool + k_off[r]) + c * 16) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");  // the keys are here
        __syncthreads();
    }
    float sc[GMAX];
    if (TC) {
        const int row = lane >> 2, k0 = (lane & 3) * 2;
        const __nv_bfloat16 *qg = (const __nv_bfloat16 *)p.q + (long long)t * p.q_row + (long long)kvh * group * hd;
        const bool lower = row < group, upper = row + 8 < group;
        float acc[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
        for (int kk = 0; kk < hd; kk += 16) {
            const uint32_t a0 = lower ? *(const uint32_t *)(qg + (long long)row * hd + kk + k0) : 0u;
            const uint32_t a1 = upper ? *(const uint32_t *)(qg + (long long)(row + 8) * hd + kk + k0) : 0u;
            const uint32_t a2 = lower ? *(const uint32_t *)(qg + (long long)row * hd + kk + k0 + 8) : 0u;
            const uint32_t a3 = upper ? *(const uint32_t *)(qg + (long long)(row + 8) * hd + kk + k0 + 8) : 0u;
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
                const uint8_t *kr = k_s + (warp * 32 + nt * 8 + row) * k_pitch + (kk + k0) * 2;
                as_mma_bf16(acc[nt], a0, a1, a2, a3, *(const uint32_t *)kr, *(const uint32_t *)(kr + 16));
            }
        }
        // the scores to where the weights will stand, [head][key]; every thread then takes its own key's
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
            const int key = warp * 32 + nt * 8 + k0;
            if (lower) p_s[row * AS_THREADS + key] = score_of(p, acc[nt][0]), p_s[row * AS_THREADS + key + 1] = score_of(p, acc[nt][1]);
            if (upper) p_s[(row + 8) * AS_THREADS + key] = score_of(p, acc[nt][2]), p_s[(row + 8) * AS_THREADS + key + 1] = score_of(p, acc[nt][3]);
        }
        __syncthreads();
#pragma unroll
        for (int g = 0; g < GMAX; g++)
            if (g < group) sc[g] = valid ? p_s[g * AS_THREADS + tid] : -INFINITY;
    } else if (valid) {
        const T *k = STAGED ? (const T *)(k_s + tid * k_pitch) : (const T *)p.k_pool + k_off[tid];
#pragma unroll
        for (int g = 0; g < GMAX; g++)
            if (g < group) sc[g] = score_of(p, dot_q<T>(q_s + g * hd, k, hd));
    } else {
#pragma unroll
        for (int g = 0; g < GMAX; g++) sc[g] = -INFINITY;
    }
    // per head: the part's maximum, the weights against it, their sum
#pragma unroll
    for (int g = 0; g < GMAX; g++) {
        if (g < group) {
            const float m = warp_max(sc[g]);
            if (lane == 0) red[warp * group + g] = m;
        }
    }
    __syncthreads();
    if (STAGED && !p.values_in_keys) {  // every thread has read its key row: the values come into the same memory, under the softmax
        const uint32_t v_dst = (uint32_t)__cvta_generic_to_shared(v_s);
        const int v_chunks = vd * (int)sizeof(T) / 16;
        for (int e = tid; e < n_valid * v_chunks; e += AS_THREADS) {
            const int r = e / v_chunks, c = e - r * v_chunks;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(v_dst + (r * v_chunks + c) * 16),
                         "l"((const uint8_t *)((const T *)p.v_pool + v_off[r]) + c * 16) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    float top[GMAX];
#pragma unroll
    for (int g = 0; g < GMAX; g++) {
        if (g < group) {
            top[g] = fmaxf(fmaxf(red[g], red[group + g]), fmaxf(red[2 * group + g], red[3 * group + g]));
            sc[g] = valid ? expf(sc[g] - top[g]) : 0.0f;
            p_s[g * AS_THREADS + tid] = sc[g];
        }
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GMAX; g++) {
        if (g < group) {
            const float s = warp_sum(sc[g]);
            if (lane == 0) red[warp * group + g] = s;
        }
    }
    if (STAGED && !p.values_in_keys) asm volatile("cp.async.wait_group 0;" ::: "memory");  // the values are here
    __syncthreads();
    if (TC) {
        // out[head][column] = sum over the part's keys of weight[head][key] * value[key][column]: a warp has every fourth
        // tile of 8 columns; a key step's weights are split once and meet all of the warp's tiles
        const int row = lane >> 2, k0 = (lane & 3) * 2;
        const bool lower = row < group, upper = row + 8 < group;
        const int n_tiles = vd / 8;
        float c[8][4];
#pragma unroll
        for (int i = 0; i < 8; i++) c[i][0] = c[i][1] = c[i][2] = c[i][3] = 0.0f;
        for (int ks = 0; ks < AS_THREADS; ks += 16) {
            if (ks >= n_valid) break;
            uint32_t ah[4], am[4], al[4];
            const float *pl = p_s + row * AS_THREADS + ks + k0, *pu = p_s + (row + 8) * AS_THREADS + ks + k0;
            as_split3(lower ? pl[0] : 0.0f, lower ? pl[1] : 0.0f, ah[0], am[0], al[0]);
            as_split3(upper ? pu[0] : 0.0f, upper ? pu[1] : 0.0f, ah[1], am[1], al[1]);
            as_split3(lower ? pl[8] : 0.0f, lower ? pl[9] : 0.0f, ah[2], am[2], al[2]);
            as_split3(upper ? pu[8] : 0.0f, upper ? pu[9] : 0.0f, ah[3], am[3], al[3]);
            // keys beyond the part's last hold whatever the memory held: their values are taken as zeros
            const bool in0 = ks + k0 < n_valid, in1 = ks + k0 + 1 < n_valid, in8 = ks + k0 + 8 < n_valid, in9 = ks + k0 + 9 < n_valid;
            const uint8_t *vr = k_s + (ks + k0) * k_pitch + row * 2;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int nt = warp + 4 * i;
                if (nt >= n_tiles) break;
                const uint8_t *v = vr + nt * 16;
                const uint32_t v0 = in0 ? *(const uint16_t *)v : 0u, v1 = in1 ? *(const uint16_t *)(v + k_pitch) : 0u;
                const uint32_t v8 = in8 ? *(const uint16_t *)(v + 8 * k_pitch) : 0u, v9 = in9 ? *(const uint16_t *)(v + 9 * k_pitch) : 0u;
                const uint32_t b0 = v0 | (v1 << 16), b1 = v8 | (v9 << 16);
                as_mma_bf16(c[i], ah[0], ah[1], ah[2], ah[3], b0, b1);
                as_mma_bf16(c[i], am[0], am[1], am[2], am[3], b0, b1);
                as_mma_bf16(c[i], al[0], al[1], al[2], al[3], b0, b1);
            }
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int nt = warp + 4 * i;
            if (nt >= n_tiles) break;
            const int col = nt * 8 + k0;
            if (lower) {
                float *dst = p.parts + (((long long)t * p.n_heads + kvh * group + row) * p.n_parts + part) * (vd + 2);
                dst[col] = c[i][0], dst[col + 1] = c[i][1];
            }
            if (upper) {
                float *dst = p.parts + (((long long)t * p.n_heads + kvh * group + row + 8) * p.n_parts + part) * (vd + 2);
                dst[col] = c[i][2], dst[col + 1] = c[i][3];
            }
        }
        if (tid < group) {
            float *dst = p.parts + (((long long)t * p.n_heads + kvh * group + tid) * p.n_parts + part) * (vd + 2);
#pragma unroll
            for (int g = 0; g < GMAX; g++)
                if (g == tid) dst[vd] = top[g];
            dst[vd + 1] = (red[tid] + red[group + tid]) + (red[2 * group + tid] + red[3 * group + tid]);
        }
        return;
    }
    // weighted values: a thread a value column (two for values beyond 128), every head of the group per value read
    float acc0[GMAX], acc1[GMAX];
#pragma unroll
    for (int g = 0; g < GMAX; g++) acc0[g] = acc1[g] = 0.0f;
    const T *v_base = (const T *)p.v_pool;
    if (tid < vd) {
        for (int jj = 0; jj < n_valid; jj++) {
            const T *v = !STAGED ? v_base + v_off[jj]
                         : p.values_in_keys ? (const T *)(k_s + jj * k_pitch) : (const T *)v_s + (long long)jj * vd;
            const float a = to_float(v[tid]);
#pragma unroll
            for (int g = 0; g < GMAX; g++)
                if (g < group) acc0[g] = fmaf(p_s[g * AS_THREADS + jj], a, acc0[g]);
            if (tid + AS_THREADS < vd) {
                const float b = to_float(v[tid + AS_THREADS]);
#pragma unroll
                for (int g = 0; g < GMAX; g++)
                    if (g < group) acc1[g] = fmaf(p_s[g * AS_THREADS + jj], b, acc1[g]);
            }
        }
    }
#pragma unroll
    for (int g = 0; g < GMAX; g++) {
        if (g < group) {
            float *dst = p.parts + (((long long)t * p.n_heads + kvh * group + g) * p.n_parts + part) * (vd + 2);
            if (tid < vd) dst[tid] = acc0[g];
            if (tid + AS_THREADS < vd) dst[tid + AS_THREADS] = acc1[g];
            if (tid == 0) {
                dst[vd] = top[g];
                dst[vd + 1] = (red[g] + red[group + g]) + (red[2 * group + g] + red[3 * group + g]);
            }
        }
    }
}

// out[t, h] = sum over the row's parts (and the sink) of their weighted values, over the sum of their sums, all
// against the largest maximum. One CTA per (token, head), parts in order.
template <typename T> __global__ void __launch_bounds__(AS_THREADS) attention_fold_kernel(AttnSplit p) {
    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, vd = p.v_dim;
    const float sink = p.sink ? p.sink[h] : -INFINITY;  // a weight: ahead of the wait
    pdl_wait();
    T *out = (T *)p.out + ((long long)t * p.n_heads + h) * vd;
    const int seq = p.token_seq[t];
    if (seq < 0) {
        for (int d = tid; d < vd; d += AS_THREADS) out[d] = from_float<T>(0.0f);
        return;
    }
    int lo, kept, total;
    visible_keys(p, p.token_pos[t], lo, kept, total);
    const int n = (total + AS_THREADS - 1) / AS_THREADS;
    const float *src = p.parts + ((long long)t * p.n_heads + h) * p.n_parts * (vd + 2);
    float top = sink;
    for (int i = 0; i < n; i++) top = fmaxf(top, src[(long long)i * (vd + 2) + vd]);
    float l = p.sink ? expf(sink - top) : 0.0f, a = 0.0f, b = 0.0f;
    for (int i = 0; i < n; i++) {
        const float *part = src + (long long)i * (vd + 2);
        const float w = expf(part[vd] - top);
        l = fmaf(part[vd + 1], w, l);
        if (tid < vd) a = fmaf(part[tid], w, a);
        if (tid + AS_THREADS < vd) b = fmaf(part[tid + AS_THREADS], w, b);
    }
    const float g = p.gate ? 1.0f / (1.0f + expf(-to_float(((const T *)p.gate)[(long long)t * p.ldg + h]))) : 1.0f;
    if (tid < vd) out[tid] = from_float<T>(a / l * g);
    if (tid + AS_THREADS < vd) out[tid + AS_THREADS] = from_float<T>(b / l * g);
}

// max_keys: an upper bound of the keys any row of the step sees (its position + 1, or window + keep_first);
// parts: float32 scratch of at least tokens * heads * ceil(max_keys / 128) * (v_dim + 2).
static int attention_split(int values_in_keys, int chunk, float softcap, const void *q, long long q_row, void *out, int dtype, int n_tokens, int n_heads,
                                   int n_kv_heads, int head_dim, int v_dim, float scale, int window, int keep_first,
                                   const float *sink, const int *token_seq, const int *token_pos, const int *seq_slot,
                                   const void *k_pool, const void *v_pool, const int *page_table, int table_width,
                                   int ring_pages, int pinned_pages, int tokens_per_page, int max_keys, float *parts,
                                   long long parts_floats, const void *gate, long long ldg, void *stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim > AS_MAX_DIM || head_dim % 8 || head_dim < 8) ABK_REFUSE("attention_split: head_dim %d is not a multiple of 8 up to %d", head_dim, AS_MAX_DIM);
    if (v_dim < 1 || v_dim > AS_MAX_DIM) ABK_REFUSE("attention_split: value size %d is not 1 to %d", v_dim, AS_MAX_DIM);
    int one_kv = 0;
    if (values_in_keys && n_kv_heads == 1 && n_heads > AS_MAX_GROUP) {
        // one kv head for more query heads than a CTA takes: the heads go in runs of the largest divisor up to 16,
        // each run a CTA of its own over the same cache rows
        int run = AS_MAX_GROUP;
        while (n_heads % run) run--;
        n_kv_heads = n_heads / run, one_kv = 1;
    }
    if (n_kv_heads < 1 || n_heads % n_kv_heads || n_heads / n_kv_heads > AS_MAX_GROUP)
        ABK_REFUSE("attention_split: %d query heads to %d kv heads (groups of up to %d)", n_heads, n_kv_heads, AS_MAX_GROUP);
    if (n_heads > 65535 || max_keys < 1) ABK_REFUSE("attention_split: %d heads, %d keys", n_heads, max_keys);
    AttnSplit p;
    p.q = q, p.q_row = q_row, p.parts = parts, p.out = out, p.n_heads = n_heads, p.n_kv_heads = n_kv_heads;
    p.head_dim = head_dim, p.v_dim = v_dim, p.scale = scale, p.window = window > 0 ? window : 0;
    p.keep_first = window > 0 && keep_first > 0 ? keep_first : 0, p.sink = sink;
    p.chunk = chunk > 0 ? chunk : 0, p.softcap = softcap > 0.0f ? softcap : 0.0f;
    p.token_seq = token_seq, p.token_pos = token_pos, p.seq_slot = seq_slot, p.k_pool = k_pool, p.v_pool = v_pool;
    p.cache.page_table = page_table, p.cache.table_width = table_width, p.cache.ring_pages = ring_pages;
    p.cache.tokens_per_page = tokens_per_page, p.cache.pinned_pages = pinned_pages;
    p.v_cache = p.cache;
    p.n_parts = (max_keys + AS_THREADS - 1) / AS_THREADS;
    p.values_in_keys = values_in_keys, p.one_kv = one_kv, p.gate = gate, p.ldg = ldg;
    if (values_in_keys && v_dim > head_dim) ABK_REFUSE("attention_split: values of %d inside keys of %d", v_dim, head_dim);
    if (p.n_parts > 65535) ABK_REFUSE("attention_split: %d keys are more than a grid takes", max_keys);
    if ((long long)n_tokens * n_heads * p.n_parts * (v_dim + 2) > parts_floats)
        ABK_REFUSE("attention_split: the scratch memory holds %lld floats, the step needs %lld", parts_floats,
                   (long long)n_tokens * n_heads * p.n_parts * (v_dim + 2));
    const int group = n_heads / n_kv_heads;
    const bool bf = dtype == ABK_BF16;
    const int esize = bf ? 2 : 4;
    const size_t small = (size_t)(group * head_dim + group * AS_THREADS + ((4 * group + 3) & ~3)) * 4;
    size_t rows = (size_t)AS_THREADS * (head_dim * esize + 16);  // the keys' rows, then the values' in the same place
    if (!values_in_keys && rows < (size_t)AS_THREADS * v_dim * esize) rows = (size_t)AS_THREADS * v_dim * esize;
    const size_t staged = small + rows;
    // rows of keys and of values that are whole 16-byte pieces at 16-byte places can be staged in shared memory
    const bool stage = (head_dim * esize) % 16 == 0 && (values_in_keys || (v_dim * esize) % 16 == 0) && staged <= 100 * 1024 &&
                       !(((uintptr_t)k_pool | (uintptr_t)v_pool) & 15);
    const size_t smem = stage ? staged : small;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_tokens, n_kv_heads, p.n_parts), fold(n_tokens, n_heads);
#define SPLIT_LAUNCH(T, STAGED, GMAX, ...)                                                                \
    do {                                                                                                  \
        if (smem + 4096 > 48 * 1024) { /* (the kernel's own 2 KB of static shared memory count too) */    \
            cudaError_t e = abk_allow_shared_memory((const void *)attention_split_kernel<T, STAGED, GMAX, ##__VA_ARGS__>, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                          \
        }                                                                                                 \
        abk_launch(attention_split_kernel<T, STAGED, GMAX, ##__VA_ARGS__>, grid, dim3(AS_THREADS), smem, s, p);         \
    } while (0)
#define SPLIT_BY_GROUP(T, STAGED)                   \
    do {                                            \
        if (group <= 1) SPLIT_LAUNCH(T, STAGED, 1); \
        else if (group <= 2) SPLIT_LAUNCH(T, STAGED, 2); \
        else if (group <= 4) SPLIT_LAUNCH(T, STAGED, 4); \
        else if (group <= 8) SPLIT_LAUNCH(T, STAGED, 8); \
        else SPLIT_LAUNCH(T, STAGED, 16);           \
    } while (0)
    const bool tensor = bf && stage && values_in_keys && head_dim % 16 == 0 && v_dim % 8 == 0 && v_dim <= 256;
    if (tensor) {
        if (group <= 8) SPLIT_LAUNCH(__nv_bfloat16, true, 8, true);
        else SPLIT_LAUNCH(__nv_bfloat16, true, 16, true);
    } else if (bf && stage) SPLIT_BY_GROUP(__nv_bfloat16, true);
    else if (bf) SPLIT_BY_GROUP(__nv_bfloat16, false);
    else if (stage) SPLIT_BY_GROUP(float, true);
    else SPLIT_BY_GROUP(float, false);
#undef SPLIT_BY_GROUP
#undef SPLIT_LAUNCH
    int rc = ABK_LAUNCH_RESULT();
    if (rc) return rc;
    if (bf) abk_launch(attention_fold_kernel<__nv_bfloat16>, fold, dim3(AS_THREADS), 0, s, p);
    else abk_launch(attention_fold_kernel<float>, fold, dim3(AS_THREADS), 0, s, p);
    return ABK_LAUNCH_RESULT();
}

extern "C" int abk_attention_split(const void *q, long long q_row, void *out, int dtype, int n_tokens, int n_heads,
                                   int n_kv_heads, int head_dim, int v_dim, float scale, int window, int keep_first,
                                   const float *sink, const int *token_seq, const int *token_pos, const int *seq_slot,
                                   const void *k_pool, const void *v_pool, const int *page_table, int table_width,
                                   int ring_pages, int pinned_pages, int tokens_per_page, int max_keys, float *parts,
                                   long long parts_floats, int chunk, float softcap, const void *gate, long long ldg,
                                   void *stream) {
    return attention_split(0, chunk, softcap, q, q_row, out, dtype, n_tokens, n_heads, n_kv_heads, head_dim, v_dim, scale, window, keep_first,
                           sink, token_seq, token_pos, seq_slot, k_pool, v_pool, page_table, table_width, ring_pages,
                           pinned_pages, tokens_per_page, max_keys, parts, parts_floats, gate, ldg, stream);
}

// Keys that carry their values (a value is the first v_dim elements of its key row; one pool): attention over shared
// latent rows (csrc/latent.cu), every query head in the one group.
extern "C" int abk_attention_split_values_in_keys(const void *q, long long q_row, void *out, int dtype, int n_tokens,
                                                  int n_heads, int n_kv_heads, int head_dim, int v_dim, float scale,
                                                  const float *sink, const int *token_seq, const int *token_pos,
                                                  const int *seq_slot, const void *k_pool, const int *page_table,
                                                  int table_width, int tokens_per_page, int max_keys, float *parts,
                                                  long long parts_floats, void *stream) {
    return attention_split(1, 0, 0.0f, q, q_row, out, dtype, n_tokens, n_heads, n_kv_heads, head_dim, v_dim, scale, 0, 0, sink,
                           token_seq, token_pos, seq_slot, k_pool, k_pool, page_table, table_width, 0, 0, tokens_per_page,
                           max_keys, parts, parts_floats, nullptr, 0, stream);
}
