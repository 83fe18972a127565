// A matrix memory per head with exponential gates kept in range by a running maximum (the recurrence of an mLSTM
// layer), over every sequence of a step, token by token, from and into the slots' states.
//
// Per head: C [key, value], n [key], m a scalar, all zero at a sequence's start (m too). For a token with q (already
// times key^-1/2 here), k, v and the gates' pre-activations zi, zf:
//     i = cap tanh((zi + bi) / cap)          f = logsigmoid(cap tanh((zf + bf) / cap))
//     m' = max(f + m, i)     C' = e^(f + m - m') C + e^(i - m') k v^T     n' = e^(f + m - m') n + e^(i - m') k
//     o = C'^T q / (max(|n' . q|, e^(-m')) + denom_eps)
// Everything here is float32: the gates, both exponentials, the state and the read-out. q, k and v come in the
// storage type, the pre-activations as float32.
//
// A CTA walks one sequence for one head and MM_COLS value columns. MM_SHARE threads share a column's key channels,
// each with its part of the column's state in registers (and the same part of n, which every column's threads keep a
// copy of: it costs a multiply-add and saves a pass; in the slot's state n and m are kept once per CTA of the head);
// the tokens' rows come MM_TOKENS at a time through shared memory, the gates made on the way in. A sequence that brings no token is left alone. The states are kept [value][key], so a
// column's threads read neighbouring words.
#define ABK_DEFINE_ERROR
#include "common.cuh"

#define MM_SHARE 16    // threads that share a value column
#define MM_COLS 8      // value columns a CTA has (MM_SHARE * MM_COLS threads)
#define MM_TOKENS 16   // tokens staged at a time
#define MM_MAX_PER 16  // key channels a thread holds at most: key sizes up to MM_SHARE * MM_MAX_PER

struct MatrixMemory {
    const void *proj;     // row t at proj + t * ld: q at q_at, k at k_at (heads x key each), v at v_at (heads x value)
    long long ld;
    int q_at, k_at, v_at;
    const float *gates;   // row t at gates + t * ld_gates: zi [heads], then zf [heads]
    long long ld_gates;
    const float *bias_i, *bias_f;  // [heads]
    float cap, denom_eps, q_scale;
    int n_heads, key, value;
    float *state_c;       // [slots][heads][value][key]
    float *state_n;       // [slots][heads][column blocks][key]: every CTA of a head keeps n and m for itself, so that none
    float *state_m;       // [slots][heads][column blocks]       reads what another has already moved on
    float *out;           // [tokens][heads * value], not yet normed
    const int *seq_start, *seq_slot;
};

__device__ __forceinline__ float log_sigmoid_f(float z) {  // -log(1 + e^-z), without overflow
    return z >= 0.0f ? -log1pf(expf(-z)) : z - log1pf(expf(z));
}

template <typename T, int PER>
__global__ void __launch_bounds__(MM_SHARE *MM_COLS) matrix_memory_kernel(MatrixMemory p) {
    extern __shared__ __align__(16) float mm_smem[];
    const int K = p.key, V = p.value;
    float *qs = mm_smem;                       // [MM_TOKENS][K]
    float *ks = qs + MM_TOKENS * K;            // [MM_TOKENS][K]
    float *vs = ks + MM_TOKENS * K;            // [MM_TOKENS][MM_COLS]
    float *gi = vs + MM_TOKENS * MM_COLS;      // [MM_TOKENS]
    float *gf = gi + MM_TOKENS;                // [MM_TOKENS]
    pdl_wait();
    const int seq = blockIdx.z, h = blockIdx.y, col0 = blockIdx.x * MM_COLS;
    const int first = p.seq_start[seq], last = p.seq_start[seq + 1];
    if (last <= first) return;  // the sequence brings no token: its state stays as it is
    const int slot = p.seq_slot[seq];
    const int part = threadIdx.x % MM_SHARE, col = col0 + threadIdx.x / MM_SHARE;
    const bool real = col < V;
    float *cst = p.state_c + (((long long)slot * p.n_heads + h) * V + (real ? col : 0)) * K;
    float *nst = p.state_n + (((long long)slot * p.n_heads + h) * gridDim.x + blockIdx.x) * K;
    float *mst = p.state_m + ((long long)slot * p.n_heads + h) * gridDim.x + blockIdx.x;
    float c[PER], nn[PER];
#pragma unroll
    for (int r = 0; r < PER; r++) {
        const int i = part + r * MM_SHARE;
        c[r] = real && i < K ? cst[i] : 0.0f;
        nn[r] = i < K ? nst[i] : 0.0f;
    }
    float m = *mst;
    const T *proj = (const T *)p.proj;
    for (int t0 = first; t0 < last; t0 += MM_TOKENS) {
        const int nt = min(MM_TOKENS, last - t0);
        __syncthreads();  // the tokens before have been read
        for (int e = threadIdx.x; e < nt * K; e += blockDim.x) {
            const int t = e / K, i = e - t * K;
            const T *row = proj + (long long)(t0 + t) * p.ld;
            qs[t * K + i] = to_float(row[p.q_at + h * K + i]) * p.q_scale;
            ks[t * K + i] = to_float(row[p.k_at + h * K + i]);
        }
        for (int e = threadIdx.x; e < nt * MM_COLS; e += blockDim.x) {
            const int t = e / MM_COLS, j = e - t * MM_COLS;
            vs[e] = col0 + j < V ? to_float(proj[(long long)(t0 + t) * p.ld + p.v_at + h * V + col0 + j]) : 0.0f;
        }
        if (threadIdx.x < nt) {
            const float *g = p.gates + (long long)(t0 + threadIdx.x) * p.ld_gates;
            gi[threadIdx.x] = p.cap * tanhf((g[h] + p.bias_i[h]) / p.cap);
            gf[threadIdx.x] = log_sigmoid_f(p.cap * tanhf((g[p.n_heads + h] + p.bias_f[h]) / p.cap));
        }
        __syncthreads();
        for (int t = 0; t < nt; t++) {
            const float i_t = gi[t], f_t = gf[t];
            const float m_new = fmaxf(f_t + m, i_t);
            const float keep = expf(f_t + m - m_new), write = expf(i_t - m_new);
            m = m_new;
            const float wv = write * vs[t * MM_COLS + threadIdx.x / MM_SHARE];
            float num = 0.0f, dot = 0.0f;
#pragma unroll
            for (int r = 0; r < PER; r++) {
                const int i = part + r * MM_SHARE;
                if (i < K) {
                    const float kk = ks[t * K + i], qq = qs[t * K + i];
                    c[r] = fmaf(keep, c[r], kk * wv);
                    nn[r] = fmaf(keep, nn[r], write * kk);
                    num = fmaf(c[r], qq, num);
                    dot = fmaf(nn[r], qq, dot);
                }
            }
#pragma unroll
            for (int off = MM_SHARE / 2; off > 0; off >>= 1) {
                num += __shfl_xor_sync(0xffffffffu, num, off);
                dot += __shfl_xor_sync(0xffffffffu, dot, off);
            }
            if (part == 0 && real)
                p.out[(long long)(t0 + t) * p.n_heads * V + h * V + col] = num / (fmaxf(fabsf(dot), expf(-m)) + p.denom_eps);
        }
    }
#pragma unroll
    for (int r = 0; r < PER; r++) {
        const int i = part + r * MM_SHARE;
        if (i < K) {
            if (real) cst[i] = c[r];
            if (threadIdx.x < MM_SHARE) nst[i] = nn[r];
        }
    }
    if (threadIdx.x == 0) *mst = m;
}

// ---------------------------------------------------------------- the same recurrence for prompts, in chunks
// A chunk of MC_TOKENS tokens that starts from (C0, n0, m0). With F_t the sum of the chunk's log forget gates up to t,
// a_s = i_s - F_s and M_t = max(m0, max over s <= t of a_s), the recurrence above unrolls to
//     m_t = F_t + M_t      C_t = e^(m0 - M_t) C0 + sum over s <= t of e^(a_s - M_t) k_s v_s^T      (n_t likewise)
// with every exponent at most 0. So a chunk's own sum U = sum_s e^(a_s - A) k_s v_s^T, A = max_s a_s, needs no state
// (chunk_sums: all chunks side by side), the states between chunks follow from the sums alone, an element at a time
// (chunk_prefix: C_end = e^(m0 - M) C0 + e^(A - M) U, M = max(m0, A), m_end = F_end + M; it leaves every chunk's start
// state where its sum was), and a chunk's outputs need its start state and its own rows (chunk_outputs: all chunks side
// by side):  C_t^T q_t = e^(m0 - M_t) C0^T q_t + sum over s <= t of e^(a_s - M_t) (q_t . k_s) v_s.
// Float32 throughout, as token by token; the sums are taken in another order.
#define MC_TOKENS 64
#define MC_VT_SUMS 32   // value columns a CTA of chunk_sums has
#define MC_VT_OUT 64    // value columns a CTA of chunk_outputs has

struct MatrixMemoryChunks {
    MatrixMemory s;
    float *work;        // per (chunk, head): [value][key] (the chunk's sum, then its start state), [key] (n likewise), 4 scalars
    int n_seqs, max_chunks;
};
// scalars of a chunk and head: 0: A (the largest a_s), 1: F_end, 2: m0 (chunk_sums leaves the slot's m at a sequence's
// first chunk, chunk_prefix the others)
__device__ __forceinline__ long long mc_stride(int K, int V) { return (long long)V * K + K + 4; }

// Which sequence and which of its chunks the CTA has; false: none.
__device__ __forceinline__ bool mc_locate(const MatrixMemoryChunks &p, int chunk, int &seq, int &local, int &t0, int &nt) {
    for (int q = 0; q < p.n_seqs; q++) {
        const int first = p.s.seq_start[q], n = p.s.seq_start[q + 1] - first;
        const int chunks = (n + MC_TOKENS - 1) / MC_TOKENS;
        if (chunk < chunks) {
            seq = q, local = chunk, t0 = first + chunk * MC_TOKENS, nt = min(MC_TOKENS, n - chunk * MC_TOKENS);
            return true;
        }
        chunk -= chunks;
    }
    return false;
}

// The chunk's gates and what follows from them alone: a[s] = i_s - F_s, cum[s] = F_s, top[s] = max over r <= s of a_r.
// Called by all threads; the arrays lie in shared memory and are ready after the call.
__device__ __forceinline__ void mc_gates(const MatrixMemory &p, int h, int t0, int nt, float *a, float *cum, float *top) {
    if (threadIdx.x < nt) {
        const float *g = p.gates + (long long)(t0 + threadIdx.x) * p.ld_gates;
        a[threadIdx.x] = p.cap * tanhf((g[h] + p.bias_i[h]) / p.cap);
        cum[threadIdx.x] = log_sigmoid_f(p.cap * tanhf((g[p.n_heads + h] + p.bias_f[h]) / p.cap));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float f_sum = 0.0f, best = -INFINITY;
        for (int t = 0; t < nt; t++) {
            f_sum += cum[t];
            cum[t] = f_sum;
            a[t] -= f_sum;
            best = fmaxf(best, a[t]);
            top[t] = best;
        }
    }
    __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(256) mm_chunk_sums_kernel(MatrixMemoryChunks p) {
    extern __shared__ __align__(16) float mc_smem[];
    const int K = p.s.key, V = p.s.value, h = blockIdx.y, v0 = blockIdx.z * MC_VT_SUMS;
    float *ks = mc_smem;                       // [MC_TOKENS][K], each row times its weight e^(a_s - A)
    float *vs = ks + MC_TOKENS * K;            // [MC_TOKENS][MC_VT_SUMS]
    float *a = vs + MC_TOKENS * MC_VT_SUMS, *cum = a + MC_TOKENS, *top = cum + MC_TOKENS;
    pdl_wait();
    int seq, local, t0, nt;
    if (!mc_locate(p, blockIdx.x, seq, local, t0, nt)) return;
    mc_gates(p.s, h, t0, nt, a, cum, top);
    const float A = top[nt - 1];
    const T *proj = (const T *)p.s.proj;
    for (int e = threadIdx.x; e < MC_TOKENS * K; e += 256) {
        const int t = e / K, i = e - t * K;
        ks[e] = t < nt ? expf(a[t] - A) * to_float(proj[(long long)(t0 + t) * p.s.ld + p.s.k_at + h * K + i]) : 0.0f;
    }
    for (int e = threadIdx.x; e < MC_TOKENS * MC_VT_SUMS; e += 256) {
        const int t = e / MC_VT_SUMS, j = e - t * MC_VT_SUMS;
        vs[e] = t < nt && v0 + j < V ? to_float(proj[(long long)(t0 + t) * p.s.ld + p.s.v_at + h * V + v0 + j]) : 0.0f;
    }
    __syncthreads();
    float *work = p.work + ((long long)blockIdx.x * p.s.n_heads + h) * mc_stride(K, V);
    // a thread: one key channel and four value columns at a time
    for (int e = threadIdx.x; e < (MC_VT_SUMS / 4) * K; e += 256) {
        const int vg = e / K, i = e - vg * K;
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int t = 0; t < nt; t++) {
            const float kk = ks[t * K + i];
            const float4 vv = *(const float4 *)(vs + t * MC_VT_SUMS + vg * 4);
            acc[0] = fmaf(kk, vv.x, acc[0]), acc[1] = fmaf(kk, vv.y, acc[1]);
            acc[2] = fmaf(kk, vv.z, acc[2]), acc[3] = fmaf(kk, vv.w, acc[3]);
        }
#pragma unroll
        for (int u = 0; u < 4; u++)
            if (v0 + vg * 4 + u < V) work[(long long)(v0 + vg * 4 + u) * K + i] = acc[u];
    }
    if (blockIdx.z == 0) {
        for (int i = threadIdx.x; i < K; i += 256) {
            float acc = 0.0f;
            for (int t = 0; t < nt; t++) acc += ks[t * K + i];
            work[(long long)V * K + i] = acc;
        }
        if (threadIdx.x == 0) {
            float *scalars = work + (long long)V * K + K;
            scalars[0] = A, scalars[1] = cum[nt - 1];
            if (local == 0) {  // the slot's m, out of the way of chunk_prefix's last write
                const int blocks = (V + MM_COLS - 1) / MM_COLS;
                scalars[2] = p.s.state_m[((long long)p.s.seq_slot[seq] * p.s.n_heads + h) * blocks];
            }
        }
    }
}

// A thread walks one element of one head's state along a sequence's chunks.
__global__ void __launch_bounds__(256) mm_chunk_prefix_kernel(MatrixMemoryChunks p) {
    const int K = p.s.key, V = p.s.value, h = blockIdx.y, seq = blockIdx.z;
    pdl_wait();
    int chunk0 = 0;
    for (int q = 0; q < seq; q++) chunk0 += (p.s.seq_start[q + 1] - p.s.seq_start[q] + MC_TOKENS - 1) / MC_TOKENS;
    const int n = p.s.seq_start[seq + 1] - p.s.seq_start[seq], chunks = (n + MC_TOKENS - 1) / MC_TOKENS;
    if (chunks == 0) return;
    const long long e = (long long)blockIdx.x * 256 + threadIdx.x;   // below V * K: C; the next K: n
    if (e >= (long long)V * K + K) return;
    const int slot = p.s.seq_slot[seq], blocks = (V + MM_COLS - 1) / MM_COLS;
    const bool is_n = e >= (long long)V * K;
    float *own = is_n ? p.s.state_n + ((long long)slot * p.s.n_heads + h) * blocks * K + (e - (long long)V * K)
                      : p.s.state_c + ((long long)slot * p.s.n_heads + h) * V * K + e;
    const long long stride = mc_stride(K, V);
    float *work = p.work + ((long long)chunk0 * p.s.n_heads + h) * stride;
    float x = *own, m = work[(long long)V * K + K + 2];
    const long long step = stride * p.s.n_heads;
    for (int c0 = 0; c0 < chunks; c0 += 4, work += 4 * step) {  // four chunks' loads in flight together
        float sum[4], A[4], F[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const bool real = c0 + u < chunks;
            const float *w = work + (real ? u : 0) * step;
            sum[u] = w[e], A[u] = w[(long long)V * K + K], F[u] = w[(long long)V * K + K + 1];
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            if (c0 + u >= chunks) break;
            float *w = work + u * step;
            const float M = fmaxf(m, A[u]);
            w[e] = x;                                                      // the chunk's start state, where its sum was
            x = fmaf(expf(m - M), x, expf(A[u] - M) * sum[u]);
            if (e == 0 && c0 + u > 0) w[(long long)V * K + K + 2] = m;     // (the first chunk's was left by chunk_sums)
            m = F[u] + M;
        }
    }
    if (is_n) {
        for (int b = 0; b < blocks; b++) own[(long long)b * K] = x;
    } else {
        *own = x;
    }
    if (e == 0) {
        float *mst = p.s.state_m + ((long long)slot * p.s.n_heads + h) * blocks;
        for (int b = 0; b < blocks; b++) mst[b] = m;
    }
}

// acc[u] += q . rows[(sg + 4 * (j0 + u))] for u < 4: a token's row against four rows a pitch apart. VEC: the key size is a
// multiple of 4 and the pitch K + 4, so both sides come as 16-byte pieces (a fifth of the loads a multiply-add).
template <bool VEC>
__device__ __forceinline__ void mc_dots(const float *q, const float *rows, int KP, int K, float *acc) {
    if (VEC) {
        for (int i = 0; i < K; i += 4) {
            const float4 qq = *(const float4 *)(q + i);
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const float4 kk = *(const float4 *)(rows + (long long)u * 4 * KP + i);
                acc[u] = fmaf(qq.w, kk.w, fmaf(qq.z, kk.z, fmaf(qq.y, kk.y, fmaf(qq.x, kk.x, acc[u]))));
            }
        }
    } else {
        for (int i = 0; i < K; i++) {
            const float qq = q[i];
#pragma unroll
            for (int u = 0; u < 4; u++) acc[u] = fmaf(qq, rows[(long long)u * 4 * KP + i], acc[u]);
        }
    }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(256) mm_chunk_outputs_kernel(MatrixMemoryChunks p) {
    extern __shared__ __align__(16) float mc_smem[];
    const int K = p.s.key, V = p.s.value, h = blockIdx.y, v0 = blockIdx.z * MC_VT_OUT, KP = VEC ? K + 4 : K + 1;
    float *qs = mc_smem;                          // [MC_TOKENS][KP]
    float *ks = qs + MC_TOKENS * KP;              // [MC_TOKENS][KP]; later the start state's columns [MC_VT_OUT][KP]
    float *ps = ks + MC_TOKENS * KP;              // [MC_TOKENS][MC_TOKENS + 1]: e^(a_s - M_t) (q_t . k_s), 0 for s > t
    float *vs = ps + MC_TOKENS * (MC_TOKENS + 1); // [MC_TOKENS][MC_VT_OUT]
    float *n0 = vs + MC_TOKENS * MC_VT_OUT;       // [K]
    float *a = n0 + K, *cum = a + MC_TOKENS, *top = cum + MC_TOKENS, *qn = top + MC_TOKENS;
    pdl_wait();
    int seq, local, t0, nt;
    if (!mc_locate(p, blockIdx.x, seq, local, t0, nt)) return;
    mc_gates(p.s, h, t0, nt, a, cum, top);
    const float *work = p.work + ((long long)blockIdx.x * p.s.n_heads + h) * mc_stride(K, V);
    const float m0 = work[(long long)V * K + K + 2];
    const T *proj = (const T *)p.s.proj;
    for (int e = threadIdx.x; e < MC_TOKENS * K; e += 256) {
        const int t = e / K, i = e - t * K;
        const T *row = proj + (long long)(t0 + t) * p.s.ld;
        qs[t * KP + i] = t < nt ? to_float(row[p.s.q_at + h * K + i]) * p.s.q_scale : 0.0f;
        ks[t * KP + i] = t < nt ? to_float(row[p.s.k_at + h * K + i]) : 0.0f;
    }
    for (int e = threadIdx.x; e < MC_TOKENS * MC_VT_OUT; e += 256) {
        const int t = e / MC_VT_OUT, j = e - t * MC_VT_OUT;
        vs[e] = t < nt && v0 + j < V ? to_float(proj[(long long)(t0 + t) * p.s.ld + p.s.v_at + h * V + v0 + j]) : 0.0f;
    }
    for (int i = threadIdx.x; i < K; i += 256) n0[i] = work[(long long)V * K + i];
    __syncthreads();
    const int t = threadIdx.x >> 2, sg = threadIdx.x & 3;   // a thread: one token's row, every fourth column
    const float M_t = t < nt ? fmaxf(m0, top[t]) : 0.0f;
    // the chunk's own scores, weighted
    for (int j0 = 0; j0 < MC_TOKENS / 4; j0 += 4) {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (sg + 4 * j0 <= t && t < nt) mc_dots<VEC>(qs + t * KP, ks + (sg + 4 * j0) * KP, KP, K, acc);
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int s = sg + 4 * (j0 + u);
            ps[t * (MC_TOKENS + 1) + s] = s <= t && t < nt ? expf(a[s] - M_t) * acc[u] : 0.0f;
        }
    }
    if (threadIdx.x < nt) {  // q_t . n0
        float acc = 0.0f;
        for (int i = 0; i < K; i++) acc = fmaf(qs[threadIdx.x * KP + i], n0[i], acc);
        qn[threadIdx.x] = acc;
    }
    __syncthreads();  // the keys have been read: the start state's columns take their place
    for (int e = threadIdx.x; e < MC_VT_OUT * K; e += 256) {
        const int j = e / K, i = e - j * K;
        ks[j * KP + i] = v0 + j < V ? work[(long long)(v0 + j) * K + i] : 0.0f;
    }
    __syncthreads();
    if (t >= nt) return;
    const float e_t = expf(m0 - M_t);
    float dot = e_t * qn[t];
    for (int s = 0; s <= t; s++) dot += ps[t * (MC_TOKENS + 1) + s];
    const float den = fmaxf(fabsf(dot), expf(-(cum[t] + M_t))) + p.s.denom_eps;
    float *out = p.s.out + (long long)(t0 + t) * p.s.n_heads * V + h * V + v0;
    for (int j0 = 0; j0 < MC_VT_OUT / 4; j0 += 4) {
        if (v0 + sg + 4 * j0 >= V) break;
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        mc_dots<VEC>(qs + t * KP, ks + (sg + 4 * j0) * KP, KP, K, acc);
#pragma unroll
        for (int u = 0; u < 4; u++) acc[u] *= e_t;
        for (int s = 0; s <= t; s++) {
            const float w = ps[t * (MC_TOKENS + 1) + s];
#pragma unroll
            for (int u = 0; u < 4; u++) acc[u] = fmaf(w, vs[s * MC_VT_OUT + sg + 4 * (j0 + u)], acc[u]);
        }
#pragma unroll
        for (int u = 0; u < 4; u++)
            if (v0 + sg + 4 * (j0 + u) < V) out[sg + 4 * (j0 + u)] = acc[u] / den;
    }
}

// The recurrence of a step that brings prompts, in chunks of 64 tokens. work: float32 scratch of at least
// max_chunks * heads * (value * key + key + 4), max_chunks >= ceil(tokens / 64) + sequences.
extern "C" int abk_matrix_memory_chunks(const void *proj, long long ld, int dtype, int q_at, int k_at, int v_at,
                                        const float *gates, long long ld_gates, const float *bias_i, const float *bias_f,
                                        float cap, float denom_eps, float q_scale, int n_heads, int key, int value,
                                        float *state_c, float *state_n, float *state_m, float *out, const int *seq_start,
                                        const int *seq_slot, int n_seqs, int max_chunks, float *work, long long work_floats,
                                        void *stream) {
    if (n_seqs <= 0 || max_chunks <= 0) return 0;
    if (key < 1 || key > MM_SHARE * MM_MAX_PER)
        ABK_REFUSE("matrix_memory_chunks: %d key channels a head are not 1 to %d", key, MM_SHARE * MM_MAX_PER);
    if (value < 1 || n_heads < 1 || n_heads > 65535 || n_seqs > 65535 || !(cap > 0.0f))
        ABK_REFUSE("matrix_memory_chunks: %d heads of %d values, %d sequences, a gate cap of %g", n_heads, value, n_seqs, cap);
    const long long stride = (long long)value * key + key + 4;
    if ((long long)max_chunks * n_heads * stride > work_floats)
        ABK_REFUSE("matrix_memory_chunks: the scratch memory holds %lld floats, the step needs %lld", work_floats,
                   (long long)max_chunks * n_heads * stride);
    MatrixMemoryChunks p;
    p.s.proj = proj, p.s.ld = ld, p.s.q_at = q_at, p.s.k_at = k_at, p.s.v_at = v_at, p.s.gates = gates, p.s.ld_gates = ld_gates;
    p.s.bias_i = bias_i, p.s.bias_f = bias_f, p.s.cap = cap, p.s.denom_eps = denom_eps, p.s.q_scale = q_scale;
    p.s.n_heads = n_heads, p.s.key = key, p.s.value = value, p.s.state_c = state_c, p.s.state_n = state_n, p.s.state_m = state_m;
    p.s.out = out, p.s.seq_start = seq_start, p.s.seq_slot = seq_slot;
    p.work = work, p.n_seqs = n_seqs, p.max_chunks = max_chunks;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem_a = (size_t)(MC_TOKENS * key + MC_TOKENS * MC_VT_SUMS + 3 * MC_TOKENS) * sizeof(float);
    const bool vec = key % 4 == 0;
    const size_t smem_c = (size_t)(2 * MC_TOKENS * (key + (vec ? 4 : 1)) + MC_TOKENS * (MC_TOKENS + 1) + MC_TOKENS * MC_VT_OUT +
                                   key + 4 * MC_TOKENS) * sizeof(float);
    const unsigned sums_tiles = (value + MC_VT_SUMS - 1) / MC_VT_SUMS, out_tiles = (value + MC_VT_OUT - 1) / MC_VT_OUT;
    const unsigned elements = (unsigned)(((long long)value * key + key + 255) / 256);
#define MC_LAUNCH(T)                                                                                             \
    do {                                                                                                         \
        cudaError_t e = abk_allow_shared_memory((const void *)mm_chunk_sums_kernel<T>, (int)smem_a);             \
        if (e == cudaSuccess) e = abk_allow_shared_memory((const void *)mm_chunk_outputs_kernel<T, true>, (int)smem_c); \
        if (e == cudaSuccess) e = abk_allow_shared_memory((const void *)mm_chunk_outputs_kernel<T, false>, (int)smem_c); \
        if (e != cudaSuccess) return (int)e;                                                                     \
        abk_launch(mm_chunk_sums_kernel<T>, dim3(max_chunks, n_heads, sums_tiles), dim3(256), smem_a, s, p);     \
        abk_launch(mm_chunk_prefix_kernel, dim3(elements, n_heads, n_seqs), dim3(256), 0, s, p);                 \
        if (vec) abk_launch(mm_chunk_outputs_kernel<T, true>, dim3(max_chunks, n_heads, out_tiles), dim3(256), smem_c, s, p); \
        else abk_launch(mm_chunk_outputs_kernel<T, false>, dim3(max_chunks, n_heads, out_tiles), dim3(256), smem_c, s, p);    \
    } while (0)
    if (dtype == ABK_BF16) MC_LAUNCH(__nv_bfloat16);
    else MC_LAUNCH(float);
#undef MC_LAUNCH
    return ABK_LAUNCH_RESULT();
}

// How many copies of n and m a head's state holds: one per CTA that walks the head.
extern "C" int abk_matrix_memory_blocks(int value) { return (value + MM_COLS - 1) / MM_COLS; }

extern "C" int abk_matrix_memory(const void *proj, long long ld, int dtype, int q_at, int k_at, int v_at, const float *gates,
                                 long long ld_gates, const float *bias_i, const float *bias_f, float cap, float denom_eps,
                                 float q_scale, int n_heads, int key, int value, float *state_c, float *state_n,
                                 float *state_m, float *out, const int *seq_start, const int *seq_slot, int n_seqs,
                                 void *stream) {
    if (n_seqs <= 0) return 0;
    if (key < 1 || key > MM_SHARE * MM_MAX_PER)
        ABK_REFUSE("matrix_memory: %d key channels a head are not 1 to %d", key, MM_SHARE * MM_MAX_PER);
    if (value < 1 || n_heads < 1 || n_heads > 65535 || n_seqs > 65535 || !(cap > 0.0f))
        ABK_REFUSE("matrix_memory: %d heads of %d values, %d sequences, a gate cap of %g", n_heads, value, n_seqs, cap);
    MatrixMemory p;
    p.proj = proj, p.ld = ld, p.q_at = q_at, p.k_at = k_at, p.v_at = v_at, p.gates = gates, p.ld_gates = ld_gates;
    p.bias_i = bias_i, p.bias_f = bias_f, p.cap = cap, p.denom_eps = denom_eps, p.q_scale = q_scale;
    p.n_heads = n_heads, p.key = key, p.value = value, p.state_c = state_c, p.state_n = state_n, p.state_m = state_m;
    p.out = out, p.seq_start = seq_start, p.seq_slot = seq_slot;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((value + MM_COLS - 1) / MM_COLS, n_heads, n_seqs), block(MM_SHARE * MM_COLS);
    const size_t smem = (size_t)(2 * MM_TOKENS * key + MM_TOKENS * MM_COLS + 2 * MM_TOKENS) * sizeof(float);
    const int per = (key + MM_SHARE - 1) / MM_SHARE;
#define MM_LAUNCH(T)                                                                    \
    do {                                                                                \
        if (per <= 2) abk_launch(matrix_memory_kernel<T, 2>, grid, block, smem, s, p);  \
        else if (per <= 4) abk_launch(matrix_memory_kernel<T, 4>, grid, block, smem, s, p); \
        else if (per <= 8) abk_launch(matrix_memory_kernel<T, 8>, grid, block, smem, s, p); \
        else abk_launch(matrix_memory_kernel<T, 16>, grid, block, smem, s, p);          \
    } while (0)
    if (dtype == ABK_BF16) MM_LAUNCH(__nv_bfloat16);
    else MM_LAUNCH(float);
#undef MM_LAUNCH
    return ABK_LAUNCH_RESULT();
}
