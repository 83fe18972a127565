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
