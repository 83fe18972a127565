// Latent attention: what stands around the attention kernels when keys and values are kept as one low-rank
// latent row per token that all heads share.
//
// A token's cache row is [c | r | 0...]: c (rank elements) is the normed down-projection, r (rot elements) one
// rotated key part shared by the heads, zeros up to the row's padded size. Head h's key is [U_h c | r] and its value
// V_h c. The scores need no key of full size: (U_h c) . q = c . (U_h^T q), so a query head is carried into the
// latent space once, [U_h^T q_plain | q_rotated], and attention runs over the cache rows themselves with one kv
// head whose values are the first `rank` elements of its keys; V_h is applied to the weighted sum of latents.
//
//   latent_prep   per token: c = w * x / sqrt(mean(x^2) + eps) over the first `rank` columns of the down-projection,
//                 the rotation of the shared key part and of every query head's rotated part (pairs (2i, 2i+1) or (i, i + rot_dims / 2),
//                 angle table [position][rot_dims / 2]; elements beyond rot_dims pass unchanged), the cache write,
//                 and the query parts put where the attention kernel wants them.
//   head_product  out[t, h, :] = W[h] x[t, h, :] for every head: a product per head with a matrix of its own
//                 (U_h^T on the plain query part, V_h on the weighted latents), float32 sums in a fixed order.
//   latent_rows   the cache rows of the step's own tokens, gathered into consecutive rows (for a prompt whose keys
//                 and values are made in full size from the latents).
//   spread_shared a step's shared rotated key part copied behind every head's plain key part.
#define ABK_DEFINE_ERROR
#include "common.cuh"

struct LatentPrep {
    const void *proj;    // row t at proj + t * ldp: query heads [heads][dim + rot] from column 0, the down-projection
    long long ldp;       // [rank + rot] from column down_at
    int down_at;
    int n_heads, dim, rot, rank, rot_dims;
    int interleaved;     // pairs (2i, 2i+1) of the rotated dimensions; 0: pairs (i, i + rot_dims / 2)
    const float *norm_w;  // [rank]
    float eps;
    const float *cos, *sin;  // [positions][rot_dims / 2]
    void *q_dst;          // head h of row t at q_dst + t * ldq + h * q_head: its rotated part goes to + q_rot_at,
    long long ldq;        // its plain part (copy_plain) to + 0; what lies beyond q_rot_at + rot in a head is zeroed
    int q_head, q_rot_at, copy_plain;
    void *pool;           // cache rows [pages][1][tokens_per_page][row]; null: nothing is written (another entry's cache)
    int row;
    PagedCache cache;
    const int *token_seq, *token_pos, *seq_slot;
};

template <typename T> __global__ void __launch_bounds__(128) latent_prep_kernel(LatentPrep p) {
    __shared__ float scratch[33];
    const int t = blockIdx.x, tid = threadIdx.x;
    pdl_wait();
    const int seq = p.token_seq[t];
    if (seq < 0) return;
    const int pos = p.token_pos[t], half = p.rot_dims / 2;
    const T *src = (const T *)p.proj + (long long)t * p.ldp;
    const float *cs = p.cos + (long long)pos * half, *sn = p.sin + (long long)pos * half;
    if (p.pool) {
        const T *down = src + p.down_at;
        float ss = 0.0f;
        for (int i = tid; i < p.rank; i += 128) {
            const float v = to_float(down[i]);
            ss = fmaf(v, v, ss);
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)p.rank + p.eps);
        const int page = cache_page(p.cache, p.seq_slot[seq], pos);
        T *dst = (T *)p.pool + cache_offset(p.cache, page, 0, 1, pos, p.row);
        for (int i = tid; i < p.rank; i += 128) dst[i] = from_float<T>(to_float(down[i]) * inv * p.norm_w[i]);
        for (int i = tid; i < half; i += 128) {
            const int ia = p.interleaved ? 2 * i : i, ib = p.interleaved ? 2 * i + 1 : i + half;
            const float u = to_float(down[p.rank + ia]), v = to_float(down[p.rank + ib]);
            dst[p.rank + ia] = from_float<T>(u * cs[i] - v * sn[i]);
            dst[p.rank + ib] = from_float<T>(v * cs[i] + u * sn[i]);
        }
        for (int i = p.rot_dims + tid; i < p.rot; i += 128) dst[p.rank + i] = down[p.rank + i];
        for (int i = p.rank + p.rot + tid; i < p.row; i += 128) dst[i] = from_float<T>(0.0f);
    }
    T *q_out = (T *)p.q_dst + (long long)t * p.ldq;
    const int per_head = p.dim + p.rot;
    for (int e = tid; e < p.n_heads * half; e += 128) {
        const int h = e / half, i = e - h * half;
        const T *q = src + (long long)h * per_head + p.dim;
        const int ia = p.interleaved ? 2 * i : i, ib = p.interleaved ? 2 * i + 1 : i + half;
        const float u = to_float(q[ia]), v = to_float(q[ib]);
        T *d = q_out + (long long)h * p.q_head + p.q_rot_at;
        d[ia] = from_float<T>(u * cs[i] - v * sn[i]);
        d[ib] = from_float<T>(v * cs[i] + u * sn[i]);
    }
    const int rest = p.rot - p.rot_dims, tail = p.q_head - p.q_rot_at - p.rot;
    for (int e = tid; e < p.n_heads * rest; e += 128) {
        const int h = e / rest, i = p.rot_dims + e % rest;
        q_out[(long long)h * p.q_head + p.q_rot_at + i] = src[(long long)h * per_head + p.dim + i];
    }
    for (int e = tid; e < p.n_heads * tail; e += 128) {
        const int h = e / tail, i = p.q_rot_at + p.rot + e % tail;
        q_out[(long long)h * p.q_head + i] = from_float<T>(0.0f);
    }
    if (p.copy_plain)
        for (int e = tid; e < p.n_heads * p.dim; e += 128) {
            const int h = e / p.dim, i = e - h * p.dim;
            q_out[(long long)h * p.q_head + i] = src[(long long)h * per_head + i];
        }
}

extern "C" int abk_latent_prep(const void *proj, long long ldp, int dtype, int n_tokens, int down_at, int n_heads, int dim,
                               int rot, int rank, int rot_dims, int interleaved, const float *norm_w, float eps, const float *cos,
                               const float *sin, void *q_dst, long long ldq, int q_head, int q_rot_at, int copy_plain,
                               void *pool, int row, const int *page_table, int table_width, int tokens_per_page,
                               const int *token_seq, const int *token_pos, const int *seq_slot, void *stream) {
    if (n_tokens <= 0) return 0;
    if (rot_dims < 0 || rot_dims % 2 || rot_dims > rot) ABK_REFUSE("latent_prep: %d rotated dimensions of %d", rot_dims, rot);
    if (q_head < q_rot_at + rot || (pool && row < rank + rot))
        ABK_REFUSE("latent_prep: a head of %d or a cache row of %d does not hold %d + %d elements", q_head, row, rank, rot);
    LatentPrep p;
    p.proj = proj, p.ldp = ldp, p.down_at = down_at, p.n_heads = n_heads, p.dim = dim, p.rot = rot, p.rank = rank;
    p.rot_dims = rot_dims, p.interleaved = interleaved, p.norm_w = norm_w, p.eps = eps, p.cos = cos, p.sin = sin, p.q_dst = q_dst, p.ldq = ldq;
    p.q_head = q_head, p.q_rot_at = q_rot_at, p.copy_plain = copy_plain, p.pool = pool, p.row = row;
    p.cache.page_table = page_table, p.cache.table_width = table_width, p.cache.ring_pages = 0;
    p.cache.tokens_per_page = tokens_per_page, p.cache.pinned_pages = 0;
    p.token_seq = token_seq, p.token_pos = token_pos, p.seq_slot = seq_slot;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == ABK_BF16) abk_launch(latent_prep_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(128), 0, s, p);
    else abk_launch(latent_prep_kernel<float>, dim3(n_tokens), dim3(128), 0, s, p);
    return ABK_LAUNCH_RESULT();
}

// ---------------------------------------------------------------- the norm of a run of columns
// dst[t, i] = w[i] * src[t, i] / sqrt(mean_i(src[t, i]^2) + eps) for i < count: a latent normed where it lies among the
// columns of a product's output (rows of any pitch; dst may be src).
template <typename T>
__global__ void __launch_bounds__(128) columns_norm_kernel(const T *src, long long lds, T *dst, long long ldd, int count,
                                                           const float *w, float eps) {
    __shared__ float scratch[33];
    const long long t = blockIdx.x;
    pdl_wait();
    const T *s = src + t * lds;
    T *d = dst + t * ldd;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < count; i += 128) {
        const float v = to_float(s[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)count + eps);
    for (int i = threadIdx.x; i < count; i += 128) d[i] = from_float<T>(to_float(s[i]) * inv * w[i]);
}

extern "C" int abk_columns_norm(const void *src, long long lds, void *dst, long long ldd, int dtype, int n_tokens, int count,
                                const float *w, float eps, void *stream) {
    if (n_tokens <= 0 || count <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == ABK_BF16)
        abk_launch(columns_norm_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(128), 0, s, (const __nv_bfloat16 *)src, lds,
                   (__nv_bfloat16 *)dst, ldd, count, w, eps);
    else
        abk_launch(columns_norm_kernel<float>, dim3(n_tokens), dim3(128), 0, s, (const float *)src, lds, (float *)dst, ldd, count, w, eps);
    return ABK_LAUNCH_RESULT();
}

// ---------------------------------------------------------------- a product per head
#define HP_ROWS 8      // rows of x a CTA holds in shared memory
#define HP_PER_WARP 4  // output features a warp makes, one after the other

template <typename T>
__global__ void __launch_bounds__(128) head_product_kernel(const T *__restrict__ x, long long ldx, int x_head,
                                                           const T *__restrict__ w, T *__restrict__ out, long long ldo,
                                                           int o_head, int n, int in, int outs, const T *__restrict__ gate,
                                                           long long ldg) {
    extern __shared__ __align__(16) float hp_x[];  // [HP_ROWS][in4], in4 = in rounded up to 4
    const int h = blockIdx.y, r0 = blockIdx.z * HP_ROWS, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rows = n - r0 < HP_ROWS ? n - r0 : HP_ROWS;
    pdl_wait();
    const int in4 = (in + 3) & ~3;
    for (int e = threadIdx.x; e < HP_ROWS * in; e += 128) {
        const int r = e / in, i = e - r * in;
        hp_x[r * in4 + i] = r < rows ? to_float(x[(long long)(r0 + r) * ldx + (long long)h * x_head + i]) : 0.0f;
    }
    __syncthreads();
    const bool vec = in % (16 / (int)sizeof(T)) == 0 && ((uintptr_t)w & 15) == 0;
    for (int u = 0; u < HP_PER_WARP; u++) {
        const int o = (blockIdx.x * 4 + warp) * HP_PER_WARP + u;
        if (o >= outs) break;
        const T *wr = w + ((long long)h * outs + o) * in;
        // a row of the matrix against each of the CTA's rows of x: the lanes' shares of the sums, each in its own order
        for (int r = 0; r < rows; r++) {
            float acc = 0.0f;
            lane_dots<1>(wr, 0, hp_x + r * in4, in, lane, vec, &acc);
            acc = warp_sum(acc);
            if (lane == 0) {
                if (gate) acc *= 1.0f / (1.0f + expf(-to_float(gate[(long long)(r0 + r) * ldg + h])));  // a gate per head
                out[(long long)(r0 + r) * ldo + (long long)h * o_head + o] = from_float<T>(acc);
            }
        }
    }
}

// x element (t, h, i) at x + t * ldx + h * x_head + i; w [heads][outs][in]; out element (t, h, o) at
// out + t * ldo + h * o_head + o. x, w and out are of one type. gate (null: none): head h of row t is multiplied by
// sigmoid(gate[t * ldg + h]).
extern "C" int abk_head_product(const void *x, long long ldx, int x_head, const void *w, void *out, long long ldo,
                                int o_head, int dtype, int n, int heads, int in, int outs, const void *gate, long long ldg,
                                void *stream) {
    if (n <= 0 || heads <= 0 || outs <= 0) return 0;
    if (in < 1 || in > 4096) ABK_REFUSE("head_product: an inner size of %d is not 1 to 4096", in);
    const long long row_tiles = ((long long)n + HP_ROWS - 1) / HP_ROWS;
    if (heads > 65535 || row_tiles > 65535) ABK_REFUSE("head_product: %d heads, %d rows are more than a grid takes", heads, n);
    dim3 grid((outs + 4 * HP_PER_WARP - 1) / (4 * HP_PER_WARP), heads, (unsigned)row_tiles);
    const size_t smem = (size_t)HP_ROWS * ((in + 3) & ~3) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == ABK_BF16) {
        if (smem > 48 * 1024) {
            cudaError_t e = abk_allow_shared_memory((const void *)head_product_kernel<__nv_bfloat16>, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        abk_launch(head_product_kernel<__nv_bfloat16>, grid, dim3(128), smem, s, (const __nv_bfloat16 *)x, ldx, x_head,
                   (const __nv_bfloat16 *)w, (__nv_bfloat16 *)out, ldo, o_head, n, in, outs, (const __nv_bfloat16 *)gate, ldg);
    } else {
        if (smem > 48 * 1024) {
            cudaError_t e = abk_allow_shared_memory((const void *)head_product_kernel<float>, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        abk_launch(head_product_kernel<float>, grid, dim3(128), smem, s, (const float *)x, ldx, x_head, (const float *)w,
                   (float *)out, ldo, o_head, n, in, outs, (const float *)gate, ldg);
    }
    return ABK_LAUNCH_RESULT();
}

// ---------------------------------------------------------------- a prompt's keys and values in full size
// rows[t] = the first `count` elements of the cache row of token t (its sequence's slot, its position).
template <typename T>
__global__ void __launch_bounds__(128) latent_rows_kernel(const T *pool, int row, PagedCache cache, T *rows, long long ld,
                                                          int count, const int *token_seq, const int *token_pos,
                                                          const int *seq_slot) {
    const int t = blockIdx.x;
    pdl_wait();
    const int seq = token_seq[t];
    T *dst = rows + (long long)t * ld;
    if (seq < 0) {
        for (int i = threadIdx.x; i < count; i += 128) dst[i] = from_float<T>(0.0f);
        return;
    }
    const int pos = token_pos[t];
    const T *src = pool + cache_offset(cache, cache_page(cache, seq_slot[seq], pos), 0, 1, pos, row);
    for (int i = threadIdx.x; i < count; i += 128) dst[i] = src[i];
}

extern "C" int abk_latent_rows(const void *pool, int row, const int *page_table, int table_width, int tokens_per_page,
                               void *rows, long long ld, int count, int dtype, int n_tokens, const int *token_seq,
                               const int *token_pos, const int *seq_slot, void *stream) {
    if (n_tokens <= 0) return 0;
    if (count > row || count > ld) ABK_REFUSE("latent_rows: %d elements of a cache row of %d into rows of %lld", count, row, ld);
    PagedCache c;
    c.page_table = page_table, c.table_width = table_width, c.ring_pages = 0, c.tokens_per_page = tokens_per_page;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == ABK_BF16)
        abk_launch(latent_rows_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(128), 0, s, (const __nv_bfloat16 *)pool, row, c,
                   (__nv_bfloat16 *)rows, ld, count, token_seq, token_pos, seq_slot);
    else
        abk_launch(latent_rows_kernel<float>, dim3(n_tokens), dim3(128), 0, s, (const float *)pool, row, c, (float *)rows,
                   ld, count, token_seq, token_pos, seq_slot);
    return ABK_LAUNCH_RESULT();
}

// keys[t, h, at + i] = shared[t, i] for every head h and i < count (keys: rows of ldk elements, heads of k_head).
template <typename T>
__global__ void __launch_bounds__(128) spread_shared_kernel(const T *shared, long long lds, T *keys, long long ldk, int k_head,
                                                            int at, int count, int heads) {
    const int t = blockIdx.x;
    pdl_wait();
    for (int e = threadIdx.x; e < heads * count; e += 128) {
        const int h = e / count, i = e - h * count;
        keys[(long long)t * ldk + (long long)h * k_head + at + i] = shared[(long long)t * lds + i];
    }
}

extern "C" int abk_spread_shared(const void *shared, long long lds, void *keys, long long ldk, int k_head, int at, int count,
                                 int heads, int dtype, int n_tokens, void *stream) {
    if (n_tokens <= 0 || count <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == ABK_BF16)
        abk_launch(spread_shared_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(128), 0, s, (const __nv_bfloat16 *)shared, lds,
                   (__nv_bfloat16 *)keys, ldk, k_head, at, count, heads);
    else
        abk_launch(spread_shared_kernel<float>, dim3(n_tokens), dim3(128), 0, s, (const float *)shared, lds, (float *)keys,
                   ldk, k_head, at, count, heads);
    return ABK_LAUNCH_RESULT();
}
