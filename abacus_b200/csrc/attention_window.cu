// Causal attention of whole prompts on the warp-level tensor cores (mma.sync m16n8k16, bfloat16 operands,
// float32 accumulation) with what the plain prefill kernels do not take: a sliding window that also keeps a
// sequence's first keys, a sink in the softmax, values of another size than keys, and softmax weights that stay
// float32 in the second product.
//
//   key j is seen from i when j <= i and (window == 0 or i - j < window or j < keep_first)
//                                    and (chunk == 0 or j / chunk == i / chunk)
//   p_j = exp(z_j - M) / (exp(sink - M) + sum_j exp(z_j - M)),  z_j = scale * (q . k_j),  out = sum_j p_j v_j
//   (with a cap c of the scores, z_j = c tanh(scale * (q . k_j) / c))
//
// Keys and values are read from the step's own rows (every sequence of the step starts at position 0), so a
// windowed layer's ring of cache pages is not touched. A CTA has 64 query rows of one head (four warps of 16
// rows) and walks tiles of 64 keys: the tiles that hold kept first keys out of the window's reach, then the
// window's (or, without a window, all up to the diagonal); tiles no row of the CTA can see are never loaded.
// Tiles come in by cp.async into rows padded by 16 bytes (ldmatrix without bank conflicts); with two stages the
// next tile comes in while this one is multiplied.
//
// The weights of the second product are float32: each is split into three bfloat16 parts (the value rounded,
// the remainder rounded, the remainder of that), which together hold its 24 bits, and the product is taken
// three times into the same float32 accumulators. Scores have bfloat16 operands and so are exact products
// summed in float32.
#define ABK_DEFINE_ERROR
#include "common.cuh"
#include "mma_tiles.cuh"

#define AW_ROWS 64
#define AW_KEYS 64
#define AW_THREADS 128
#define AW_MAX_VT 16  // value columns / 8 a warp accumulates: values of up to 128

struct AttnWindow {
    const __nv_bfloat16 *qkv;  // rows of `row` elements: q heads, then (at k_off) k heads, then (at v_off) v heads
    long long row;
    __nv_bfloat16 *out;        // [tokens, n_heads * v_dim]
    int n_heads, n_kv_heads, head_dim, v_dim;
    int k_off, v_off;
    float scale_log2;          // score scale times log2(e)
    float scale, softcap;      // softcap > 0: z <- softcap * tanh(scale * (q . k) / softcap), in float32, before the softmax
    int window, keep_first;
    int chunk;                 // > 0: key j is seen from i only if j / chunk == i / chunk (positions from the sequence's start)
    const float *sink;         // [n_heads] or null
    const int *seq_start;      // [n_seqs + 1]
    int n_seqs;
    int stages;                // 2: the next tile of keys and values comes in while this one is multiplied; 1: one tile at a time
};

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void *src, bool real) {
    const int bytes = real ? 16 : 0;  // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
// 2^x by the special-function unit (float32, about two units in the last place; -inf gives 0)
__device__ __forceinline__ float exp2_sfu(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// 64 rows of `width` elements (a multiple of 8) from global rows `first ..` (rows from `limit` on are zeros) into
// shared rows of `pitch` bytes whose first `padded` elements (a multiple of 16 >= width) are all written.
__device__ __forceinline__ void load_tile(uint32_t dst, int pitch, int padded, const __nv_bfloat16 *src, long long row_pitch,
                                          int first, int limit, int width) {
    const int chunks = padded >> 3;
    for (int e = threadIdx.x; e < 64 * chunks; e += AW_THREADS) {
        const int r = e / chunks, c = e - r * chunks;
        const bool real = first + r < limit && c * 8 < width;
        cp_async_16(dst + r * pitch + c * 16, real ? src + (long long)(first + r) * row_pitch + c * 8 : src, real);
    }
}

__global__ void __launch_bounds__(AW_THREADS) attention_window_kernel(AttnWindow p) {
    extern __shared__ __align__(16) uint8_t aw_smem[];
    const int D = p.head_dim, VD = p.v_dim;
    const int d16 = (D + 15) & ~15, v16 = (VD + 15) & ~15;
    const int pitch_k = d16 * 2 + 16, pitch_v = v16 * 2 + 16;
    const uint32_t q_s = (uint32_t)__cvta_generic_to_shared(aw_smem);
    const uint32_t k_s = q_s + AW_ROWS * pitch_k;                   // p.stages stages
    const uint32_t v_s = k_s + p.stages * AW_KEYS * pitch_k;        // p.stages stages
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c2 = (lane & 3) * 2;
    const int h = blockIdx.y, kvh = h / (p.n_heads / p.n_kv_heads);
    const float sink2 = p.sink ? p.sink[h] * 1.4426950408889634f : -INFINITY;  // a weight: ahead of the wait
    pdl_wait();
    // which sequence and which of its tiles of 64 rows this CTA has
    int seq = -1, tile = blockIdx.x, start = 0, n = 0;
    for (int s = 0; s < p.n_seqs; s++) {
        start = p.seq_start[s], n = p.seq_start[s + 1] - start;
        const int tiles = (n + AW_ROWS - 1) / AW_ROWS;
        if (tile < tiles) {
            seq = s;
            break;
        }
        tile -= tiles;
    }
    if (seq < 0) return;
    const int r0 = tile * AW_ROWS, r_last = min(r0 + AW_ROWS - 1, n - 1);
    const __nv_bfloat16 *base = p.qkv + (long long)start * p.row;
    const __nv_bfloat16 *kg = base + p.k_off + (long long)kvh * D, *vg = base + p.v_off + (long long)kvh * VD;

    // tiles of keys: first those with kept first keys that lie before the window's first tile, then the window's
    int lo = p.window > 0 && r0 - p.window + 1 > 0 ? r0 - p.window + 1 : 0;  // first key the CTA's first row sees in its window
    if (p.chunk > 0) lo = max(lo, r0 / p.chunk * p.chunk);  // or in its chunk (later rows' chunks start no earlier)
    const int w_first = lo / AW_KEYS, w_last = r_last / AW_KEYS;
    const int kept_tiles = p.window > 0 ? min((p.keep_first + AW_KEYS - 1) / AW_KEYS, w_first) : 0;
    const int n_tiles = kept_tiles + w_last - w_first + 1;
#define TILE_AT(i) ((i) < kept_tiles ? (i) : w_first + (i) - kept_tiles)

    load_tile(q_s, pitch_k, d16, base + (long long)h * D, p.row, r0, n, D);
    load_tile(k_s, pitch_k, d16, kg, p.row, TILE_AT(0) * AW_KEYS, n, D);
    load_tile(v_s, pitch_v, v16, vg, p.row, TILE_AT(0) * AW_KEYS, n, VD);
    cp_async_commit();

    float o[AW_MAX_VT][4];
#pragma unroll
    for (int t = 0; t < AW_MAX_VT; t++) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.0f;
    float m[2] = {sink2, sink2}, l[2] = {p.sink ? 1.0f : 0.0f, p.sink ? 1.0f : 0.0f};
    const int n_vt = v16 >> 3;  // value column tiles of 8 (an even number)
    const int row_a = r0 + warp * 16 + g, row_b = row_a + 8;  // the two query rows (positions) this thread has a part of
    const int chunk_a = p.chunk > 0 ? row_a / p.chunk * p.chunk : 0, chunk_b = p.chunk > 0 ? row_b / p.chunk * p.chunk : 0;
    const float cap_inv = p.softcap > 0.0f ? 1.0f / p.softcap : 0.0f, cap_log2 = p.softcap * 1.4426950408889634f;

    for (int it = 0; it < n_tiles; it++) {
        const int stage = p.stages == 2 ? it & 1 : 0, key0 = TILE_AT(it) * AW_KEYS;
        if (p.stages == 2 && it + 1 < n_tiles) {  // the next tile into the other stage (its last readers passed the barrier below)
            const int next = TILE_AT(it + 1) * AW_KEYS;
            load_tile(k_s + (stage ^ 1) * AW_KEYS * pitch_k, pitch_k, d16, kg, p.row, next, n, D);
            load_tile(v_s + (stage ^ 1) * AW_KEYS * pitch_v, pitch_v, v16, vg, p.row, next, n, VD);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            if (p.stages == 1 && it > 0) {  // one stage: this tile now (other CTAs of the SM work meanwhile)
                load_tile(k_s, pitch_k, d16, kg, p.row, key0, n, D);
                load_tile(v_s, pitch_v, v16, vg, p.row, key0, n, VD);
                cp_async_commit();
            }
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t kt = k_s + stage * AW_KEYS * pitch_k, vt = v_s + stage * AW_KEYS * pitch_v;

        // scores of this warp's 16 rows against the tile's 64 keys
        float s[8][4];
#pragma unroll
        for (int t = 0; t < 8; t++) s[t][0] = s[t][1] = s[t][2] = s[t][3] = 0.0f;
        for (int ks = 0; ks < d16 / 16; ks++) {
            uint32_t a[4];
            ldsm_x4(q_s + (warp * 16 + (lane & 15)) * pitch_k + (ks * 16 + (lane >> 4) * 8) * 2, a[0], a[1], a[2], a[3]);
#pragma unroll
            for (int tp = 0; tp < 4; tp++) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(kt + (tp * 16 + (lane & 7) + ((lane >> 4) << 3)) * pitch_k + (ks * 16 + ((lane >> 3) & 1) * 8) * 2,
                        b0, b1, b2, b3);
                mma_bf16(s[2 * tp], a, b0, b1);
                mma_bf16(s[2 * tp + 1], a, b2, b3);
            }
        }
        // what each row may see, the tile's maximum per row
        const bool kept_tile = it < kept_tiles;  // all its keys lie before every row's window: only kept first keys count
        // a tile whose every key every row of this warp sees (below the diagonal, inside the window, rows within the
        // sequence) needs no look at single keys: most tiles of a long window
        const int warp_first = r0 + warp * 16, warp_last = warp_first + 15;
        const bool clear = !kept_tile && key0 + AW_KEYS - 1 <= warp_first && warp_last < n &&
                           (p.window <= 0 || warp_last - key0 < p.window) &&
                           (p.chunk <= 0 || key0 >= warp_last / p.chunk * p.chunk);
        if (p.softcap > 0.0f) {  // capped scores, in float32: z = cap * tanh(scale * (q . k) / cap)
#pragma unroll
            for (int t = 0; t < 8; t++) {
#pragma unroll
                for (int e = 0; e < 4; e++) s[t][e] = cap_log2 * tanhf(s[t][e] * p.scale * cap_inv);
            }
        }
        const float to_log2 = p.softcap > 0.0f ? 1.0f : p.scale_log2;
        float top[2] = {-INFINITY, -INFINITY};
        if (clear) {
#pragma unroll
            for (int t = 0; t < 8; t++) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    s[t][e] *= to_log2;
                    top[e >> 1] = fmaxf(top[e >> 1], s[t][e]);
                }
            }
        } else {
#pragma unroll
            for (int t = 0; t < 8; t++) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int j = key0 + t * 8 + c2 + (e & 1), i = e < 2 ? row_a : row_b;
                    bool seen = j <= i && i < n;
                    if (kept_tile) seen = seen && j < p.keep_first;
                    else if (p.window > 0) seen = seen && (i - j < p.window || j < p.keep_first);
                    if (p.chunk > 0) seen = seen && j >= (e < 2 ? chunk_a : chunk_b);
                    s[t][e] = seen ? s[t][e] * to_log2 : -INFINITY;
                    top[e >> 1] = fmaxf(top[e >> 1], s[t][e]);
                }
            }
        }
        float corr[2], ref[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const float m_new = fmaxf(m[r], quad_max(top[r]));
            ref[r] = m_new == -INFINITY ? 0.0f : m_new;  // a row that has seen nothing yet: all its weights are 0
            corr[r] = exp2_sfu(m[r] - ref[r]);           // (0 when m is still -inf)
            m[r] = m_new;
        }
        float sum[2] = {0.0f, 0.0f};
#pragma unroll
        for (int t = 0; t < 8; t++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                s[t][e] = exp2_sfu(s[t][e] - ref[e >> 1]);
                sum[e >> 1] += s[t][e];
            }
        }
#pragma unroll
        for (int r = 0; r < 2; r++) l[r] = l[r] * corr[r] + quad_sum(sum[r]);
#pragma unroll
        for (int t = 0; t < AW_MAX_VT; t++) {
            if (t < n_vt) o[t][0] *= corr[0], o[t][1] *= corr[0], o[t][2] *= corr[1], o[t][3] *= corr[1];
        }
        // the weights as three bfloat16 parts each, times the values
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
            uint32_t part[3][4];
#pragma unroll
            for (int f = 0; f < 4; f++) {  // fragment register f: n-tile 2 ks + (f >> 1), accumulator pair f & 1
                float x0 = s[2 * ks + (f >> 1)][2 * (f & 1)], x1 = s[2 * ks + (f >> 1)][2 * (f & 1) + 1];
#pragma unroll
                for (int q = 0; q < 3; q++) {
                    const __nv_bfloat162 hi = __floats2bfloat162_rn(x0, x1);
                    part[q][f] = *(const uint32_t *)&hi;
                    x0 -= __low2float(hi), x1 -= __high2float(hi);
                }
            }
#pragma unroll
            for (int tp = 0; tp < AW_MAX_VT / 2; tp++) {
                if (2 * tp < n_vt) {
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4_t(vt + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * pitch_v + (tp * 16 + (lane >> 4) * 8) * 2,
                              b0, b1, b2, b3);
#pragma unroll
                    for (int q = 0; q < 3; q++) {
                        mma_bf16(o[2 * tp], part[q], b0, b1);
                        mma_bf16(o[2 * tp + 1], part[q], b2, b3);
                    }
                }
            }
        }
        __syncthreads();  // the stage is loaded again by the iteration after next
    }
#undef TILE_AT
    // out = o / l
    const float inv_a = 1.0f / l[0], inv_b = 1.0f / l[1];
#pragma unroll
    for (int t = 0; t < AW_MAX_VT; t++) {
        const int col = t * 8 + c2;
        if (t < n_vt && col < VD) {
            if (row_a < n) {
                const __nv_bfloat162 v = __floats2bfloat162_rn(o[t][0] * inv_a, o[t][1] * inv_a);
                *(__nv_bfloat162 *)(p.out + ((long long)(start + row_a) * p.n_heads + h) * VD + col) = v;
            }
            if (row_b < n) {
                const __nv_bfloat162 v = __floats2bfloat162_rn(o[t][2] * inv_b, o[t][3] * inv_b);
                *(__nv_bfloat162 *)(p.out + ((long long)(start + row_b) * p.n_heads + h) * VD + col) = v;
            }
        }
    }
}

// max_tiles: an upper bound of the step's tiles of 64 rows, sum over its sequences of ceil(rows / 64) (the host
// knows the rows; CTAs beyond the real tiles return at once).
extern "C" int abk_attention_window(const void *qkv, long long row, void *out, int n_heads, int n_kv_heads, int head_dim,
                                    int v_dim, int k_off, int v_off, float scale, int window, int keep_first,
                                    const float *sink, const int *seq_start, int n_seqs, int max_tiles, int chunk,
                                    float softcap, void *stream) {
    if (n_seqs <= 0 || max_tiles <= 0) return 0;
    if (head_dim % 8 || head_dim < 8 || head_dim > 256) ABK_REFUSE("attention_window: head_dim %d is not a multiple of 8 up to 256", head_dim);
    if (v_dim % 8 || v_dim < 8 || v_dim > 8 * AW_MAX_VT) ABK_REFUSE("attention_window: value size %d is not a multiple of 8 up to %d", v_dim, 8 * AW_MAX_VT);
    if (row % 8 || k_off % 8 || v_off % 8 || ((uintptr_t)qkv & 15)) ABK_REFUSE("attention_window: rows of q, k and v are not 16-byte aligned");
    if (n_kv_heads < 1 || n_heads % n_kv_heads) ABK_REFUSE("attention_window: %d query heads do not divide into %d kv heads", n_heads, n_kv_heads);
    if (n_heads > 65535) ABK_REFUSE("attention_window: %d heads are more than a grid takes", n_heads);
    if (keep_first < 0 || window <= 0) keep_first = 0;
    AttnWindow p;
    p.qkv = (const __nv_bfloat16 *)qkv, p.row = row, p.out = (__nv_bfloat16 *)out, p.n_heads = n_heads, p.n_kv_heads = n_kv_heads;
    p.head_dim = head_dim, p.v_dim = v_dim, p.k_off = k_off, p.v_off = v_off, p.scale_log2 = scale * 1.4426950408889634f;
    p.window = window > 0 ? window : 0, p.keep_first = keep_first, p.sink = sink, p.seq_start = seq_start, p.n_seqs = n_seqs;
    p.scale = scale, p.softcap = softcap > 0.0f ? softcap : 0.0f, p.chunk = chunk > 0 ? chunk : 0;
    const int d16 = (head_dim + 15) & ~15, v16 = (v_dim + 15) & ~15;
    static int stages_env = -1;  // ABACUS_WINDOW_STAGES=1|2 pins the number of stages (for comparison)
    if (stages_env < 0) {
        const char *e = getenv("ABACUS_WINDOW_STAGES");
        stages_env = e && (e[0] == '1' || e[0] == '2') ? e[0] - '0' : 0;
    }
    // one stage by default: measured on a B200 (16 heads of 128, window 1,024) a CTA that waits for its tile while the
    // SM's other CTAs work (four fit) beats two stages with three CTAs an SM: 1,100 against 1,376 us for 8 x 2,048 tokens
    p.stages = stages_env ? stages_env : 1;
    const int smem = (1 + p.stages) * 64 * (d16 * 2 + 16) + p.stages * 64 * (v16 * 2 + 16);
    cudaError_t e = abk_allow_shared_memory((const void *)attention_window_kernel, smem);
    if (e != cudaSuccess) return (int)e;
    abk_launch(attention_window_kernel, dim3(max_tiles, n_heads), dim3(AW_THREADS), (size_t)smem, (cudaStream_t)stream, p);
    return ABK_LAUNCH_RESULT();
}
