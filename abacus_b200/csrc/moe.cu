// A feed-forward of routed experts: every token goes through `top` of `experts` small feed-forward layers, chosen by
// a router.
//
//   moe_route       per token: router logits z = R x in float32 (x as stored), the `top` largest (a tie goes to the
//                   lower index), and each chosen expert's weight: sigmoid(z) (score 0) or its softmax over the
//                   chosen (score 1), or (score 2) s = softmax(z) over all router outputs, the choice by s + correction
//                   (a learned shift per output that the weights do not see), the weight s * scale. A pair is
//                   (token, k-th choice), numbered token * top + k; pairs of padding rows carry expert -1. Router
//                   outputs from `n_real` on stand for experts without matrices that return their input: such a
//                   pair carries -2 - (output - n_real), which the products skip and moe_combine_weighted knows. With `always` >= 0 every token has one more pair, its last: that expert with
//                   weight 1 (a shared expert that lies stacked behind the routed ones).
//   routed_product  out[pair] = act(W[expert of pair] (scale of pair * x[row of pair])): a product whose matrix is
//                   chosen per row. With a scale the input is multiplied by it and rounded to its stored type first
//                   (the weight acts on the expert's input). A CTA stages the pair's row in shared memory; a warp makes
//                   an output feature at a time, lanes along the inner dimension, so the expert's rows stream
//                   coalesced. Float32 sums in a fixed order.
//   moe_combine     out[t] (+)= sum over k of pairs[t * top + k], in the order of k.
//   moe_combine_weighted  out[t] = sum over k of weight[t, k] * (pairs[t * top + k], or x[t] for an expert that returns
//                   its input), in the order of k: the weight on the experts' outputs, in float32. The pairs' rows lie in
//                   the pairs' order, or (with `place`) sorted by expert, pair p at row place[p].
//   routed_product also has the gated form: W holds gate rows then up rows, out = silu(gate . x) * (up . x).
//   relu_squared    x = max(x, 0)^2 in place.
#define ABK_DEFINE_ERROR
#include "common.cuh"

#define MR_THREADS 256
template <typename T>
__global__ void __launch_bounds__(MR_THREADS) moe_route_kernel(const T *x, long long ldx, const float *router, int d, int experts,
                                                        int top, int score, int always, const int *token_seq,
                                                        int *pair_expert, float *pair_weight, const float *correction,
                                                        float weight_scale, int n_real) {
    extern __shared__ __align__(16) float mr_smem[];  // [d, rounded up to 4] the row, [experts] logits, [experts] taken flags,
    float *xs = mr_smem, *z = xs + ((d + 3) & ~3);    // [experts] what the choice goes by
    int *taken = (int *)(z + experts);
    float *key = (float *)(taken + experts);
    const int softmax_chosen = score == 1;
    const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int per = top + (always >= 0 ? 1 : 0);  // pairs a token has: its choices, then the expert every token uses
    pair_expert += (long long)t * per, pair_weight += (long long)t * per;
    pdl_wait();
    if (token_seq[t] < 0) {
        for (int k = tid; k < per; k += MR_THREADS) pair_expert[k] = -1, pair_weight[k] = 0.0f;
        return;
    }
    if (always >= 0 && tid == 0) pair_expert[top] = always, pair_weight[top] = 1.0f;
    for (int i = tid; i < d; i += MR_THREADS) xs[i] = to_float(x[(long long)t * ldx + i]);
    for (int e = tid; e < experts; e += MR_THREADS) taken[e] = 0;
    __syncthreads();
    const bool vec = d % 4 == 0 && ((uintptr_t)router & 15) == 0;
    constexpr int W = MR_THREADS / 32;
    for (int e = warp; e < experts;) {  // a warp's router rows, up to four at a time so that their loads are in flight together
        const int left = (experts - e + W - 1) / W, rows = left < 4 ? left : 4;
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const float *w = router + (long long)e * d;
        if (rows == 4) lane_dots<4>(w, (long long)W * d, xs, d, lane, vec, acc);
        else if (rows == 3) lane_dots<3>(w, (long long)W * d, xs, d, lane, vec, acc);
        else if (rows == 2) lane_dots<2>(w, (long long)W * d, xs, d, lane, vec, acc);
        else lane_dots<1>(w, 0, xs, d, lane, vec, acc);
        for (int u = 0; u < rows; u++) {
            const float sum = warp_sum(acc[u]);
            if (lane == 0) z[e + u * W] = sum;
        }
        e += rows * W;
    }
    __syncthreads();
    if (warp != 0) return;
    if (score == 2) {  // z becomes softmax(z) over all outputs; the choice goes by it plus the correction
        float mx = -INFINITY, sum = 0.0f;
        for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, z[e]);
        mx = warp_max(mx);
        for (int e = lane; e < experts; e += 32) sum += expf(z[e] - mx);
        sum = warp_sum(sum);
        for (int e = lane; e < experts; e += 32) {
            z[e] = expf(z[e] - mx) / sum;
            key[e] = z[e] + (correction ? correction[e] : 0.0f);
        }
    } else {
        for (int e = lane; e < experts; e += 32) key[e] = z[e];
    }
    __syncwarp();
    float chosen_max = -INFINITY, denom = 0.0f;
    for (int k = 0; k < top; k++) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < experts; e += 32)
            if (!taken[e] && (key[e] > best || at == 0x7fffffff)) best = key[e], at = e;  // (the first of a lane's own is its lowest)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (oa != 0x7fffffff && (at == 0x7fffffff || ob > best || (ob == best && oa < at))) best = ob, at = oa;
        }
        if (k == 0) chosen_max = best;
        denom += expf(best - chosen_max);
        if (lane == 0) {
            taken[at] = 1;
            pair_expert[k] = at < n_real ? at : -2 - (at - n_real);
            pair_weight[k] = score == 2 ? z[at] * weight_scale : softmax_chosen ? best : 1.0f / (1.0f + expf(-best));
        }
        __syncwarp();
    }
    if (softmax_chosen && lane == 0)
        for (int k = 0; k < top; k++) {
            pair_weight[k] = expf(pair_weight[k] - chosen_max) / denom;
        }
}

extern "C" int abk_moe_route(const void *x, long long ldx, int dtype, const float *router, int n_tokens, int d, int experts,
                             int top, int score, int always, const int *token_seq, int *pair_expert,
                             float *pair_weight, const float *correction, float weight_scale, int n_real, void *stream) {
    if (n_tokens <= 0) return 0;
    if (top < 1 || top > experts) ABK_REFUSE("moe_route: %d of %d experts", top, experts);
    if (score < 0 || score > 2) ABK_REFUSE("moe_route: score %d is not built", score);
    if (n_real < 0 || n_real > experts) n_real = experts;
    const size_t smem = (size_t)(((d + 3) & ~3) + 3 * experts) * 4;
    if (smem > 200 * 1024) ABK_REFUSE("moe_route: a row of %d and %d experts do not fit shared memory", d, experts);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == ABK_BF16) {
        if (smem > 48 * 1024) {
            cudaError_t e = abk_allow_shared_memory((const void *)moe_route_kernel<__nv_bfloat16>, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        abk_launch(moe_route_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(MR_THREADS), smem, s, (const __nv_bfloat16 *)x, ldx, router,
                   d, experts, top, score, always, token_seq, pair_expert, pair_weight, correction, weight_scale, n_real);
    } else {
        if (smem > 48 * 1024) {
            cudaError_t e = abk_allow_shared_memory((const void *)moe_route_kernel<float>, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        abk_launch(moe_route_kernel<float>, dim3(n_tokens), dim3(MR_THREADS), smem, s, (const float *)x, ldx, router, d, experts, top,
                   score, always, token_seq, pair_expert, pair_weight, correction, weight_scale, n_real);
    }
    return ABK_LAUNCH_RESULT();
}

#define RP_PER_WARP 4
enum { RP_NONE = 0, RP_RELU_SQUARED = 1, RP_SILU_GATED = 2 };  // gated: w has 2 * outs rows a matrix, gate rows then up rows

template <typename T, typename TO, int ACT>
__global__ void __launch_bounds__(128) routed_product_kernel(const T *__restrict__ x, long long ldx, int pairs_per_row,
                                                             const T *__restrict__ w, const int *pair_expert,
                                                             const float *pair_scale, TO *__restrict__ out, long long ldo,
                                                             int in, int outs) {
    extern __shared__ __align__(16) float rp_x[];  // [in]
    const int pair = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_wait();
    const int e = pair_expert[pair];
    const int o0 = (blockIdx.y * 4 + warp) * RP_PER_WARP;
    if (e < 0) {  // a padding row
        if (lane < RP_PER_WARP && o0 + lane < outs) out[(long long)pair * ldo + o0 + lane] = from_float<TO>(0.0f);
        return;
    }
    const T *row = x + (long long)(pair / pairs_per_row) * ldx;
    if (pair_scale) {
        const float sc = pair_scale[pair];
        for (int i = threadIdx.x; i < in; i += 128) rp_x[i] = to_float(from_float<T>(sc * to_float(row[i])));
    } else {
        for (int i = threadIdx.x; i < in; i += 128) rp_x[i] = to_float(row[i]);
    }
    __syncthreads();
    if (o0 >= outs) return;
    const T *wr = w + ((long long)e * (ACT == RP_SILU_GATED ? 2 * outs : outs) + o0) * in;
    const bool vec = in % (16 / (int)sizeof(T)) == 0 && ((uintptr_t)w & 15) == 0;
    float acc[RP_PER_WARP] = {0.0f, 0.0f, 0.0f, 0.0f};
    float up[RP_PER_WARP] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (ACT == RP_SILU_GATED) {
        const T *wu = wr + (long long)outs * in;
        if (o0 + RP_PER_WARP <= outs) lane_dots<RP_PER_WARP>(wu, in, rp_x, in, lane, vec, up);
        else
            for (int u = 0; o0 + u < outs; u++) lane_dots<1>(wu + (long long)u * in, 0, rp_x, in, lane, vec, up + u);
    }
    if (o0 + RP_PER_WARP <= outs) lane_dots<RP_PER_WARP>(wr, in, rp_x, in, lane, vec, acc);  // four rows' loads in flight together
    else
        for (int u = 0; o0 + u < outs; u++) lane_dots<1>(wr + (long long)u * in, 0, rp_x, in, lane, vec, acc + u);
#pragma unroll
    for (int u = 0; u < RP_PER_WARP; u++) {
        float v = warp_sum(acc[u]);
        if (ACT == RP_RELU_SQUARED) v = v > 0.0f ? v * v : 0.0f;
        if (ACT == RP_SILU_GATED) {  // gate and up as stored tensors of the model's type, like the dense feed-forward's
            const float g = to_float(from_float<T>(v)), w_up = to_float(from_float<T>(warp_sum(up[u])));
            v = g / (1.0f + expf(-g)) * w_up;
        }
        if (lane == 0 && o0 + u < outs) out[(long long)pair * ldo + o0 + u] = from_float<TO>(v);
    }
}

// x: the row of pair p is x + (p / pairs_per_row) * ldx (pairs_per_row 1: a row per pair; `top`: a row per token);
// w [experts][outs][in] of x's type; out [pairs][ldo] of x's type or (out_f32) float32.
extern "C" int abk_routed_product(const void *x, long long ldx, int pairs_per_row, int dtype, const void *w,
                                  const int *pair_expert, const float *pair_scale, void *out, long long ldo, int out_f32,
                                  int activation, int n_pairs, int in, int outs, void *stream) {
    if (n_pairs <= 0 || outs <= 0) return 0;
    if (in < 1 || (size_t)in * 4 > 200 * 1024) ABK_REFUSE("routed_product: an inner size of %d does not fit shared memory", in);
    if (pairs_per_row < 1) pairs_per_row = 1;
    dim3 grid(n_pairs, (outs + 4 * RP_PER_WARP - 1) / (4 * RP_PER_WARP));
    if (grid.y > 65535) ABK_REFUSE("routed_product: %d output features are more than a grid takes", outs);
    const size_t smem = (size_t)in * 4;
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
#define RP_LAUNCH(T, TO, ACT)                                                                                       \
    do {                                                                                                            \
        if (smem > 48 * 1024) {                                                                                     \
            cudaError_t e = abk_allow_shared_memory((const void *)routed_product_kernel<T, TO, ACT>, (int)smem);    \
            if (e != cudaSuccess) return (int)e;                                                                    \
        }                                                                                                           \
        abk_launch(routed_product_kernel<T, TO, ACT>, grid, dim3(128), smem, s, (const T *)x, ldx, pairs_per_row,   \
                   (const T *)w, pair_expert, pair_scale, (TO *)out, ldo, in, outs);                                \
    } while (0)
    const bool relu2 = activation == RP_RELU_SQUARED, gated = activation == RP_SILU_GATED;
    if (activation != RP_NONE && !relu2 && !gated) ABK_REFUSE("routed_product: activation %d is not built", activation);
    if (dtype == ABK_BF16 && out_f32) { if (gated) RP_LAUNCH(bf, float, 2); else if (relu2) RP_LAUNCH(bf, float, 1); else RP_LAUNCH(bf, float, 0); }
    else if (dtype == ABK_BF16) { if (gated) RP_LAUNCH(bf, bf, 2); else if (relu2) RP_LAUNCH(bf, bf, 1); else RP_LAUNCH(bf, bf, 0); }
    else { if (gated) RP_LAUNCH(float, float, 2); else if (relu2) RP_LAUNCH(float, float, 1); else RP_LAUNCH(float, float, 0); }
#undef RP_LAUNCH
    return ABK_LAUNCH_RESULT();
}

__global__ void __launch_bounds__(256) moe_combine_kernel(const float *pairs, float *out, long long total, int d, int top,
                                                          int add) {
    pdl_wait();
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= total) return;
    const long long t = i / d, j = i - t * d;
    float acc = pairs[(t * top) * d + j];
    for (int k = 1; k < top; k++) acc += pairs[(t * top + k) * d + j];
    out[i] = add ? out[i] + acc : acc;
}

// out float32 [tokens][d]; pairs float32 [tokens * top][d]; add: out already holds what the pairs join (a shared expert).
extern "C" int abk_moe_combine(const float *pairs, float *out, int n_tokens, int d, int top, int add, void *stream) {
    const long long total = (long long)n_tokens * d;
    if (total <= 0) return 0;
    abk_launch(moe_combine_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, pairs, out,
               total, d, top, add);
    return ABK_LAUNCH_RESULT();
}

template <typename T>
__global__ void __launch_bounds__(256) moe_combine_weighted_kernel(const float *pairs, const float *weight, const int *expert,
                                                                   const T *x, long long ldx, float *out, long long total, int d,
                                                                   int top, const int *place) {
    pdl_wait();
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= total) return;
    const long long t = i / d, j = i - t * d;
    float acc = 0.0f;
    for (int k = 0; k < top; k++) {
        const int e = expert[t * top + k];
        if (e == -1) continue;  // a padding row
        const long long at = place && e >= 0 ? place[t * top + k] : t * top + k;  // rows sorted by expert: the pair's place
        acc = fmaf(weight[t * top + k], e >= 0 ? pairs[at * d + j] : to_float(x[t * ldx + j]), acc);
    }
    out[i] = acc;
}

// out float32 [tokens][d] = sum_k weight[t, k] * (pairs[t * top + k], or x[t] where expert[t, k] <= -2). place (or null):
// pair p's row in `pairs` is place[p] (rows sorted by expert), not p.
extern "C" int abk_moe_combine_weighted(const float *pairs, const float *weight, const int *expert, const void *x, long long ldx,
                                        int dtype, float *out, int n_tokens, int d, int top, const int *place, void *stream) {
    const long long total = (long long)n_tokens * d;
    if (total <= 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == ABK_BF16)
        abk_launch(moe_combine_weighted_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, pairs, weight,
                   expert, (const __nv_bfloat16 *)x, ldx, out, total, d, top, place);
    else
        abk_launch(moe_combine_weighted_kernel<float>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, pairs, weight, expert,
                   (const float *)x, ldx, out, total, d, top, place);
    return ABK_LAUNCH_RESULT();
}

template <typename T> __global__ void __launch_bounds__(256) relu_squared_kernel(T *x, long long total) {
    pdl_wait();
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= total) return;
    const float v = to_float(x[i]);
    x[i] = from_float<T>(v > 0.0f ? v * v : 0.0f);
}

extern "C" int abk_relu_squared(void *x, int dtype, long long total, void *stream) {
    if (total <= 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == ABK_BF16) abk_launch(relu_squared_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (__nv_bfloat16 *)x, total);
    else abk_launch(relu_squared_kernel<float>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (float *)x, total);
    return ABK_LAUNCH_RESULT();
}

// ------------------------------------------------------------------ experts by a table
// A token's experts by its id: pair t * top + k is expert table[token[t]][k] with weight 1 / top. Rows of padding, tokens
// outside the table and entries that name no expert give -1 (no expert) and weight 0; the latter two set bit 0 of status.
__global__ void __launch_bounds__(256) moe_table_kernel(const int *tokens, const int *token_seq, const int *table, int vocab, int experts,
                                                        int top, int n_pairs, int *pair_expert, float *pair_weight, int *status) {
    pdl_wait();
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= n_pairs) return;
    const int t = i / top, k = i - t * top;
    int e = -1;
    if (token_seq[t] >= 0) {
        const int tok = tokens[t];
        if (tok >= 0 && tok < vocab) e = table[(long long)tok * top + k];
        if (e < 0 || e >= experts) {
            e = -1;
            atomicOr(status, 1);
        }
    }
    pair_expert[i] = e;
    pair_weight[i] = e >= 0 ? 1.0f / (float)top : 0.0f;
}

extern "C" int abk_moe_table(const int *tokens, const int *token_seq, const int *table, int vocab, int experts, int top,
                             int n_tokens, int *pair_expert, float *pair_weight, int *status, void *stream) {
    const long long n_pairs = (long long)n_tokens * top;
    if (n_pairs <= 0) return 0;
    if (n_pairs > 0x7fffffffLL) ABK_REFUSE("moe_table: %lld pairs are more than a grid takes", n_pairs);
    abk_launch(moe_table_kernel, dim3((unsigned)((n_pairs + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, tokens, token_seq,
               table, vocab, experts, top, (int)n_pairs, pair_expert, pair_weight, status);
    return ABK_LAUNCH_RESULT();
}
