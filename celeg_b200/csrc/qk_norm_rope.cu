// Stand-alone launch of the q/k post-processing; the work of a unit is in qk_norm_rope.cuh.
#include "qk_norm_rope.cuh"

namespace celeg_b200 {

template <typename A>
__global__ void qk_norm_rope_store_kernel(A* qkv, A* k_cache, A* v_cache, const QkNormRopeArgs args) {
    chain_release();
    chain_wait();
    const int warps_per_block = blockDim.x >> 5;
    const long long unit = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    if (unit >= (long long)args.tokens * (args.q_heads + 2 * args.kv_heads)) return;
    qk_norm_rope_unit<A>(qkv, k_cache, v_cache, args, unit, threadIdx.x & 31);
}

// The common shape (rotation over the whole head, head size 64, 128 or 256, many tokens): a warp takes
// one token and a run of its heads, so the angles' sine and cosine, which depend on the position and the
// pair only, are computed once for the run instead of once per head (they were most of the instructions
// of the per-head kernel), and the page of the token is looked up once. Same arithmetic per element.
template <typename A, int PAIRS>
__global__ void __launch_bounds__(128)
qk_norm_rope_tokens_kernel(A* qkv, A* k_cache, A* v_cache, const QkNormRopeArgs a, const int run) {
    chain_release();
    chain_wait();
    const int lane = threadIdx.x & 31;
    const int heads = a.q_heads + 2 * a.kv_heads;
    const int runs = (heads + run - 1) / run;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= (long long)a.tokens * runs) return;
    const int t = (int)(unit / runs);
    const int h_begin = (int)(unit % runs) * run;
    const int h_end = min(heads, h_begin + run);
    constexpr int kHead = PAIRS * 64, kHalf = PAIRS * 32;
    const int pos = a.positions[t];
    float sn[PAIRS], cs[PAIRS];
#pragma unroll
    for (int j = 0; j < PAIRS; ++j) sincosf((float)pos * a.inv_freq[lane + 32 * j], &sn[j], &cs[j]);
    long long cache_row = -1;                       // offset of (page, kv head 0, slot in page), in elements
    if (a.store_kv == 1 && h_end > a.q_heads) {
        const int page = a.block_table[(size_t)a.token_span[t] * a.table_stride + pos / a.page_tokens];
        if (page < 0) {                             // the host never builds such a table
            if (lane == 0) atomicExch(a.error_flag, 1);
        } else {
            cache_row = (long long)page * a.page_stride + (long long)(pos % a.page_tokens) * kHead;
        }
    }
    for (int h = h_begin; h < h_end; ++h) {
        A* vec = qkv + ((size_t)t * heads + h) * kHead;
        const bool is_q = h < a.q_heads;
        const bool is_k = !is_q && h < a.q_heads + a.kv_heads;
        A* dst = vec;
        if (!is_q && a.store_kv == 2) {
            if (!is_k) continue;                    // k in place, v untouched
        } else if (!is_q) {
            if (cache_row < 0) continue;
            const int kvh = is_k ? h - a.q_heads : h - a.q_heads - a.kv_heads;
            dst = (is_k ? k_cache : v_cache) + cache_row + (size_t)kvh * a.page_tokens * kHead;
        }
        float x[PAIRS], y[PAIRS];
#pragma unroll
        for (int j = 0; j < PAIRS; ++j) {
            x[j] = to_float(load_l2(vec + lane + 32 * j));
            y[j] = to_float(load_l2(vec + lane + 32 * j + kHalf));
        }
        if (!is_q && !is_k) {                       // v: plain copy
#pragma unroll
            for (int j = 0; j < PAIRS; ++j) {
                dst[lane + 32 * j] = from_float<A>(x[j]);
                dst[lane + 32 * j + kHalf] = from_float<A>(y[j]);
            }
            continue;
        }
        const float* weight = is_q ? a.q_weight : a.k_weight;
        float scale = 1.0f;
        if (weight) {
            float sum = 0.0f;
#pragma unroll
            for (int j = 0; j < PAIRS; ++j) sum += x[j] * x[j];
#pragma unroll
            for (int j = 0; j < PAIRS; ++j) sum += y[j] * y[j];
            sum = warp_sum(sum);
            scale = 1.0f / sqrtf(sum / (float)kHead + a.eps);
        }
#pragma unroll
        for (int j = 0; j < PAIRS; ++j) {
            const int i = lane + 32 * j;
            float u = x[j], v = y[j];
            if (weight) {
                u = u * scale * weight[i];
                v = v * scale * weight[i + kHalf];
            }
            dst[i] = from_float<A>(u * cs[j] - v * sn[j]);
            dst[i + kHalf] = from_float<A>(v * cs[j] + u * sn[j]);
        }
    }
}

// The same for many tokens with 16-byte accesses: a warp per token; LANES = head size / 16 lanes share a head,
// lane `sub` of them holds elements [8 sub, 8 sub + 8) and their rotation partners [8 (sub + LANES), ...), so a
// warp takes 32 / LANES heads at a time. A lane's sines and cosines are computed once per token and serve
// every head; the sum of squares meets over the LANES lanes by shuffles. Arithmetic as in the kernels above
// (float32 throughout, one rounding at the end); only the order of the sum of squares differs.
template <int LANES>
__global__ void __launch_bounds__(128)
qk_norm_rope_tokens_vec_kernel(__nv_bfloat16* qkv, __nv_bfloat16* k_cache, __nv_bfloat16* v_cache, const QkNormRopeArgs a) {
    chain_release();
    constexpr int kHead = LANES * 16, kHalf = LANES * 8, kHeadsAtOnce = 32 / LANES;
    const int lane = threadIdx.x & 31;
    const int sub = lane % LANES, slot = lane / LANES;
    // constant data first: this lane's frequencies and norm weights
    float freq[8], wq[16], wk[16];
#pragma unroll
    for (int e = 0; e < 8; ++e) freq[e] = a.inv_freq[sub * 8 + e];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        wq[e] = a.q_weight ? a.q_weight[sub * 8 + e] : 1.0f;
        wq[8 + e] = a.q_weight ? a.q_weight[kHalf + sub * 8 + e] : 1.0f;
        wk[e] = a.k_weight ? a.k_weight[sub * 8 + e] : 1.0f;
        wk[8 + e] = a.k_weight ? a.k_weight[kHalf + sub * 8 + e] : 1.0f;
    }
    chain_wait();
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= a.tokens) return;
    const int heads = a.q_heads + 2 * a.kv_heads;
    const int pos = a.positions[t];
    float sn[8], cs[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) sincosf((float)pos * freq[e], &sn[e], &cs[e]);
    long long cache_row = -1;                       // offset of (page, kv head 0, slot in page), in elements
    if (a.store_kv == 1) {
        const int page = a.block_table[(size_t)a.token_span[t] * a.table_stride + pos / a.page_tokens];
        if (page < 0) {                             // the host never builds such a table
            if (lane == 0) atomicExch(a.error_flag, 1);
        } else {
            cache_row = (long long)page * a.page_stride + (long long)(pos % a.page_tokens) * kHead;
        }
    }
    __nv_bfloat16* row = qkv + (size_t)t * heads * kHead;
    for (int h0 = 0; h0 < heads; h0 += kHeadsAtOnce) {
        const int h = h0 + slot;
        const bool is_q = h < a.q_heads;
        const bool is_k = !is_q && h < a.q_heads + a.kv_heads;
        bool active = h < heads;
        __nv_bfloat16* vec = row + (size_t)h * kHead;
        __nv_bfloat16* dst = vec;
        if (active && !is_q) {
            if (a.store_kv == 2) {
                active = is_k;                      // k in place, v untouched
            } else if (cache_row < 0) {
                active = false;                     // q heads only, or no page
            } else {
                const int kvh = is_k ? h - a.q_heads : h - a.q_heads - a.kv_heads;
                dst = (is_k ? k_cache : v_cache) + cache_row + (size_t)kvh * a.page_tokens * kHead;
            }
        }
        uint4 lo4 = make_uint4(0u, 0u, 0u, 0u), hi4 = lo4;
        if (active) {
            lo4 = __ldcg(reinterpret_cast<const uint4*>(vec + sub * 8));
            hi4 = __ldcg(reinterpret_cast<const uint4*>(vec + kHalf + sub * 8));
        }
        const bool is_v = !is_q && !is_k;
        float x[8], y[8];
        {
            const __nv_bfloat162* l2 = reinterpret_cast<const __nv_bfloat162*>(&lo4);
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&hi4);
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2) {
                const float2 l = __bfloat1622float2(l2[e2]), u = __bfloat1622float2(h2[e2]);
                x[2 * e2] = l.x;
                x[2 * e2 + 1] = l.y;
                y[2 * e2] = u.x;
                y[2 * e2 + 1] = u.y;
            }
        }
        // (every lane takes part in the shuffles; heads past the end and v heads carry zeros or are not used)
        const float* weight = is_q ? a.q_weight : a.k_weight;
        float sum = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) sum += x[e] * x[e];
#pragma unroll
        for (int e = 0; e < 8; ++e) sum += y[e] * y[e];
#pragma unroll
        for (int offset = 1; offset < LANES; offset <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
        if (!active) continue;
        if (is_v) {                                 // v: plain copy
            *reinterpret_cast<uint4*>(dst + sub * 8) = lo4;
            *reinterpret_cast<uint4*>(dst + kHalf + sub * 8) = hi4;
            continue;
        }
        const float scale = weight ? 1.0f / sqrtf(sum / (float)kHead + a.eps) : 1.0f;
        uint4 out_lo, out_hi;
        __nv_bfloat162* ol = reinterpret_cast<__nv_bfloat162*>(&out_lo);
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&out_hi);
        float rl[8], rh[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float u = x[e], v = y[e];
            if (weight) {
                u = u * scale * (is_q ? wq[e] : wk[e]);
                v = v * scale * (is_q ? wq[8 + e] : wk[8 + e]);
            }
            rl[e] = u * cs[e] - v * sn[e];
            rh[e] = v * cs[e] + u * sn[e];
        }
#pragma unroll
        for (int e2 = 0; e2 < 4; ++e2) {
            ol[e2] = __floats2bfloat162_rn(rl[2 * e2], rl[2 * e2 + 1]);
            oh[e2] = __floats2bfloat162_rn(rh[2 * e2], rh[2 * e2 + 1]);
        }
        *reinterpret_cast<uint4*>(dst + sub * 8) = out_lo;
        *reinterpret_cast<uint4*>(dst + kHalf + sub * 8) = out_hi;
    }
}

}  // namespace celeg_b200

using namespace celeg_b200;

CELEG_API int celeg_qk_norm_rope_store(void* qkv, const float* q_weight, const float* k_weight,
                                       const float* inv_freq, const int* positions, const int* token_span,
                                       const int* block_table, int table_stride, void* k_cache, void* v_cache,
                                       long long page_stride, int tokens, int q_heads, int kv_heads,
                                       int head_dim, int rotary_dim, int page_tokens, float eps, int store_kv,
                                       int* error_flag, int act_dtype, cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && q_heads > 0 && kv_heads >= 0 && head_dim > 0 && page_tokens > 0,
                  "qk_norm_rope_store: invalid sizes tokens=%d q_heads=%d kv_heads=%d head_dim=%d page_tokens=%d",
                  tokens, q_heads, kv_heads, head_dim, page_tokens);
    CELEG_REQUIRE(head_dim <= kMaxHeadDim, "qk_norm_rope_store: head_dim %d exceeds %d", head_dim, kMaxHeadDim);
    CELEG_REQUIRE(rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0,
                  "qk_norm_rope_store: rotary_dim %d must be even and at most head_dim %d", rotary_dim, head_dim);
    CELEG_REQUIRE(eps > 0.0f || (!q_weight && !k_weight), "qk_norm_rope_store: eps must be positive");
    CELEG_REQUIRE(store_kv >= 0 && store_kv <= 2, "qk_norm_rope_store: store_kv is 0 (q only), 1 (k and v to the cache) "
                  "or 2 (k in place), not %d", store_kv);
    if (tokens == 0) return 0;
    const long long units = (long long)tokens * (q_heads + 2 * kv_heads);
    const int warps = 4;
    const unsigned blocks = (unsigned)((units + warps - 1) / warps);
    if (!inv_freq) rotary_dim = head_dim & ~1;       // without rotation the pair loop just normalises
    const QkNormRopeArgs args = {q_weight, k_weight, inv_freq, positions, token_span, block_table, table_stride,
                                 page_stride, tokens, q_heads, kv_heads, head_dim, rotary_dim, page_tokens, eps,
                                 store_kv, error_flag};
    // many tokens of the common shape: a warp per token and run of eight heads
    if (act_dtype == kBFloat16 && inv_freq && rotary_dim == head_dim && tokens >= 64 &&
        (head_dim == 64 || head_dim == 128 || head_dim == 256)) {
        const bool aligned = ((((size_t)qkv) | ((size_t)k_cache) | ((size_t)v_cache)) & 15) == 0 &&
                             (page_stride % 8) == 0;
        if (aligned) {
            const unsigned token_blocks = (unsigned)((tokens + warps - 1) / warps);
            __nv_bfloat16* q = (__nv_bfloat16*)qkv;
            __nv_bfloat16* kc = (__nv_bfloat16*)k_cache;
            __nv_bfloat16* vc = (__nv_bfloat16*)v_cache;
            if (head_dim == 64)
                launch_chained(qk_norm_rope_tokens_vec_kernel<4>, token_blocks, warps * 32, 0, stream, q, kc, vc, args);
            else if (head_dim == 128)
                launch_chained(qk_norm_rope_tokens_vec_kernel<8>, token_blocks, warps * 32, 0, stream, q, kc, vc, args);
            else
                launch_chained(qk_norm_rope_tokens_vec_kernel<16>, token_blocks, warps * 32, 0, stream, q, kc, vc, args);
            return check_launch("qk_norm_rope_store");
        }
        const int run = 8;
        const long long runs = (long long)tokens * ((q_heads + 2 * kv_heads + run - 1) / run);
        const unsigned run_blocks = (unsigned)((runs + warps - 1) / warps);
        __nv_bfloat16* q = (__nv_bfloat16*)qkv;
        __nv_bfloat16* kc = (__nv_bfloat16*)k_cache;
        __nv_bfloat16* vc = (__nv_bfloat16*)v_cache;
        if (head_dim == 64)
            launch_chained(qk_norm_rope_tokens_kernel<__nv_bfloat16, 1>, run_blocks, warps * 32, 0, stream, q, kc, vc, args, run);
        else if (head_dim == 128)
            launch_chained(qk_norm_rope_tokens_kernel<__nv_bfloat16, 2>, run_blocks, warps * 32, 0, stream, q, kc, vc, args, run);
        else
            launch_chained(qk_norm_rope_tokens_kernel<__nv_bfloat16, 4>, run_blocks, warps * 32, 0, stream, q, kc, vc, args, run);
        return check_launch("qk_norm_rope_store");
    }
    if (act_dtype == kFloat32)
        launch_chained(qk_norm_rope_store_kernel<float>, blocks, warps * 32, 0, stream, (float*)qkv,
                       (float*)k_cache, (float*)v_cache, args);
    else if (act_dtype == kBFloat16)
        launch_chained(qk_norm_rope_store_kernel<__nv_bfloat16>, blocks, warps * 32, 0, stream,
                       (__nv_bfloat16*)qkv, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, args);
    else
        CELEG_REQUIRE(false, "qk_norm_rope_store: unknown dtype code %d", act_dtype);
    return check_launch("qk_norm_rope_store");
}
