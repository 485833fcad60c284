// Post-processing of the fused q|k|v projection, one warp per (token, head):
//   q heads:  per-head RMSNorm (weight [d]) -> split-half rotary embedding -> written back in place
//   k heads:  per-head RMSNorm -> rotary embedding -> written into the request's cache page
//   v heads:  copied into the cache page
// Sum of squares, reciprocal root, angle (position * inv_freq[i]) and the rotation are float32;
// the result is rounded once to the cache / activation type.
//
// Cache layout of one layer: [page][kv_head][slot in page][d], so one (page, head) tile is a
// contiguous [page_tokens, d] box.
//
// Counterparts in celeg (5-6 launches): per-head rmsnorm (include/celeg/backend/cuda/attention_norm.hpp:25-63),
// paired_qk_norm_rope_kernel (src/backend/cuda/kernels/rope_pairing.cu:82-176), scale_kernel,
// store_kv_paged_batch_kernel (src/backend/cuda/kernels/kv_cache.cuh:215-).
#include "common.cuh"

namespace celeg_b200 {

constexpr int kMaxHeadDim = 512;

template <typename A>
__global__ void qk_norm_rope_store_kernel(A* qkv, const float* __restrict__ q_weight,
                                          const float* __restrict__ k_weight,
                                          const float* __restrict__ inv_freq, const int* positions,
                                          const int* token_span,
                                          const int* block_table, int table_stride,
                                          A* k_cache, A* v_cache,
                                          long long page_stride, int tokens, int q_heads, int kv_heads,
                                          int head_dim, int rotary_dim, int page_tokens, float eps,
                                          int store_kv, int* error_flag) {
    chain_release();
    chain_wait();
    const int warps_per_block = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    const int heads = q_heads + 2 * kv_heads;
    const long long unit = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    if (unit >= (long long)tokens * heads) return;
    const int t = (int)(unit / heads);
    const int h = (int)(unit % heads);
    A* vec = qkv + ((size_t)t * heads + h) * head_dim;
    const int pos = positions[t];
    const bool is_q = h < q_heads;
    const bool is_k = !is_q && h < q_heads + kv_heads;
    const int kvh = is_q ? 0 : (is_k ? h - q_heads : h - q_heads - kv_heads);

    A* dst = vec;
    if (!is_q) {
        if (!store_kv) return;
        const int logical = pos / page_tokens;
        const int page = block_table[(size_t)token_span[t] * table_stride + logical];
        if (page < 0) {                              // the host never builds such a table
            if (lane == 0) atomicExch(error_flag, 1);
            return;
        }
        A* base = is_k ? k_cache : v_cache;
        dst = base + (size_t)page * page_stride + ((size_t)kvh * page_tokens + (pos % page_tokens)) * head_dim;
    }
    if (!is_q && !is_k) {                            // v: plain copy
        for (int i = lane; i < head_dim; i += 32) dst[i] = vec[i];
        return;
    }
    const float* weight = is_q ? q_weight : k_weight;
    float inv = 1.0f;
    if (weight) {
        float sum = 0.0f;
        for (int i = lane; i < head_dim; i += 32) {
            const float x = to_float(vec[i]);
            sum += x * x;
        }
        sum = warp_sum(sum);
        inv = 1.0f / sqrtf(sum / (float)head_dim + eps);
    }
    const int half = rotary_dim >> 1;
    // rotated part: pairs (i, i + half), i < half
    for (int i = lane; i < half; i += 32) {
        float a = to_float(vec[i]);
        float b = to_float(vec[i + half]);
        if (weight) {
            a = a * inv * weight[i];
            b = b * inv * weight[i + half];
        }
        float ra = a, rb = b;
        if (inv_freq) {
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            ra = a * cs - b * sn;
            rb = b * cs + a * sn;
        }
        dst[i] = from_float<A>(ra);
        dst[i + half] = from_float<A>(rb);
    }
    // pass-through part beyond the rotary dimensions
    for (int i = rotary_dim + lane; i < head_dim; i += 32) {
        float a = to_float(vec[i]);
        if (weight) a = a * inv * weight[i];
        dst[i] = from_float<A>(a);
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
    if (tokens == 0) return 0;
    const long long units = (long long)tokens * (q_heads + 2 * kv_heads);
    const int warps = 4;
    const unsigned blocks = (unsigned)((units + warps - 1) / warps);
    if (!inv_freq) rotary_dim = head_dim & ~1;       // without rotation the pair loop just normalises
    if (act_dtype == kFloat32)
        launch_chained(qk_norm_rope_store_kernel<float>, blocks, warps * 32, 0, stream,
            (float*)qkv, q_weight, k_weight, inv_freq, positions, token_span, block_table, table_stride,
            (float*)k_cache, (float*)v_cache, page_stride, tokens, q_heads, kv_heads, head_dim, rotary_dim,
            page_tokens, eps, store_kv, error_flag);
    else if (act_dtype == kBFloat16)
        launch_chained(qk_norm_rope_store_kernel<__nv_bfloat16>, blocks, warps * 32, 0, stream,
            (__nv_bfloat16*)qkv, q_weight, k_weight, inv_freq, positions, token_span, block_table, table_stride,
            (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, page_stride, tokens, q_heads, kv_heads, head_dim,
            rotary_dim, page_tokens, eps, store_kv, error_flag);
    else
        CELEG_REQUIRE(false, "qk_norm_rope_store: unknown dtype code %d", act_dtype);
    return check_launch("qk_norm_rope_store");
}
