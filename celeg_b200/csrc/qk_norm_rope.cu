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
    const QkNormRopeArgs args = {q_weight, k_weight, inv_freq, positions, token_span, block_table, table_stride,
                                 page_stride, tokens, q_heads, kv_heads, head_dim, rotary_dim, page_tokens, eps,
                                 store_kv, error_flag};
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
