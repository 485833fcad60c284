// Paged causal grouped-query attention, general form: any head size, float32 or bfloat16 cache,
// any mix of spans. One warp per (query token, query head); the 32 lanes take 32 keys at a time
// for the scores and split the head dimension for the weighted sum of values; softmax is online
// (running maximum and denominator) in float32. A token's result depends only on its own keys,
// read in position order, so it is the same bit for bit however the batch was cut.
//
// This is the whole attention of the float32 path and the fall-back of the bfloat16 path for
// head sizes the tensor-core kernels refuse.
//
// Counterpart in celeg: gqa_decode_paged_batch_kernel (src/backend/cuda/kernels/attention_paged.cuh:3-166),
// one block of 64 threads per (row, head) walking the keys one by one.
#include "common.cuh"

namespace celeg_b200 {

constexpr int kAccRegs = 16;     // head_dim <= 32 * kAccRegs

template <typename A>
__global__ void attention_generic_kernel(const A* __restrict__ q, int q_row_stride, A* __restrict__ out,
                                         const A* __restrict__ k_cache, const A* __restrict__ v_cache,
                                         long long page_stride, const int* __restrict__ positions,
                                         const int* __restrict__ token_span,
                                         const int* __restrict__ block_table, int table_stride, int tokens,
                                         int q_heads, int kv_heads, int head_dim, int page_tokens, int window,
                                         float scale, int* __restrict__ error_flag) {
    extern __shared__ float q_smem[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int warps = blockDim.x >> 5;
    const long long unit = (long long)blockIdx.x * warps + warp;
    if (unit >= (long long)tokens * q_heads) return;
    const int t = (int)(unit / q_heads);
    const int h = (int)(unit % q_heads);
    const int kvh = h / (q_heads / kv_heads);
    const int pos = positions[t];
    const int* table = block_table + (size_t)token_span[t] * table_stride;
    float* qs = q_smem + warp * head_dim;
    const A* qv = q + (size_t)t * q_row_stride + (size_t)h * head_dim;
    for (int i = lane; i < head_dim; i += 32) qs[i] = to_float(qv[i]) * scale;
    __syncwarp();

    float acc[kAccRegs];
#pragma unroll
    for (int r = 0; r < kAccRegs; ++r) acc[r] = 0.0f;
    float running_max = -INFINITY;
    float denom = 0.0f;
    const int first_key = window > 0 ? max(0, pos - window + 1) : 0;

    for (int base = first_key; base <= pos; base += 32) {
        const int key = base + lane;
        const bool valid = key <= pos;
        long long offset = 0;
        float score = -INFINITY;
        if (valid) {
            const int page = table[key / page_tokens];
            if (page < 0) {
                atomicExch(error_flag, 2);
            } else {
                offset = (long long)page * page_stride +
                         ((long long)kvh * page_tokens + (key % page_tokens)) * head_dim;
                const A* kv = k_cache + offset;
                float s = 0.0f;
                for (int i = 0; i < head_dim; ++i) s += qs[i] * to_float(kv[i]);
                score = s;
            }
        }
        const float block_max = warp_max(score);
        const float new_max = fmaxf(running_max, block_max);
        if (new_max == -INFINITY) continue;          // nothing readable in this block of keys
        const float correction = expf(running_max - new_max);   // exp(-inf) = 0 on the first block
        const float p = score == -INFINITY ? 0.0f : expf(score - new_max);
        denom = denom * correction + warp_sum(p);
#pragma unroll
        for (int r = 0; r < kAccRegs; ++r) acc[r] *= correction;
        running_max = new_max;
        const int count = min(32, pos - base + 1);
        for (int j = 0; j < count; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const long long oj = __shfl_sync(0xffffffffu, offset, j);
            const A* vv = v_cache + oj;
#pragma unroll
            for (int r = 0; r < kAccRegs; ++r) {
                const int i = lane + 32 * r;
                if (i < head_dim) acc[r] += pj * to_float(vv[i]);
            }
        }
    }
    const float inv = denom > 0.0f ? 1.0f / denom : 0.0f;
    A* ov = out + ((size_t)t * q_heads + h) * head_dim;
#pragma unroll
    for (int r = 0; r < kAccRegs; ++r) {
        const int i = lane + 32 * r;
        if (i < head_dim) ov[i] = from_float<A>(acc[r] * inv);
    }
}

}  // namespace celeg_b200

using namespace celeg_b200;

// q: [tokens, q_row_stride] with head h at columns h*head_dim; out: [tokens, q_heads*head_dim].
CELEG_API int celeg_attention_generic(const void* q, int q_row_stride, void* out, const void* k_cache,
                                      const void* v_cache, long long page_stride, const int* positions,
                                      const int* token_span, const int* block_table, int table_stride,
                                      int tokens, int q_heads, int kv_heads, int head_dim, int page_tokens,
                                      int window, float scale, int* error_flag, int act_dtype,
                                      cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && q_heads > 0 && kv_heads > 0 && head_dim > 0 && page_tokens > 0,
                  "attention: invalid sizes tokens=%d q_heads=%d kv_heads=%d head_dim=%d page_tokens=%d", tokens,
                  q_heads, kv_heads, head_dim, page_tokens);
    CELEG_REQUIRE(q_heads % kv_heads == 0, "attention: %d query heads are not a multiple of %d kv heads", q_heads,
                  kv_heads);
    CELEG_REQUIRE(head_dim <= 32 * kAccRegs, "attention: head_dim %d exceeds %d", head_dim, 32 * kAccRegs);
    if (tokens == 0) return 0;
    const int warps = 4;
    const long long units = (long long)tokens * q_heads;
    const unsigned blocks = (unsigned)((units + warps - 1) / warps);
    const size_t smem = (size_t)warps * head_dim * sizeof(float);
    if (act_dtype == kFloat32)
        attention_generic_kernel<float><<<blocks, warps * 32, smem, stream>>>(
            (const float*)q, q_row_stride, (float*)out, (const float*)k_cache, (const float*)v_cache, page_stride,
            positions, token_span, block_table, table_stride, tokens, q_heads, kv_heads, head_dim, page_tokens,
            window, scale, error_flag);
    else if (act_dtype == kBFloat16)
        attention_generic_kernel<__nv_bfloat16><<<blocks, warps * 32, smem, stream>>>(
            (const __nv_bfloat16*)q, q_row_stride, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_cache,
            (const __nv_bfloat16*)v_cache, page_stride, positions, token_span, block_table, table_stride, tokens,
            q_heads, kv_heads, head_dim, page_tokens, window, scale, error_flag);
    else
        CELEG_REQUIRE(false, "attention: unknown dtype code %d", act_dtype);
    return check_launch("attention_generic");
}
