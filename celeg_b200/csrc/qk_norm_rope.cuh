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
//
// The work of one (token, head) unit is a device function, shared by the kernels of qk_norm_rope.cu
// and the decode attention, which does it for its own token. The projection is read past the L1 cache.
#pragma once
#include "common.cuh"

namespace celeg_b200 {

constexpr int kMaxHeadDim = 512;

__device__ __forceinline__ float load_l2(const float* p) { return __ldcg(p); }
__device__ __forceinline__ __nv_bfloat16 load_l2(const __nv_bfloat16* p) {
    const unsigned short raw = __ldcg(reinterpret_cast<const unsigned short*>(p));
    return __ushort_as_bfloat16(raw);
}

struct QkNormRopeArgs {
    const float* q_weight;
    const float* k_weight;
    const float* inv_freq;
    const int* positions;
    const int* token_span;
    const int* block_table;
    int table_stride;
    long long page_stride;
    int tokens, q_heads, kv_heads, head_dim, rotary_dim, page_tokens;
    float eps;
    int store_kv;      // 0: q heads only; 1: k (normalised, rotated) and v go to the cache; 2: k heads are
                       // normalised and rotated in place like q heads, v heads and the cache are left alone
    int* error_flag;
};

// One warp: head `unit % heads` of token `unit / heads`, heads = q_heads + 2 kv_heads.
template <typename A>
__device__ __forceinline__ void qk_norm_rope_unit(A* qkv, A* k_cache, A* v_cache, const QkNormRopeArgs& a,
                                                  const long long unit, const int lane) {
    const float* q_weight = a.q_weight;
    const float* k_weight = a.k_weight;
    const float* inv_freq = a.inv_freq;
    const int* positions = a.positions;
    const int* token_span = a.token_span;
    const int* block_table = a.block_table;
    const int table_stride = a.table_stride;
    const long long page_stride = a.page_stride;
    const int q_heads = a.q_heads, kv_heads = a.kv_heads, head_dim = a.head_dim, rotary_dim = a.rotary_dim;
    const int page_tokens = a.page_tokens, store_kv = a.store_kv;
    const float eps = a.eps;
    int* error_flag = a.error_flag;
    const int heads = q_heads + 2 * kv_heads;
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
        if (store_kv == 2 && !is_k) return;          // k heads in place (below), v heads untouched
    }
    if (!is_q && store_kv != 2) {
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
        for (int i = lane; i < head_dim; i += 32) dst[i] = load_l2(vec + i);
        return;
    }
    const float* weight = is_q ? q_weight : k_weight;
    if (inv_freq && rotary_dim == head_dim && (head_dim & 63) == 0 && head_dim <= 256) {
        // the common shape in one pass: a lane holds its pairs (i, i + half) in registers between the
        // sum of squares and the rotation, so the row is read once and every load is in flight at once
        // (same arithmetic, in the same order, as the general path below)
        const int half_dim = head_dim >> 1;
        const int pairs = head_dim >> 6;                       // per lane: 1, 2 or 4
        float a[4], b[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = lane + 32 * j;
            a[j] = j < pairs ? to_float(load_l2(vec + i)) : 0.0f;
            b[j] = j < pairs ? to_float(load_l2(vec + i + half_dim)) : 0.0f;
        }
        float scale = 1.0f;
        if (weight) {
            // the general path adds x^2 over i = lane, lane + 32, ...: first the a's, then the b's
            float sum = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) sum += a[j] * a[j];
#pragma unroll
            for (int j = 0; j < 4; ++j) sum += b[j] * b[j];
            sum = warp_sum(sum);
            scale = 1.0f / sqrtf(sum / (float)head_dim + eps);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (j < pairs) {
                const int i = lane + 32 * j;
                float x = a[j], y = b[j];
                if (weight) {
                    x = x * scale * weight[i];
                    y = y * scale * weight[i + half_dim];
                }
                float sn, cs;
                sincosf((float)pos * inv_freq[i], &sn, &cs);
                dst[i] = from_float<A>(x * cs - y * sn);
                dst[i + half_dim] = from_float<A>(y * cs + x * sn);
            }
        }
        return;
    }
    float inv = 1.0f;
    if (weight) {
        float sum = 0.0f;
        for (int i = lane; i < head_dim; i += 32) {
            const float x = to_float(load_l2(vec + i));
            sum += x * x;
        }
        sum = warp_sum(sum);
        inv = 1.0f / sqrtf(sum / (float)head_dim + eps);
    }
    const int half = rotary_dim >> 1;
    // rotated part: pairs (i, i + half), i < half
    for (int i = lane; i < half; i += 32) {
        float a = to_float(load_l2(vec + i));
        float b = to_float(load_l2(vec + i + half));
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
        float a = to_float(load_l2(vec + i));
        if (weight) a = a * inv * weight[i];
        dst[i] = from_float<A>(a);
    }
}

}  // namespace celeg_b200
