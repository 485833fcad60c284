// Paged grouped-query attention for decoded tokens (one query token per request), bfloat16
// cache, split over the keys ("flash decoding"):
//
//   grid = (key splits, kv heads, tokens); a block serves the G = q_heads / kv_heads query heads
//   that share one kv head over `chunk` consecutive keys, so K and V are read once per group.
//   Each block writes an unnormalised partial result with its running maximum and denominator
//   to scratch memory; the block that finishes last for a (token, kv head) merges the partials
//   (log-sum-exp) and writes the output. No block waits for another: the last one is found with
//   an atomic counter, which it resets for the next launch.
//
// Scores, maxima, exponentials and sums are float32. Any head size that is a multiple of 8 up
// to 256, any group size up to 16, any page size; other shapes go to the general kernel.
//
// Counterpart in celeg: gqa_decode_paged_segment_partial_kernel + gqa_decode_segment_reduce_batch_kernel
// (src/backend/cuda/kernels/attention_paged.cuh:287-368, 456-487), one block per query head.
#include "common.cuh"

namespace celeg_b200 {

constexpr int kDecodeThreads = 128;
constexpr int kMaxGroup = 16;
constexpr int kMaxDecodeHeadDim = 256;

struct DecodeParams {
    const __nv_bfloat16* q;        // [tokens, q_row_stride], head h at h*head_dim
    int q_row_stride;
    __nv_bfloat16* out;            // [tokens, q_heads*head_dim]
    const __nv_bfloat16* k_cache;  // [pages, kv_heads, page_tokens, head_dim]
    const __nv_bfloat16* v_cache;
    long long page_stride;
    const int* positions;          // [tokens]
    const int* token_span;         // [tokens]
    const int* block_table;        // [spans, table_stride]
    int table_stride;
    int q_heads, kv_heads, head_dim, page_tokens, window, chunk, max_splits;
    float scale;
    float* partial_o;              // [tokens, q_heads, max_splits, head_dim]
    float* partial_ml;             // [tokens, q_heads, max_splits, 2]
    int* counters;                 // [tokens, kv_heads], zero between launches
    int* error_flag;
};

__device__ __forceinline__ void bf16x8_to_float(const uint4& raw, float* f) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = __bfloat1622float2(p[i]);
        f[2 * i] = v.x;
        f[2 * i + 1] = v.y;
    }
}

__global__ void __launch_bounds__(kDecodeThreads) attention_decode_kernel(const DecodeParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    chain_release();
    chain_wait();
    const int split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int group = p.q_heads / p.kv_heads;
    const int d = p.head_dim;
    const int pos = p.positions[t];
    const int first = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int total = pos + 1 - first;
    const int n_splits = (total + p.chunk - 1) / p.chunk;
    if (split >= n_splits) return;
    const int begin = first + split * p.chunk;
    const int count = min(p.chunk, pos + 1 - begin);

    // shared: q [group][d] float | scores [group][chunk] float | offsets [chunk] long long | flag
    float* q_s = reinterpret_cast<float*>(smem_raw);
    float* s_s = q_s + group * d;
    long long* off_s = reinterpret_cast<long long*>(s_s + group * p.chunk + ((group * p.chunk + group * d) & 1));
    __shared__ float head_max[kMaxGroup], head_sum[kMaxGroup];
    __shared__ int is_last;

    const int* table = p.block_table + (size_t)p.token_span[t] * p.table_stride;
    for (int i = tid; i < group * d; i += kDecodeThreads) {
        const int g = i / d, c = i % d;
        q_s[i] = __bfloat162float(p.q[(size_t)t * p.q_row_stride + (size_t)(kvh * group + g) * d + c]) * p.scale;
    }
    for (int k = tid; k < count; k += kDecodeThreads) {
        const int key = begin + k;
        const int page = table[key / p.page_tokens];
        if (page < 0) {
            atomicExch(p.error_flag, 2);
            off_s[k] = 0;
        } else {
            off_s[k] = (long long)page * p.page_stride + ((long long)kvh * p.page_tokens + key % p.page_tokens) * d;
        }
    }
    __syncthreads();

    // scores: one key per thread, all heads of the group
    for (int k = tid; k < count; k += kDecodeThreads) {
        const __nv_bfloat16* kr = p.k_cache + off_s[k];
        float acc[kMaxGroup];
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g) acc[g] = 0.0f;
        for (int c = 0; c < d; c += 8) {
            float kf[8];
            bf16x8_to_float(*reinterpret_cast<const uint4*>(kr + c), kf);
#pragma unroll
            for (int g = 0; g < kMaxGroup; ++g) {
                if (g < group) {
                    const float* qg = q_s + g * d + c;
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[g] += qg[i] * kf[i];
                }
            }
        }
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g)
            if (g < group) s_s[g * p.chunk + k] = acc[g];
    }
    __syncthreads();

    // per head: maximum, exponentials, sum (one warp per head, heads round-robin over warps)
    for (int g = warp; g < group; g += kDecodeThreads / 32) {
        float* row = s_s + g * p.chunk;
        float m = -INFINITY;
        for (int k = lane; k < count; k += 32) m = fmaxf(m, row[k]);
        m = warp_max(m);
        float sum = 0.0f;
        for (int k = lane; k < count; k += 32) {
            const float e = expf(row[k] - m);
            row[k] = e;
            sum += e;
        }
        sum = warp_sum(sum);
        if (lane == 0) {
            head_max[g] = m;
            head_sum[g] = sum;
        }
    }
    __syncthreads();

    // weighted sum of values: the block's threads form `lanes_k` groups that take every lanes_k-th
    // key; inside a group a thread owns (head g, dims c..c+7). The groups' sums meet in shared
    // memory (the score rows of heads are no longer needed once every thread has its weights,
    // but they are read during the loop, so the meeting place is the q area plus the tail).
    const int vecs = d / 8;
    const int items = group * vecs;                       // (head, 8 dims) pairs
    const int lanes_k = items >= kDecodeThreads ? 1 : kDecodeThreads / items;
    float* red_s = reinterpret_cast<float*>(off_s + p.chunk);        // [lanes_k][group * d]
    for (int base_item = 0; base_item < items; base_item += kDecodeThreads) {
        const int item = base_item + (lanes_k > 1 ? tid % items : tid);
        const int kg = lanes_k > 1 ? tid / items : 0;
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
        const bool active = item < items && kg < lanes_k;
        const int g = active ? item / vecs : 0, c = active ? (item % vecs) * 8 : 0;
        if (active) {
            const float* row = s_s + g * p.chunk;
#pragma unroll 4
            for (int k = kg; k < count; k += lanes_k) {
                float vf[8];
                bf16x8_to_float(*reinterpret_cast<const uint4*>(p.v_cache + off_s[k] + c), vf);
                const float w = row[k];
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += w * vf[i];
            }
            if (lanes_k > 1) {
                float* dst = red_s + (size_t)kg * group * d + g * d + c;
#pragma unroll
                for (int i = 0; i < 8; ++i) dst[i] = acc[i];
            } else {
                const int h = kvh * group + g;
                float* dst = p.partial_o + (((size_t)t * p.q_heads + h) * p.max_splits + split) * d + c;
#pragma unroll
                for (int i = 0; i < 8; ++i) dst[i] = acc[i];
            }
        }
    }
    if (lanes_k > 1) {
        __syncthreads();
        for (int i = tid; i < group * d; i += kDecodeThreads) {
            float sum = 0.0f;
            for (int kg = 0; kg < lanes_k; ++kg) sum += red_s[(size_t)kg * group * d + i];
            const int h = kvh * group + i / d;
            p.partial_o[(((size_t)t * p.q_heads + h) * p.max_splits + split) * d + i % d] = sum;
        }
    }
    if (tid < group) {
        const int h = kvh * group + tid;
        float* ml = p.partial_ml + (((size_t)t * p.q_heads + h) * p.max_splits + split) * 2;
        ml[0] = head_max[tid];
        ml[1] = head_sum[tid];
    }

    // the block that arrives last merges
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int* counter = p.counters + (size_t)t * p.kv_heads + kvh;
        const int arrived = atomicAdd(counter, 1);
        is_last = arrived == n_splits - 1;
        if (is_last) *counter = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int item = tid; item < group * d; item += kDecodeThreads) {
        const int g = item / d, c = item % d;
        const int h = kvh * group + g;
        const float* ml = p.partial_ml + ((size_t)t * p.q_heads + h) * p.max_splits * 2;
        const float* po = p.partial_o + ((size_t)t * p.q_heads + h) * p.max_splits * d + c;
        float m = -INFINITY;
        for (int s = 0; s < n_splits; ++s) m = fmaxf(m, __ldcg(ml + 2 * s));
        float denom = 0.0f, acc = 0.0f;
        for (int s = 0; s < n_splits; ++s) {
            const float w = expf(__ldcg(ml + 2 * s) - m);
            denom += w * __ldcg(ml + 2 * s + 1);
            acc += w * __ldcg(po + (size_t)s * d);
        }
        p.out[((size_t)t * p.q_heads + h) * d + c] = __float2bfloat16_rn(acc / denom);
    }
}

}  // namespace celeg_b200

using namespace celeg_b200;

// Bytes of scratch the caller must provide for `tokens` query tokens.
CELEG_API long long celeg_attention_decode_scratch_bytes(int tokens, int q_heads, int kv_heads, int head_dim,
                                                         int max_splits) {
    const long long o = (long long)tokens * q_heads * max_splits * head_dim * 4;
    const long long ml = (long long)tokens * q_heads * max_splits * 2 * 4;
    const long long counters = (long long)tokens * kv_heads * 4;
    return o + ml + counters;
}

// `counters` must be zero before the first launch; every launch leaves them zero.
CELEG_API int celeg_attention_decode(const void* q, int q_row_stride, void* out, const void* k_cache,
                                     const void* v_cache, long long page_stride, const int* positions,
                                     const int* token_span, const int* block_table, int table_stride, int tokens,
                                     int q_heads, int kv_heads, int head_dim, int page_tokens, int window,
                                     float scale, int chunk, int max_splits, float* partial_o, float* partial_ml,
                                     int* counters, int* error_flag, cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && q_heads > 0 && kv_heads > 0 && head_dim > 0 && page_tokens > 0,
                  "attention_decode: invalid sizes tokens=%d q_heads=%d kv_heads=%d head_dim=%d page_tokens=%d",
                  tokens, q_heads, kv_heads, head_dim, page_tokens);
    CELEG_REQUIRE(q_heads % kv_heads == 0 && q_heads / kv_heads <= kMaxGroup,
                  "attention_decode: group size %d/%d is not an integer of at most %d", q_heads, kv_heads,
                  kMaxGroup);
    CELEG_REQUIRE(head_dim % 8 == 0 && head_dim <= kMaxDecodeHeadDim,
                  "attention_decode: head_dim %d must be a multiple of 8 of at most %d", head_dim,
                  kMaxDecodeHeadDim);
    CELEG_REQUIRE(q_row_stride % 8 == 0, "attention_decode: q row stride %d must be a multiple of 8", q_row_stride);
    CELEG_REQUIRE(chunk > 0 && max_splits > 0 && max_splits <= 65535 && tokens <= 65535 && kv_heads <= 65535,
                  "attention_decode: invalid split chunk=%d max_splits=%d", chunk, max_splits);
    if (tokens == 0) return 0;
    const int group = q_heads / kv_heads;
    const int items = group * (head_dim / 8);
    const int lanes_k = items >= kDecodeThreads ? 1 : kDecodeThreads / items;
    size_t smem = (size_t)(group * head_dim + group * chunk + 1) * sizeof(float) + (size_t)chunk * sizeof(long long) +
                  (lanes_k > 1 ? (size_t)lanes_k * group * head_dim * sizeof(float) : 0);
    CELEG_REQUIRE(smem <= 200 * 1024, "attention_decode: chunk %d needs %zu bytes of shared memory", chunk, smem);
    if (smem > 40 * 1024) {       // static shared memory counts against the 48 KiB default as well
        const cudaError_t status = cudaFuncSetAttribute(attention_decode_kernel,
                                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        CELEG_REQUIRE(status == cudaSuccess, "attention_decode: %s", cudaGetErrorString(status));
    }
    DecodeParams p;
    p.q = (const __nv_bfloat16*)q;
    p.q_row_stride = q_row_stride;
    p.out = (__nv_bfloat16*)out;
    p.k_cache = (const __nv_bfloat16*)k_cache;
    p.v_cache = (const __nv_bfloat16*)v_cache;
    p.page_stride = page_stride;
    p.positions = positions;
    p.token_span = token_span;
    p.block_table = block_table;
    p.table_stride = table_stride;
    p.q_heads = q_heads;
    p.kv_heads = kv_heads;
    p.head_dim = head_dim;
    p.page_tokens = page_tokens;
    p.window = window;
    p.chunk = chunk;
    p.max_splits = max_splits;
    p.scale = scale;
    p.partial_o = partial_o;
    p.partial_ml = partial_ml;
    p.counters = counters;
    p.error_flag = error_flag;
    dim3 grid(max_splits, kv_heads, tokens);
    launch_chained(attention_decode_kernel, grid, kDecodeThreads, smem, stream, p);
    return check_launch("attention_decode");
}

// ---------------------------------------------------------------------------------------------
// celeg_attention_decode_static: the same kernel for callers that cannot allocate.
//
// Some hosts of this library must not, or cannot, call cudaMalloc when they need attention: a
// serving process that has handed every remaining byte of device memory to its own pool (a
// later cudaMalloc simply fails), or a latency-critical loop for which the implicit
// device-wide synchronisation of cudaMalloc/cudaFree is not acceptable. For them the scratch
// memory of the split-key kernel lives in a fixed array inside this library instead of being
// passed in. This entry point has no counterpart in celeg.
//
// Cost and limits: every GPU that loads this library holds kStaticScratchBytes (8 MiB) until the
// process exits. A call whose partial results, maxima/denominators and counters do not fit is
// refused with an error message, nothing is launched. All calls share the one array: it keeps
// whatever the previous call left, so the counters are cleared on the stream before every
// launch, and two calls that overlap on the GPU (different streams, no ordering between them)
// race on it and give wrong results. The FIRST call on each device looks up the array's device
// address (cudaGetSymbolAddress, with that device current) and remembers it; make that first
// call before any stream capture begins. No cudaMalloc, cudaFree or allocating library routine
// is called here.
#include <mutex>

namespace celeg_b200 {

constexpr long long kStaticScratchBytes = 8ll * 1024 * 1024;
constexpr int kMaxDevices = 64;

// In host code this name is only a handle for cudaGetSymbolAddress, never a pointer to pass on.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

static std::mutex g_static_mutex;
static void* g_static_address[kMaxDevices] = {};

static int static_scratch_for_current_device(void** address) {
    int device = -1;
    cudaError_t status = cudaGetDevice(&device);
    if (status != cudaSuccess || device < 0 || device >= kMaxDevices) {
        set_error("attention_decode_static: cannot tell the current device (%s)",
                  status == cudaSuccess ? "index out of range" : cudaGetErrorString(status));
        return -3;
    }
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (g_static_address[device] == nullptr) {
        void* found = nullptr;
        status = cudaGetSymbolAddress(&found, g_static_scratch);
        if (status != cudaSuccess || found == nullptr) {
            set_error("attention_decode_static: cudaGetSymbolAddress failed on device %d: %s", device,
                      cudaGetErrorString(status));
            return -3;
        }
        g_static_address[device] = found;
    }
    *address = g_static_address[device];
    return 0;
}

}  // namespace celeg_b200

CELEG_API long long celeg_attention_decode_static_capacity() { return kStaticScratchBytes; }

CELEG_API int celeg_attention_decode_static(const void* q, int q_row_stride, void* out, const void* k_cache,
                                            const void* v_cache, long long page_stride, const int* positions,
                                            const int* token_span, const int* block_table, int table_stride,
                                            int tokens, int q_heads, int kv_heads, int head_dim, int page_tokens,
                                            int window, float scale, int chunk, int max_splits, int* error_flag,
                                            cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && q_heads > 0 && kv_heads > 0 && head_dim > 0 && max_splits > 0,
                  "attention_decode_static: invalid sizes tokens=%d q_heads=%d kv_heads=%d head_dim=%d "
                  "max_splits=%d", tokens, q_heads, kv_heads, head_dim, max_splits);
    // layout inside the array, each part on a 256-byte boundary: counters | maxima and sums | partial outputs
    const long long counter_bytes = ((long long)tokens * kv_heads * 4 + 255) / 256 * 256;
    const long long ml_bytes = ((long long)tokens * q_heads * max_splits * 2 * 4 + 255) / 256 * 256;
    const long long o_bytes = (long long)tokens * q_heads * max_splits * head_dim * 4;
    const long long needed = counter_bytes + ml_bytes + o_bytes;
    CELEG_REQUIRE(needed <= kStaticScratchBytes,
                  "attention_decode_static: this call needs %lld bytes of scratch (tokens=%d q_heads=%d "
                  "max_splits=%d head_dim=%d), the built-in array holds %lld; use celeg_attention_decode with "
                  "caller-provided scratch for sizes beyond it", needed, tokens, q_heads, max_splits, head_dim,
                  kStaticScratchBytes);
    if (tokens == 0) return 0;
    void* base = nullptr;
    const int found = static_scratch_for_current_device(&base);
    if (found != 0) return found;
    unsigned char* bytes = static_cast<unsigned char*>(base);
    int* counters = reinterpret_cast<int*>(bytes);
    float* partial_ml = reinterpret_cast<float*>(bytes + counter_bytes);
    float* partial_o = reinterpret_cast<float*>(bytes + counter_bytes + ml_bytes);
    const cudaError_t cleared = cudaMemsetAsync(counters, 0, (size_t)counter_bytes, stream);
    CELEG_REQUIRE(cleared == cudaSuccess, "attention_decode_static: clearing the counters failed: %s",
                  cudaGetErrorString(cleared));
    return celeg_attention_decode(q, q_row_stride, out, k_cache, v_cache, page_stride, positions, token_span,
                                  block_table, table_stride, tokens, q_heads, kv_heads, head_dim, page_tokens,
                                  window, scale, chunk, max_splits, partial_o, partial_ml, counters, error_flag,
                                  stream);
}
