// Stand-alone launch of paged decode attention: one (key split, kv head, token) item per block.
// The item's code and its description are in attention_decode.cuh.
#include "attention_decode.cuh"

namespace celeg_b200 {

struct BlockSync {
    __device__ __forceinline__ void operator()() const { __syncthreads(); }
};

// (the forms are laid out for five blocks per SM at head size 64 with one stage, three with two stages or at head
// size 128: the registers must allow them too)
template <int D_PAD, int BN>
__global__ void __launch_bounds__(kDecodeThreads, (D_PAD == 64 && BN == 32) ? 5 : (D_PAD <= 128 && BN <= 64 && D_PAD * BN <= 4096) ? 3 : 1)
attention_decode_kernel(const DecodeParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    chain_release();
    chain_wait();
    attention_decode_item<D_PAD, BN>(p, blockIdx.x, blockIdx.y, blockIdx.z, smem_raw, threadIdx.x, BlockSync());
}

// One warp an item, four items a block (see attention_decode_item_solo).
template <int D_PAD>
__global__ void __launch_bounds__(kDecodeThreads) attention_decode_solo_kernel(const DecodeParams p, const int items) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    chain_release();
    chain_wait();
    const int warp = threadIdx.x >> 5;
    const int item = blockIdx.x * kDecodeWarps + warp;
    if (item >= items) return;
    attention_decode_item_solo<D_PAD>(p, item % p.kv_heads, item / p.kv_heads,
                                      smem_raw + (size_t)warp * decode_solo_warp_bytes<D_PAD>(), threadIdx.x & 31);
}

template <int D_PAD>
static int launch_decode_solo(const DecodeParams& p, int tokens, cudaStream_t stream) {
    constexpr size_t smem = kDecodeWarps * decode_solo_warp_bytes<D_PAD>();
    if (smem > 40 * 1024) {
        const cudaError_t status = cudaFuncSetAttribute(attention_decode_solo_kernel<D_PAD>,
                                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) {
            set_error("attention_decode: %s", cudaGetErrorString(status));
            return -2;
        }
    }
    const int items = tokens * p.kv_heads;
    launch_chained(attention_decode_solo_kernel<D_PAD>, dim3((items + kDecodeWarps - 1) / kDecodeWarps), kDecodeThreads,
                   smem, stream, p, items);
    return check_launch("attention_decode (one warp an item)");
}

template <int D_PAD, int BN>
static int launch_decode(const DecodeParams& p, dim3 grid, cudaStream_t stream) {
    constexpr size_t smem = decode_item_bytes<D_PAD, BN>();
    // the merge of the splits keeps a maximum and a sum per split (of as many heads as fit) where the K/V tiles were
    constexpr size_t tiles = (size_t)kDecodeWarps * 2 * BN * D_PAD * sizeof(__nv_bfloat16);
    CELEG_REQUIRE((size_t)p.max_splits * 2 * sizeof(float) <= tiles,
                  "attention_decode: the maxima and sums of %d splits do not fit the merge's %zu bytes of shared memory",
                  p.max_splits, tiles);
    if (smem > 40 * 1024) {       // static shared memory counts against the 48 KiB default as well
        const cudaError_t status = cudaFuncSetAttribute(attention_decode_kernel<D_PAD, BN>,
                                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) {
            set_error("attention_decode: %s", cudaGetErrorString(status));
            return -2;
        }
    }
    launch_chained(attention_decode_kernel<D_PAD, BN>, grid, kDecodeThreads, smem, stream, p);
    return check_launch("attention_decode");
}

}  // namespace celeg_b200

using namespace celeg_b200;

static int device_sms() {
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (sms <= 0) sms = 148;
    }
    return sms;
}

static long long g_decode_solo_items = 1536;     // (measured: level with the four-warp form at 1,024 items, ahead from 2,048)

// For measurements: from how many (token, kv head) items on a launch of short contexts gives a warp an item.
CELEG_API void celeg_attention_decode_solo_items(long long items) { g_decode_solo_items = items; }

// Bytes of scratch the caller must provide for `tokens` query tokens.
CELEG_API long long celeg_attention_decode_scratch_bytes(int tokens, int q_heads, int kv_heads, int head_dim,
                                                         int max_splits) {
    const long long o = (long long)tokens * q_heads * max_splits * head_dim * 4;
    const long long ml = (long long)tokens * q_heads * max_splits * 2 * 4;
    const long long counters = (long long)tokens * kv_heads * 4;
    return o + ml + counters;
}

static int attention_decode_checked(const void* q, int q_row_stride, void* out, const void* k_cache,
                                    const void* v_cache, long long page_stride, const int* positions,
                                    const int* token_span, const int* block_table, int table_stride, int tokens,
                                    int q_heads, int kv_heads, int head_dim, int page_tokens, int window, float scale,
                                    int chunk, int max_splits, float* partial_o, float* partial_ml, int* counters,
                                    int* error_flag, int fuse_qk, const float* q_norm_w, const float* k_norm_w,
                                    const float* inv_freq, int rotary_dim, float norm_eps, cudaStream_t stream) {
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
    if (fuse_qk) {
        CELEG_REQUIRE(q_row_stride >= (q_heads + 2 * kv_heads) * head_dim,
                      "attention_decode: with the q/k post-processing fused the rows must hold q, k and v (%d < %d)",
                      q_row_stride, (q_heads + 2 * kv_heads) * head_dim);
        CELEG_REQUIRE(rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0 &&
                          (norm_eps > 0.0f || (!q_norm_w && !k_norm_w)),
                      "attention_decode: rotary_dim %d must be even and at most head_dim %d, eps positive", rotary_dim,
                      head_dim);
    }
    if (tokens == 0) return 0;
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
    p.fuse_qk = fuse_qk;
    p.q_norm_w = q_norm_w;
    p.k_norm_w = k_norm_w;
    p.inv_freq = inv_freq;
    p.rotary_dim = rotary_dim;
    p.norm_eps = norm_eps;
    p.k_cache_w = (__nv_bfloat16*)const_cast<void*>(k_cache);
    p.v_cache_w = (__nv_bfloat16*)const_cast<void*>(v_cache);
    dim3 grid(max_splits, kv_heads, tokens);
    // Short contexts (an item has at most two tiles of keys per warp), or more items than the SMs hold at three a
    // time: a block with one stage of 32 keys per warp needs half the shared memory, so more items run at a
    // time, which is worth more than a warp's next tile arriving under its current one (measured at 64
    // requests: 22.6 -> 18.5 us at 540 keys, 184 -> 173 us at 8,000; at 8 requests of 8,000 keys 42 -> 33 us;
    // with 256 items and fewer the two-stage form is ahead).
    const bool few_keys = chunk <= 256 || (long long)tokens * kv_heads * max_splits >= 3LL * device_sms();
    // ... and with very many such items (one split each) a warp serves an item alone
    if (chunk <= 256 && max_splits == 1 && (head_dim & 1) == 0 && (long long)tokens * kv_heads >= g_decode_solo_items) {
        if (head_dim <= 64) return launch_decode_solo<64>(p, tokens, stream);
        if (head_dim <= 128) return launch_decode_solo<128>(p, tokens, stream);
    }
    if (head_dim <= 64) return few_keys ? launch_decode<64, 32>(p, grid, stream) : launch_decode<64, 64>(p, grid, stream);
    if (head_dim <= 128) return few_keys ? launch_decode<128, 32>(p, grid, stream) : launch_decode<128, 64>(p, grid, stream);
    return launch_decode<256, 32>(p, grid, stream);
}

template <int D_PAD, int BN>
static int resident_blocks_of() {
    constexpr size_t smem = decode_item_bytes<D_PAD, BN>();
    if (smem > 40 * 1024 &&
        cudaFuncSetAttribute(attention_decode_kernel<D_PAD, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
            cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_decode_kernel<D_PAD, BN>, kDecodeThreads, smem) !=
        cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return per_sm * device_sms();
}

// How many blocks of the one-stage form (the form of launches with many blocks) the device holds at a time for
// this head size; the host lays its splits of the keys out against this number. 0 if it cannot be asked.
CELEG_API int celeg_attention_decode_resident_blocks(int head_dim) {
    if (head_dim <= 64) return resident_blocks_of<64, 32>();
    if (head_dim <= 128) return resident_blocks_of<128, 32>();
    return resident_blocks_of<256, 32>();
}

// `counters` must be zero before the first launch; every launch leaves them zero.
CELEG_API int celeg_attention_decode(const void* q, int q_row_stride, void* out, const void* k_cache,
                                     const void* v_cache, long long page_stride, const int* positions,
                                     const int* token_span, const int* block_table, int table_stride, int tokens,
                                     int q_heads, int kv_heads, int head_dim, int page_tokens, int window,
                                     float scale, int chunk, int max_splits, float* partial_o, float* partial_ml,
                                     int* counters, int* error_flag, cudaStream_t stream) {
    return attention_decode_checked(q, q_row_stride, out, k_cache, v_cache, page_stride, positions, token_span,
                                    block_table, table_stride, tokens, q_heads, kv_heads, head_dim, page_tokens, window,
                                    scale, chunk, max_splits, partial_o, partial_ml, counters, error_flag, 0, nullptr,
                                    nullptr, nullptr, 0, 0.0f, stream);
}

// The same with the q/k post-processing of the step's tokens done inside: qkv holds the raw projection
// rows [q heads | k heads | v heads]; per-head RMSNorm (weights may be null) and split-half rotation
// (inv_freq may be null) are applied to q in shared memory and to the token's own key, which is written
// into the cache with its value. The caches are written: no other kernel may read the tokens' own positions
// in them at the same time.
CELEG_API int celeg_attention_decode_fused(void* qkv, int q_row_stride, void* out, void* k_cache, void* v_cache,
                                           long long page_stride, const int* positions, const int* token_span,
                                           const int* block_table, int table_stride, int tokens, int q_heads,
                                           int kv_heads, int head_dim, int page_tokens, int window, float scale,
                                           int chunk, int max_splits, float* partial_o, float* partial_ml,
                                           int* counters, int* error_flag, const float* q_norm_w,
                                           const float* k_norm_w, const float* inv_freq, int rotary_dim, float norm_eps,
                                           cudaStream_t stream) {
    return attention_decode_checked(qkv, q_row_stride, out, k_cache, v_cache, page_stride, positions, token_span,
                                    block_table, table_stride, tokens, q_heads, kv_heads, head_dim, page_tokens, window,
                                    scale, chunk, max_splits, partial_o, partial_ml, counters, error_flag, 1, q_norm_w,
                                    k_norm_w, inv_freq, rotary_dim, norm_eps, stream);
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

#include "attention_decode_static.h"

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
