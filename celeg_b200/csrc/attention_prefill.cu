// Paged causal grouped-query attention for batches that hold prompt portions (and, beside them,
// single decoded tokens), bfloat16, on the tensor cores:
//
//   grid = (query heads, query tiles). A query tile is up to 128 consecutive tokens of one span
//   (a span = what one request brings to the step); 8 warps own 16 query rows each. Keys and
//   values are fetched page by page through the request's block table into shared memory, 64
//   keys at a time (cp.async, XOR-swizzled 16-byte chunks, two tiles in flight: the next one loads
//   while the current one is in the tensor cores), Q K^T and P V run as
//   mma.sync m16n8k16 with float32 accumulators, softmax is online (running maximum and
//   denominator in float32, exponentials by exp2 of pre-scaled scores).
//
// Any head size that is a multiple of 8 up to 256 (padded with zeros to 64, 128 or 256 in shared
// memory), any number of heads and groups, any page size, optional window. A token's keys are
// those of its own request at positions <= its own, whether they were written by this step or by
// earlier ones.
//
// Counterparts in celeg: the ragged path runs gqa_decode_paged_batch_kernel with one block per
// (token, head) walking all keys (src/backend/cuda/kernels/attention_paged.cuh:3-166); its
// single-sequence flash kernel is scalar (src/backend/cuda/kernels/attention_gemm.cuh:15-217).
#include "common.cuh"
#include "mma_tiles.cuh"

namespace celeg_b200 {

constexpr int kPrefillThreads = 256;
constexpr int kBlockM = 128;
constexpr int kBlockN = 64;

struct PrefillParams {
    const __nv_bfloat16* q;        // [tokens, q_row_stride], head h at h*head_dim
    int q_row_stride;
    __nv_bfloat16* out;            // [tokens, q_heads*head_dim]
    const __nv_bfloat16* k_cache;  // [pages, kv_heads, page_tokens, head_dim]
    const __nv_bfloat16* v_cache;
    long long page_stride;
    const int* positions;          // [tokens]
    const int* span_begin;         // [spans + 1]
    const int* block_table;        // [spans, table_stride]
    int table_stride;
    int spans, q_heads, kv_heads, head_dim, page_tokens, window;
    float scale_log2;              // softmax scale * log2(e)
    int* error_flag;
};

template <int D_PAD>
__global__ void __launch_bounds__(kPrefillThreads, D_PAD <= 64 ? 2 : 1) attention_prefill_kernel(const PrefillParams p) {
    constexpr int kChunks = D_PAD / 8;       // 16-byte chunks per row
    constexpr int kKTiles = D_PAD / 16;      // k tiles of Q K^T
    constexpr int kOTiles = D_PAD / 8;       // n tiles of the output
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* kv_s = q_s + kBlockM * D_PAD;          // two stages of [K tile | V tile]
    __shared__ int tile_span, tile_first;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, c2 = (lane & 3) * 2;
    if (tid == 0) {
        int seen = 0, found = -1, first = 0;
        for (int r = 0; r < p.spans; ++r) {
            const int len = p.span_begin[r + 1] - p.span_begin[r];
            const int tiles = (len + kBlockM - 1) / kBlockM;
            if ((int)blockIdx.y < seen + tiles) {
                // the last tile of a span has the most keys: it comes first in launch order (tiles are the
                // slow grid dimension), so that the grid drains with short tiles
                found = r;
                first = (tiles - 1 - ((int)blockIdx.y - seen)) * kBlockM;
                break;
            }
            seen += tiles;
        }
        tile_span = found;
        tile_first = first;
    }
    __syncthreads();
    const int span = tile_span;
    if (span < 0) return;
    const int h = blockIdx.x;
    const int kvh = h / (p.q_heads / p.kv_heads);
    const int d = p.head_dim;
    const int span_len = p.span_begin[span + 1] - p.span_begin[span];
    const int t0 = p.span_begin[span] + tile_first;
    const int rows = min(kBlockM, span_len - tile_first);
    const int pos0 = p.positions[t0];
    const int pos_last = pos0 + rows - 1;
    const int* table = p.block_table + (size_t)span * p.table_stride;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    for (int idx = tid; idx < kBlockM * kChunks; idx += kPrefillThreads) {
        const int r = idx / kChunks, ch = idx % kChunks;
        __nv_bfloat16* dst = q_s + tile_offset<D_PAD>(r, ch);
        if (r < rows && ch * 8 < d)
            cp_async_16(dst, p.q + (size_t)(t0 + r) * p.q_row_stride + (size_t)h * d + ch * 8);
        else
            *reinterpret_cast<uint4*>(dst) = zero;
    }

    float o[kOTiles][4];
#pragma unroll
    for (int i = 0; i < kOTiles; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.0f;
    float run_max[2] = {-INFINITY, -INFINITY};
    float run_sum[2] = {0.0f, 0.0f};

    const int first_key = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int q_row = warp * 16 + g;                 // this thread's first row; the second is q_row + 8

    // asynchronous copy of the key/value tile `kb` into stage `stage`; keys outside [first_key, pos_last] are zeros
    auto load_tile = [&](int kb, int stage) {
        __nv_bfloat16* k_dst = kv_s + (size_t)stage * 2 * kBlockN * D_PAD;
        __nv_bfloat16* v_dst = k_dst + kBlockN * D_PAD;
        for (int idx = tid; idx < kBlockN * kChunks; idx += kPrefillThreads) {
            const int r = idx / kChunks, ch = idx % kChunks;
            const int key = kb * kBlockN + r;
            __nv_bfloat16* kd = k_dst + tile_offset<D_PAD>(r, ch);
            __nv_bfloat16* vd = v_dst + tile_offset<D_PAD>(r, ch);
            bool filled = false;
            if (key >= first_key && key <= pos_last && ch * 8 < d) {     // pages before the window may be gone
                const int page = table[key / p.page_tokens];
                if (page < 0) {
                    atomicExch(p.error_flag, 2);
                } else {
                    const size_t off = (size_t)page * p.page_stride +
                                       ((size_t)kvh * p.page_tokens + key % p.page_tokens) * d + ch * 8;
                    cp_async_16(kd, p.k_cache + off);
                    cp_async_16(vd, p.v_cache + off);
                    filled = true;
                }
            }
            if (!filled) {
                *reinterpret_cast<uint4*>(kd) = zero;
                *reinterpret_cast<uint4*>(vd) = zero;
            }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    const int kb_first = first_key / kBlockN;
    load_tile(kb_first, 0);                          // this group also carries the Q tile's copies
    for (int kb = kb_first, it = 0; kb * kBlockN <= pos_last; ++kb, ++it) {
        const bool more = (kb + 1) * kBlockN <= pos_last;
        if (more) {
            load_tile(kb + 1, (it + 1) & 1);         // that stage was last read two tiles ago (barrier below)
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        const __nv_bfloat16* k_s = kv_s + (size_t)(it & 1) * 2 * kBlockN * D_PAD;
        const __nv_bfloat16* v_s = k_s + kBlockN * D_PAD;

        // S = Q K^T for this warp's 16 rows and the 64 keys of the tile
        float s[kBlockN / 8][4];
#pragma unroll
        for (int i = 0; i < kBlockN / 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[i][e] = 0.0f;
        const int mi = lane >> 3, lr = lane & 7;
#pragma unroll
        for (int kt = 0; kt < kKTiles; ++kt) {
            unsigned a[4];
            ldmatrix_x4(a, q_s + tile_offset<D_PAD>(warp * 16 + (mi & 1) * 8 + lr, kt * 2 + (mi >> 1)));
#pragma unroll
            for (int np = 0; np < kBlockN / 16; ++np) {
                unsigned b[4];
                ldmatrix_x4(b, k_s + tile_offset<D_PAD>(np * 16 + (mi >> 1) * 8 + lr, kt * 2 + (mi & 1)));
                mma_bf16(s[2 * np], a, b[0], b[1]);
                mma_bf16(s[2 * np + 1], a, b[2], b[3]);
            }
        }

        // scale, mask, online softmax. A tile whose last key is not after the warp's first row (and, with
        // a window, whose first key is inside every row's window) needs no mask at all.
        float tile_max[2] = {-INFINITY, -INFINITY};
        const int warp_first_pos = pos0 + warp * 16;
        const bool full_tile = kb * kBlockN + kBlockN - 1 <= warp_first_pos && warp * 16 + 15 < rows &&
                               (p.window <= 0 || kb * kBlockN > warp_first_pos + 15 - p.window);
        if (full_tile) {
#pragma unroll
            for (int nt = 0; nt < kBlockN / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float v = s[nt][e] * p.scale_log2;
                    s[nt][e] = v;
                    tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
                }
            }
        } else {
#pragma unroll
            for (int nt = 0; nt < kBlockN / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int row = q_row + (e >> 1) * 8;
                    const int key = kb * kBlockN + nt * 8 + c2 + (e & 1);
                    const int qpos = pos0 + row;
                    const bool valid = row < rows && key <= qpos && (p.window <= 0 || key > qpos - p.window);
                    const float v = valid ? s[nt][e] * p.scale_log2 : -INFINITY;
                    s[nt][e] = v;
                    tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
                }
            }
        }
        float correction[2], safe_max[2];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            float m = tile_max[half];
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
            const float new_max = fmaxf(run_max[half], m);
            correction[half] = new_max == -INFINITY ? 1.0f : exp2f(run_max[half] - new_max);
            safe_max[half] = new_max == -INFINITY ? 0.0f : new_max;
            run_max[half] = new_max;
            run_sum[half] *= correction[half];
        }
#pragma unroll
        for (int nt = 0; nt < kBlockN / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pv = exp2f(s[nt][e] - safe_max[e >> 1]);      // exp2(-inf) = 0 for masked keys
                s[nt][e] = pv;
                run_sum[e >> 1] += pv;
            }
        }
#pragma unroll
        for (int i = 0; i < kOTiles; ++i) {
            o[i][0] *= correction[0];
            o[i][1] *= correction[0];
            o[i][2] *= correction[1];
            o[i][3] *= correction[1];
        }

        // O += P V
#pragma unroll
        for (int kt = 0; kt < kBlockN / 16; ++kt) {
            unsigned a[4];
            a[0] = pack_bf16(s[2 * kt][0], s[2 * kt][1]);
            a[1] = pack_bf16(s[2 * kt][2], s[2 * kt][3]);
            a[2] = pack_bf16(s[2 * kt + 1][0], s[2 * kt + 1][1]);
            a[3] = pack_bf16(s[2 * kt + 1][2], s[2 * kt + 1][3]);
#pragma unroll
            for (int np = 0; np < kOTiles / 2; ++np) {
                unsigned b[4];
                ldmatrix_x4_trans(b, v_s + tile_offset<D_PAD>(kt * 16 + (mi & 1) * 8 + lr, np * 2 + (mi >> 1)));
                mma_bf16(o[2 * np], a, b[0], b[1]);
                mma_bf16(o[2 * np + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();                             // every warp is done with this stage
    }

    // normalise and store
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        float sum = run_sum[half];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        run_sum[half] = sum > 0.0f ? 1.0f / sum : 0.0f;
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int row = q_row + half * 8;
        if (row >= rows) continue;
        __nv_bfloat16* dst = p.out + ((size_t)(t0 + row) * p.q_heads + h) * d;
#pragma unroll
        for (int i = 0; i < kOTiles; ++i) {
            const int col = i * 8 + c2;
            if (col < d) {
                *reinterpret_cast<unsigned*>(dst + col) =
                    pack_bf16(o[i][half * 2] * run_sum[half], o[i][half * 2 + 1] * run_sum[half]);
            }
        }
    }
}

template <int D_PAD>
static int launch_prefill(const PrefillParams& p, int tiles, cudaStream_t stream) {
    const size_t smem = (size_t)(kBlockM + 4 * kBlockN) * D_PAD * sizeof(__nv_bfloat16);   // Q + two K/V stages
    if (smem > 40 * 1024) {       // static shared memory counts against the 48 KiB default as well
        const cudaError_t status = cudaFuncSetAttribute(attention_prefill_kernel<D_PAD>,
                                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) {
            set_error("attention_prefill: %s", cudaGetErrorString(status));
            return -2;
        }
    }
    dim3 grid(p.q_heads, tiles);
    attention_prefill_kernel<D_PAD><<<grid, kPrefillThreads, smem, stream>>>(p);
    return check_launch("attention_prefill");
}

}  // namespace celeg_b200

using namespace celeg_b200;

CELEG_API int celeg_attention_prefill(const void* q, int q_row_stride, void* out, const void* k_cache,
                                      const void* v_cache, long long page_stride, const int* positions,
                                      const int* span_begin, const int* block_table, int table_stride,
                                      int tokens, int spans, int q_heads, int kv_heads, int head_dim,
                                      int page_tokens, int window, float scale, int* error_flag,
                                      cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && spans >= 0 && q_heads > 0 && kv_heads > 0 && head_dim > 0 && page_tokens > 0,
                  "attention_prefill: invalid sizes tokens=%d spans=%d q_heads=%d kv_heads=%d head_dim=%d "
                  "page_tokens=%d", tokens, spans, q_heads, kv_heads, head_dim, page_tokens);
    CELEG_REQUIRE(q_heads % kv_heads == 0, "attention_prefill: %d query heads are not a multiple of %d kv heads",
                  q_heads, kv_heads);
    CELEG_REQUIRE(head_dim % 8 == 0 && head_dim <= 256,
                  "attention_prefill: head_dim %d must be a multiple of 8 of at most 256", head_dim);
    CELEG_REQUIRE(q_row_stride % 8 == 0, "attention_prefill: q row stride %d must be a multiple of 8",
                  q_row_stride);
    CELEG_REQUIRE(q_heads <= 65535, "attention_prefill: %d heads exceed one launch", q_heads);
    if (tokens == 0 || spans == 0) return 0;
    PrefillParams p;
    p.q = (const __nv_bfloat16*)q;
    p.q_row_stride = q_row_stride;
    p.out = (__nv_bfloat16*)out;
    p.k_cache = (const __nv_bfloat16*)k_cache;
    p.v_cache = (const __nv_bfloat16*)v_cache;
    p.page_stride = page_stride;
    p.positions = positions;
    p.span_begin = span_begin;
    p.block_table = block_table;
    p.table_stride = table_stride;
    p.spans = spans;
    p.q_heads = q_heads;
    p.kv_heads = kv_heads;
    p.head_dim = head_dim;
    p.page_tokens = page_tokens;
    p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.error_flag = error_flag;
    const int tiles = (tokens + kBlockM - 1) / kBlockM + spans;      // upper bound on sum of ceil(len / 64)
    if (head_dim <= 64) return launch_prefill<64>(p, tiles, stream);
    if (head_dim <= 128) return launch_prefill<128>(p, tiles, stream);
    return launch_prefill<256>(p, tiles, stream);
}
