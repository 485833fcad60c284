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
// The query heads of a group are the rows of a 16-row tensor-core tile (mma.sync m16n8k16), keys and
// values reach shared memory by asynchronous copies through the block table, each warp walks its own
// key tiles. Scores, maxima, exponentials and sums are float32. Any head size that is a multiple of 8
// up to 256, any group size up to 16, any page size; other shapes go to the general kernel.
//
// Counterpart in celeg: gqa_decode_paged_segment_partial_kernel + gqa_decode_segment_reduce_batch_kernel
// (src/backend/cuda/kernels/attention_paged.cuh:287-368, 456-487), one block per query head.
//
// The work of one (key split, kv head, token) item is a device function of a block's four warps; the
// kernels in attention_decode.cu give one item to each block.
#pragma once
#include "common.cuh"
#include "mma_tiles.cuh"

namespace celeg_b200 {

constexpr int kDecodeThreads = 128;
constexpr int kDecodeWarps = kDecodeThreads / 32;
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
    // Optional: the q/k post-processing of the step's own token done here instead of by a kernel of its
    // own. Then q (and the k and v behind it in the same rows: [q heads | k heads | v heads]) is the raw
    // projection; an item normalises and rotates its query heads itself, and the item whose keys include
    // the token's own position does the same for that key, writes it and the value into the cache and uses
    // them from shared memory (nobody else reads that row in this launch).
    int fuse_qk;
    const float* q_norm_w;         // [head_dim] or null
    const float* k_norm_w;
    const float* inv_freq;         // [rotary_dim / 2] or null
    int rotary_dim;
    float norm_eps;
    __nv_bfloat16* k_cache_w;      // the caches again, writable
    __nv_bfloat16* v_cache_w;
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

// Shared memory of one block: Q tile [16][D_PAD] + per warp a K and a V tile [BN][D_PAD], bfloat16.
// After the key loop the K/V area is reused for the warps' partial results (float).
template <int D_PAD, int BN>
__host__ __device__ constexpr size_t decode_smem_bytes() {
    return (size_t)(16 + kDecodeWarps * 2 * BN) * D_PAD * sizeof(__nv_bfloat16);
}

// What the threads of one item share beside the tiles; it lies behind them.
struct DecodeShared {
    float warp_max[kDecodeWarps][16], warp_sum[kDecodeWarps][16];
    float head_max[kMaxGroup], head_sum[kMaxGroup];
    int is_last;
    int pad[3];
    alignas(16) __nv_bfloat16 new_k[kMaxDecodeHeadDim];    // the step's own key and value (fused q/k)
    alignas(16) __nv_bfloat16 new_v[kMaxDecodeHeadDim];
};

// Per-head RMSNorm and split-half rotation of one head that a warp holds in shared memory (element i at
// at(i)), the arithmetic of qk_norm_rope.cuh: sum of squares, reciprocal root, angle and rotation in float32,
// one rounding to bfloat16. `out(i)` is where element i goes (may be the same place).
template <typename At, typename Out>
__device__ __forceinline__ void decode_norm_rope_head(At at, Out out, const float* weight, const float* inv_freq,
                                                      const int head_dim, const int rotary_dim, const float eps,
                                                      const int pos, const int lane) {
    float inv = 1.0f;
    if (weight) {
        float sum = 0.0f;
        for (int i = lane; i < head_dim; i += 32) {
            const float x = __bfloat162float(*at(i));
            sum += x * x;
        }
        sum = warp_sum(sum);
        inv = 1.0f / sqrtf(sum / (float)head_dim + eps);
    }
    const int half = rotary_dim >> 1;
    for (int i = lane; i < half; i += 32) {
        float a = __bfloat162float(*at(i));
        float b = __bfloat162float(*at(i + half));
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
        *out(i) = __float2bfloat16_rn(ra);
        *out(i + half) = __float2bfloat16_rn(rb);
    }
    for (int i = rotary_dim + lane; i < head_dim; i += 32) {
        float a = __bfloat162float(*at(i));
        if (weight) a = a * inv * weight[i];
        *out(i) = __float2bfloat16_rn(a);
    }
}

template <int D_PAD, int BN>
__host__ __device__ constexpr size_t decode_item_bytes() {
    return decode_smem_bytes<D_PAD, BN>() + sizeof(DecodeShared);
}

// 128 threads (`tid` 0..127; `sync` is a barrier among exactly them) serve the `group` query heads that share kv head `kvh` for token t over `chunk` keys.
// The heads are the rows of a 16-row MMA tile (rows past `group` are zero). Each of the 4 warps walks
// its own key tiles (BN keys at a time): asynchronous copies of K and V through the block table into
// the warp's shared memory, Q K^T and P V on mma.sync, online softmax in float32; no block-wide
// barrier inside the loop. Then the warps' results are merged in shared memory, and the block
// either writes the output (one split) or a partial for the last block to merge.
template <int D_PAD, int BN, typename Sync>
__device__ __forceinline__ void attention_decode_item(const DecodeParams& p, const int split, const int kvh, const int t,
                                                      unsigned char* smem_raw, const int tid, Sync sync) {
    constexpr int kChunks = D_PAD / 8;
    constexpr int kKTiles = D_PAD / 16;
    constexpr int kOTiles = D_PAD / 8;
    constexpr int kStages = (D_PAD <= 128 && BN >= 64) ? 2 : 1;     // stages per warp
    constexpr int TN = BN / kStages;                       // keys per stage (the warp's shared memory is BN keys of K and of V)
    constexpr int kKeysPerLane = TN / 32;
    static_assert(TN % 32 == 0, "a stage holds a multiple of 32 keys");
    const int lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, c2 = (lane & 3) * 2;
    const int group = p.q_heads / p.kv_heads;
    const int d = p.head_dim;
    const int pos = p.positions[t];
    const int first = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int total = pos + 1 - first;
    const int n_splits = (total + p.chunk - 1) / p.chunk;
    if (n_splits > p.max_splits) {
        // the launch has fewer blocks than this token has chunks of keys: its output would never be merged.
        // Nothing is counted or written for it; the caller reads code 3.
        if (tid == 0) atomicExch(p.error_flag, 3);
        return;
    }
    if (split >= n_splits) return;
    const int begin = first + split * p.chunk;
    const int end = min(begin + p.chunk, pos + 1);

    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* k_s = q_s + 16 * D_PAD + (size_t)warp * 2 * BN * D_PAD;      // this warp's stages
    DecodeShared& shared = *reinterpret_cast<DecodeShared*>(smem_raw + decode_smem_bytes<D_PAD, BN>());
    float (&warp_max_s)[kDecodeWarps][16] = shared.warp_max;
    float (&warp_sum_s)[kDecodeWarps][16] = shared.warp_sum;
    float (&head_max)[kMaxGroup] = shared.head_max;
    float (&head_sum)[kMaxGroup] = shared.head_sum;
    int& is_last = shared.is_last;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const int* table = p.block_table + (size_t)p.token_span[t] * p.table_stride;

    // The first tile of keys and values is asked for before anything else (the query's own preparation below
    // takes as long as the tile needs to arrive). The token's own key and value may not be in the cache yet:
    // their row is put right in shared memory when the tile is there (see the loop).
    // A warp's part of the shared memory is kStages stages of [K tile | V tile] of TN keys: with two
    // stages the next tile is on its way (page lookups included) while this one is in the tensor cores.
    auto issue = [&](const int tile_begin, const int stage) {
        __nv_bfloat16* k_dst = k_s + (size_t)stage * 2 * TN * D_PAD;
        __nv_bfloat16* v_dst = k_dst + TN * D_PAD;
        // page offsets of this lane's keys, then the copies of the whole tile in one go
        long long offs[kKeysPerLane];
#pragma unroll
        for (int i = 0; i < kKeysPerLane; ++i) {
            const int key = tile_begin + lane + 32 * i;
            offs[i] = -1;
            if (key < end) {
                const int page = table[key / p.page_tokens];
                if (page < 0)
                    atomicExch(p.error_flag, 2);
                else
                    offs[i] = (long long)page * p.page_stride + ((long long)kvh * p.page_tokens + key % p.page_tokens) * d;
            }
        }
#pragma unroll
        for (int i = 0; i < TN * kChunks / 32; ++i) {
            const int idx = lane + 32 * i;
            const int r = idx / kChunks, ch = idx % kChunks;
            long long off = -1;
#pragma unroll
            for (int j = 0; j < kKeysPerLane; ++j) {
                const long long candidate = __shfl_sync(0xffffffffu, offs[j], r & 31);
                if ((r >> 5) == j) off = candidate;
            }
            __nv_bfloat16* kd = k_dst + tile_offset<D_PAD>(r, ch);
            __nv_bfloat16* vd = v_dst + tile_offset<D_PAD>(r, ch);
            if (off >= 0 && ch * 8 < d) {
                cp_async_16(kd, p.k_cache + off + ch * 8);
                cp_async_16(vd, p.v_cache + off + ch * 8);
            } else {
                *reinterpret_cast<uint4*>(kd) = zero;
                *reinterpret_cast<uint4*>(vd) = zero;
            }
        }
        cp_async_commit();
    };
    constexpr int kTileStride = kDecodeWarps * TN;
    int tile_begin = begin + warp * TN;
    if (kStages == 2 && tile_begin < end) issue(tile_begin, 0);
    for (int idx = tid; idx < 16 * kChunks; idx += kDecodeThreads) {
        const int r = idx / kChunks, ch = idx % kChunks;
        __nv_bfloat16* dst = q_s + tile_offset<D_PAD>(r, ch);
        if (r < group && ch * 8 < d)
            *reinterpret_cast<uint4*>(dst) = __ldcg(reinterpret_cast<const uint4*>(
                p.q + (size_t)t * p.q_row_stride + (size_t)(kvh * group + r) * d + ch * 8));
        else
            *reinterpret_cast<uint4*>(dst) = zero;
    }
    sync();
    const bool own_key_here = p.fuse_qk && end == pos + 1;       // this item's keys include the token's own
    if (p.fuse_qk) {
        const int rotary = p.inv_freq ? p.rotary_dim : (d & ~1);    // without rotation the pair loop just normalises
        // the query heads of the group, in place in their tile: a warp per head
        for (int r = warp; r < group; r += kDecodeWarps) {
            auto at = [&](int i) { return q_s + tile_offset<D_PAD>(r, i >> 3) + (i & 7); };
            decode_norm_rope_head(at, at, p.q_norm_w, p.inv_freq, d, rotary, p.norm_eps, pos, lane);
        }
        if (own_key_here) {
            // the token's own key (warp 0) and value (warp 1): into shared memory and into the cache
            const int page = table[pos / p.page_tokens];
            if (page < 0) {
                if (tid == 0) atomicExch(p.error_flag, 1);
            } else {
                const long long cache_at = (long long)page * p.page_stride +
                                           ((long long)kvh * p.page_tokens + pos % p.page_tokens) * d;
                const __nv_bfloat16* row = p.q + (size_t)t * p.q_row_stride;
                if (warp == 0) {
                    const __nv_bfloat16* raw = row + (size_t)(p.q_heads + kvh) * d;
                    for (int i = lane; i < d; i += 32) shared.new_k[i] = __ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(raw + i)));
                    __syncwarp();
                    auto at = [&](int i) { return shared.new_k + i; };
                    decode_norm_rope_head(at, at, p.k_norm_w, p.inv_freq, d, rotary, p.norm_eps, pos, lane);
                    __syncwarp();
                    for (int i = lane; i < d; i += 32) p.k_cache_w[cache_at + i] = shared.new_k[i];
                } else if (warp == 1) {
                    const __nv_bfloat16* raw = row + (size_t)(p.q_heads + p.kv_heads + kvh) * d;
                    for (int i = lane; i < d; i += 32) {
                        const __nv_bfloat16 v = __ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(raw + i)));
                        shared.new_v[i] = v;
                        p.v_cache_w[cache_at + i] = v;
                    }
                }
            }
        }
        sync();
    }

    float o[kOTiles][4];
#pragma unroll
    for (int i = 0; i < kOTiles; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.0f;
    float run_max[2] = {-INFINITY, -INFINITY};
    float run_sum[2] = {0.0f, 0.0f};
    const float scale_log2 = p.scale * 1.4426950408889634f;
    const int mi = lane >> 3, lr = lane & 7;

    for (int iteration = 0; tile_begin < end; ++iteration, tile_begin += kTileStride) {
        const int stage = kStages == 2 ? (iteration & 1) : 0;
        if (kStages == 2) {
            if (tile_begin + kTileStride < end) {
                issue(tile_begin + kTileStride, stage ^ 1);
                cp_async_wait_group<1>();
            } else {
                cp_async_wait_group<0>();
            }
        } else {
            issue(tile_begin, 0);
            cp_async_wait_group<0>();
        }
        __syncwarp();
        __nv_bfloat16* k_t = k_s + (size_t)stage * 2 * TN * D_PAD;
        __nv_bfloat16* v_t = k_t + TN * D_PAD;
        if (own_key_here && pos >= tile_begin && pos < tile_begin + TN) {
            // the token's own key and value: not in the cache for this launch's readers, but in shared memory
            const int r = pos - tile_begin;
            for (int ch = lane; ch * 8 < d; ch += 32) {
                *reinterpret_cast<uint4*>(k_t + tile_offset<D_PAD>(r, ch)) = *reinterpret_cast<const uint4*>(shared.new_k + ch * 8);
                *reinterpret_cast<uint4*>(v_t + tile_offset<D_PAD>(r, ch)) = *reinterpret_cast<const uint4*>(shared.new_v + ch * 8);
            }
            __syncwarp();
        }

        float s[TN / 8][4];
#pragma unroll
        for (int i = 0; i < TN / 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[i][e] = 0.0f;
#pragma unroll
        for (int kt = 0; kt < kKTiles; ++kt) {
            unsigned a[4];
            ldmatrix_x4(a, q_s + tile_offset<D_PAD>((mi & 1) * 8 + lr, kt * 2 + (mi >> 1)));
#pragma unroll
            for (int np = 0; np < TN / 16; ++np) {
                unsigned b[4];
                ldmatrix_x4(b, k_t + tile_offset<D_PAD>(np * 16 + (mi >> 1) * 8 + lr, kt * 2 + (mi & 1)));
                mma_bf16(s[2 * np], a, b[0], b[1]);
                mma_bf16(s[2 * np + 1], a, b[2], b[3]);
            }
        }
        float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < TN / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = tile_begin + nt * 8 + c2 + (e & 1);
                const float v = key < end ? s[nt][e] * scale_log2 : -INFINITY;
                s[nt][e] = v;
                tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
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
        for (int nt = 0; nt < TN / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pv = exp2f(s[nt][e] - safe_max[e >> 1]);
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
#pragma unroll
        for (int kt = 0; kt < TN / 16; ++kt) {
            unsigned a[4];
            a[0] = pack_bf16(s[2 * kt][0], s[2 * kt][1]);
            a[1] = pack_bf16(s[2 * kt][2], s[2 * kt][3]);
            a[2] = pack_bf16(s[2 * kt + 1][0], s[2 * kt + 1][1]);
            a[3] = pack_bf16(s[2 * kt + 1][2], s[2 * kt + 1][3]);
#pragma unroll
            for (int np = 0; np < kOTiles / 2; ++np) {
                unsigned b[4];
                ldmatrix_x4_trans(b, v_t + tile_offset<D_PAD>(kt * 16 + (mi & 1) * 8 + lr, np * 2 + (mi >> 1)));
                mma_bf16(o[2 * np], a, b[0], b[1]);
                mma_bf16(o[2 * np + 1], a, b[2], b[3]);
            }
        }
            __syncwarp();                               // every lane is done with the stage before it is refilled
    }

    // row sums over the four lanes that share a row; then the warps' results meet in shared memory
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        run_sum[half] += __shfl_xor_sync(0xffffffffu, run_sum[half], 1);
        run_sum[half] += __shfl_xor_sync(0xffffffffu, run_sum[half], 2);
    }
    sync();                                // every warp is done with its K/V tiles
    float* o_s = reinterpret_cast<float*>(smem_raw + 16 * D_PAD * sizeof(__nv_bfloat16));   // [warps][group][D_PAD]
    if ((lane & 3) == 0) {
        warp_max_s[warp][g] = run_max[0];
        warp_max_s[warp][g + 8] = run_max[1];
        warp_sum_s[warp][g] = run_sum[0];
        warp_sum_s[warp][g + 8] = run_sum[1];
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = g + half * 8;
        if (r < group) {
#pragma unroll
            for (int i = 0; i < kOTiles; ++i) {
                float* dst = o_s + ((size_t)warp * group + r) * D_PAD + i * 8 + c2;
                dst[0] = o[i][half * 2];
                dst[1] = o[i][half * 2 + 1];
            }
        }
    }
    sync();
    if (tid < group) {
        float m = -INFINITY;
        for (int w = 0; w < kDecodeWarps; ++w) m = fmaxf(m, warp_max_s[w][tid]);
        float sum = 0.0f;
        for (int w = 0; w < kDecodeWarps; ++w)
            sum += warp_max_s[w][tid] == -INFINITY ? 0.0f : warp_sum_s[w][tid] * exp2f(warp_max_s[w][tid] - m);
        head_max[tid] = m;
        head_sum[tid] = sum;
    }
    sync();
    for (int i = tid; i < group * d; i += kDecodeThreads) {
        const int r = i / d, col = i % d;
        const float m = head_max[r];
        float v = 0.0f;
        for (int w = 0; w < kDecodeWarps; ++w) {
            const float wm = warp_max_s[w][r];
            if (wm != -INFINITY) v += o_s[((size_t)w * group + r) * D_PAD + col] * exp2f(wm - m);
        }
        const int h = kvh * group + r;
        if (n_splits == 1)
            p.out[((size_t)t * p.q_heads + h) * d + col] = __float2bfloat16_rn(v / head_sum[r]);
        else
            p.partial_o[(((size_t)t * p.q_heads + h) * p.max_splits + split) * d + col] = v;
    }
    if (n_splits == 1) return;
    if (tid < group) {
        const int h = kvh * group + tid;
        float* ml = p.partial_ml + (((size_t)t * p.q_heads + h) * p.max_splits + split) * 2;
        ml[0] = head_max[tid];                      // in units of log2: exponentials below use exp2
        ml[1] = head_sum[tid];
    }

    // the item that arrives last merges the splits
    __threadfence();
    sync();
    if (tid == 0) {
        int* counter = p.counters + (size_t)t * p.kv_heads + kvh;
        const int arrived = atomicAdd(counter, 1);
        is_last = arrived == n_splits - 1;
        if (is_last) *counter = 0;
    }
    sync();
    if (!is_last) return;
    __threadfence();
    // More than eight splits: the merge in three short phases, so that it costs few round trips to the L2 at the
    // very end of the kernel whatever their number (a single request with 130 k keys has 37): all maxima and sums of the
    // group's heads into shared memory in one go; a warp per head turns them into the splits' weights and the
    // head's sum; then a thread takes two outputs together and the splits' partial outputs in batches of eight.
    // (One load after the other it was 2 n round trips for n splits; a pass over the maxima before the pass over
    // the outputs, one output after the other, 4 ceil(n / 8).) The K/V tiles' shared memory holds the weights;
    // if all heads' do not fit at once the heads are taken in several passes (the launch checks that one head's do).
    if (n_splits <= 8) {
        // the common case in one round trip an output: maxima, sums and outputs of all splits together
        for (int item = tid; item < group * d; item += kDecodeThreads) {
            const int r = item / d, col = item % d;
            const int h = kvh * group + r;
            const float* ml = p.partial_ml + ((size_t)t * p.q_heads + h) * p.max_splits * 2;
            const float* po = p.partial_o + ((size_t)t * p.q_heads + h) * p.max_splits * d + col;
            float part_m[8], part_l[8], part_o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const bool have = j < n_splits;
                part_m[j] = have ? __ldcg(ml + 2 * j) : -INFINITY;
                part_l[j] = have ? __ldcg(ml + 2 * j + 1) : 0.0f;
                part_o[j] = have ? __ldcg(po + (size_t)j * d) : 0.0f;
            }
            float m = -INFINITY, denom = 0.0f, total_o = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) m = fmaxf(m, part_m[j]);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (j < n_splits) {
                    const float w = exp2f(part_m[j] - m);
                    denom += w * part_l[j];
                    total_o += w * part_o[j];
                }
            }
            p.out[((size_t)t * p.q_heads + h) * d + col] = __float2bfloat16_rn(total_o / denom);
        }
        return;
    }
    constexpr int kMergeFloats = kDecodeWarps * 2 * BN * D_PAD / 2;      // the K/V tiles, counted in floats
    const int heads_a_pass = max(1, min(group, kMergeFloats / (2 * n_splits)));
    for (int r0 = 0; r0 < group; r0 += heads_a_pass) {
        const int heads = min(heads_a_pass, group - r0);
        float* merge_w = o_s;                              // [heads][n_splits] maxima, then weights
        float* merge_l = o_s + (size_t)heads * n_splits;   // [heads][n_splits] sums
        for (int idx = tid; idx < heads * n_splits; idx += kDecodeThreads) {
            const int r = r0 + idx / n_splits, j = idx % n_splits;
            const float* ml = p.partial_ml + (((size_t)t * p.q_heads + kvh * group + r) * p.max_splits + j) * 2;
            merge_w[idx] = __ldcg(ml);
            merge_l[idx] = __ldcg(ml + 1);
        }
        sync();
        for (int i = warp; i < heads; i += kDecodeWarps) {
            float* w_r = merge_w + (size_t)i * n_splits;
            const float* l_r = merge_l + (size_t)i * n_splits;
            float m = -INFINITY;
            for (int j = lane; j < n_splits; j += 32) m = fmaxf(m, w_r[j]);
            m = warp_max(m);
            float denom = 0.0f;
            for (int j = lane; j < n_splits; j += 32) {
                const float w = exp2f(w_r[j] - m);
                w_r[j] = w;
                denom += w * l_r[j];
            }
            denom = warp_sum(denom);
            if (lane == 0) head_sum[r0 + i] = denom;
        }
        sync();
        const int outputs = heads * d;
        for (int base = 0; base < outputs; base += 2 * kDecodeThreads) {
            const float* po[2];
            const float* w_r[2];
            bool live[2];
            float total_o[2] = {0.0f, 0.0f};
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int item = base + tid + u * kDecodeThreads;
                live[u] = item < outputs;
                const int i = live[u] ? item / d : 0, col = live[u] ? item % d : 0;
                po[u] = p.partial_o + ((size_t)t * p.q_heads + kvh * group + r0 + i) * p.max_splits * d + col;
                w_r[u] = merge_w + (size_t)i * n_splits;
            }
            for (int sp0 = 0; sp0 < n_splits; sp0 += 8) {
                float part_o[2][8];
#pragma unroll
                for (int u = 0; u < 2; ++u)
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        part_o[u][j] = live[u] && sp0 + j < n_splits ? __ldcg(po[u] + (size_t)(sp0 + j) * d) : 0.0f;
#pragma unroll
                for (int u = 0; u < 2; ++u)
#pragma unroll
                    for (int j = 0; j < 8; ++j)                  // (in the order of the splits)
                        if (sp0 + j < n_splits) total_o[u] += w_r[u][sp0 + j] * part_o[u][j];
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                if (!live[u]) continue;
                const int item = base + tid + u * kDecodeThreads;
                const int r = r0 + item / d;
                p.out[((size_t)t * p.q_heads + kvh * group + r) * d + item % d] =
                    __float2bfloat16_rn(total_o[u] / head_sum[r]);
            }
        }
        if (r0 + heads_a_pass < group) sync();             // the next pass writes over the weights
    }
}

// ------------------------------------------------------------------------------------------- one warp an item
// Many requests with short contexts (hundreds of tokens x kv heads, at most a few tiles of keys each): an item is
// too little work for four warps. What such a launch then consists of is the blocks' starts and the three
// block-wide barriers at which the warps' partial results meet, not the keys. Here ONE warp serves an item over all
// of its keys (one split), a block holds four independent items, and nothing is exchanged between warps: the
// warp's own accumulators are the result. Same arithmetic per tile as above (and the same fused q/k step).
template <int D_PAD>
__host__ __device__ constexpr size_t decode_solo_warp_bytes() {
    return (size_t)(16 + 2 * 32 + 2) * D_PAD * sizeof(__nv_bfloat16);      // Q tile, K tile, V tile, the own key and value
}

template <int D_PAD>
__device__ __forceinline__ void attention_decode_item_solo(const DecodeParams& p, const int kvh, const int t,
                                                           unsigned char* warp_smem, const int lane) {
    constexpr int TN = 32;
    constexpr int kChunks = D_PAD / 8;
    constexpr int kKTiles = D_PAD / 16;
    constexpr int kOTiles = D_PAD / 8;
    const int g = lane >> 2, c2 = (lane & 3) * 2;
    const int group = p.q_heads / p.kv_heads;
    const int d = p.head_dim;
    const int pos = p.positions[t];
    const int first = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int end = pos + 1;
    if (end - first > p.chunk) {
        // more keys than the launch was laid out for (one split): nothing is written, the caller reads code 3
        if (lane == 0) atomicExch(p.error_flag, 3);
        return;
    }
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(warp_smem);
    __nv_bfloat16* k_t = q_s + 16 * D_PAD;
    __nv_bfloat16* v_t = k_t + TN * D_PAD;
    __nv_bfloat16* new_k = v_t + TN * D_PAD;
    __nv_bfloat16* new_v = new_k + D_PAD;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const int* table = p.block_table + (size_t)p.token_span[t] * p.table_stride;

    auto issue = [&](const int tile_begin) {
        const int key = tile_begin + lane;
        long long mine = -1;
        if (key < end) {
            const int page = table[key / p.page_tokens];
            if (page < 0)
                atomicExch(p.error_flag, 2);
            else
                mine = (long long)page * p.page_stride + ((long long)kvh * p.page_tokens + key % p.page_tokens) * d;
        }
#pragma unroll
        for (int i = 0; i < TN * kChunks / 32; ++i) {
            const int idx = lane + 32 * i;
            const int r = idx / kChunks, ch = idx % kChunks;
            const long long off = __shfl_sync(0xffffffffu, mine, r);
            __nv_bfloat16* kd = k_t + tile_offset<D_PAD>(r, ch);
            __nv_bfloat16* vd = v_t + tile_offset<D_PAD>(r, ch);
            if (off >= 0 && ch * 8 < d) {
                cp_async_16(kd, p.k_cache + off + ch * 8);
                cp_async_16(vd, p.v_cache + off + ch * 8);
            } else {
                *reinterpret_cast<uint4*>(kd) = zero;
                *reinterpret_cast<uint4*>(vd) = zero;
            }
        }
        cp_async_commit();
    };
    issue(first);                                     // the first tile is on its way while the query is prepared
    for (int idx = lane; idx < 16 * kChunks; idx += 32) {
        const int r = idx / kChunks, ch = idx % kChunks;
        __nv_bfloat16* dst = q_s + tile_offset<D_PAD>(r, ch);
        if (r < group && ch * 8 < d)
            *reinterpret_cast<uint4*>(dst) = __ldcg(reinterpret_cast<const uint4*>(
                p.q + (size_t)t * p.q_row_stride + (size_t)(kvh * group + r) * d + ch * 8));
        else
            *reinterpret_cast<uint4*>(dst) = zero;
    }
    __syncwarp();
    if (p.fuse_qk) {
        const int rotary = p.inv_freq ? p.rotary_dim : (d & ~1);
        for (int r = 0; r < group; ++r) {
            auto at = [&](int i) { return q_s + tile_offset<D_PAD>(r, i >> 3) + (i & 7); };
            decode_norm_rope_head(at, at, p.q_norm_w, p.inv_freq, d, rotary, p.norm_eps, pos, lane);
        }
        // the token's own key and value: into shared memory and into the cache
        const int page = table[pos / p.page_tokens];
        if (page < 0) {
            if (lane == 0) atomicExch(p.error_flag, 1);
        } else {
            const long long cache_at = (long long)page * p.page_stride +
                                       ((long long)kvh * p.page_tokens + pos % p.page_tokens) * d;
            const __nv_bfloat16* row = p.q + (size_t)t * p.q_row_stride;
            const __nv_bfloat16* raw_k = row + (size_t)(p.q_heads + kvh) * d;
            const __nv_bfloat16* raw_v = row + (size_t)(p.q_heads + p.kv_heads + kvh) * d;
            for (int i = lane; i < d; i += 32) {
                new_k[i] = __ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(raw_k + i)));
                const __nv_bfloat16 v = __ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(raw_v + i)));
                new_v[i] = v;
                p.v_cache_w[cache_at + i] = v;
            }
            __syncwarp();
            auto at = [&](int i) { return new_k + i; };
            decode_norm_rope_head(at, at, p.k_norm_w, p.inv_freq, d, rotary, p.norm_eps, pos, lane);
            __syncwarp();
            for (int i = lane; i < d; i += 32) p.k_cache_w[cache_at + i] = new_k[i];
        }
        __syncwarp();
    }

    float o[kOTiles][4];
#pragma unroll
    for (int i = 0; i < kOTiles; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.0f;
    float run_max[2] = {-INFINITY, -INFINITY};
    float run_sum[2] = {0.0f, 0.0f};
    const float scale_log2 = p.scale * 1.4426950408889634f;
    const int mi = lane >> 3, lr = lane & 7;

    for (int tile_begin = first; tile_begin < end; tile_begin += TN) {
        if (tile_begin > first) issue(tile_begin);
        cp_async_wait_group<0>();
        __syncwarp();
        if (p.fuse_qk && pos >= tile_begin && pos < tile_begin + TN) {
            const int r = pos - tile_begin;
            for (int ch = lane; ch * 8 < d; ch += 32) {
                *reinterpret_cast<uint4*>(k_t + tile_offset<D_PAD>(r, ch)) = *reinterpret_cast<const uint4*>(new_k + ch * 8);
                *reinterpret_cast<uint4*>(v_t + tile_offset<D_PAD>(r, ch)) = *reinterpret_cast<const uint4*>(new_v + ch * 8);
            }
            __syncwarp();
        }
        float s[TN / 8][4];
#pragma unroll
        for (int i = 0; i < TN / 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[i][e] = 0.0f;
#pragma unroll
        for (int kt = 0; kt < kKTiles; ++kt) {
            unsigned a[4];
            ldmatrix_x4(a, q_s + tile_offset<D_PAD>((mi & 1) * 8 + lr, kt * 2 + (mi >> 1)));
#pragma unroll
            for (int np = 0; np < TN / 16; ++np) {
                unsigned b[4];
                ldmatrix_x4(b, k_t + tile_offset<D_PAD>(np * 16 + (mi >> 1) * 8 + lr, kt * 2 + (mi & 1)));
                mma_bf16(s[2 * np], a, b[0], b[1]);
                mma_bf16(s[2 * np + 1], a, b[2], b[3]);
            }
        }
        float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < TN / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = tile_begin + nt * 8 + c2 + (e & 1);
                const float v = key < end ? s[nt][e] * scale_log2 : -INFINITY;
                s[nt][e] = v;
                tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
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
        for (int nt = 0; nt < TN / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pv = exp2f(s[nt][e] - safe_max[e >> 1]);
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
#pragma unroll
        for (int kt = 0; kt < TN / 16; ++kt) {
            unsigned a[4];
            a[0] = pack_bf16(s[2 * kt][0], s[2 * kt][1]);
            a[1] = pack_bf16(s[2 * kt][2], s[2 * kt][3]);
            a[2] = pack_bf16(s[2 * kt + 1][0], s[2 * kt + 1][1]);
            a[3] = pack_bf16(s[2 * kt + 1][2], s[2 * kt + 1][3]);
#pragma unroll
            for (int np = 0; np < kOTiles / 2; ++np) {
                unsigned b[4];
                ldmatrix_x4_trans(b, v_t + tile_offset<D_PAD>(kt * 16 + (mi & 1) * 8 + lr, np * 2 + (mi >> 1)));
                mma_bf16(o[2 * np], a, b[0], b[1]);
                mma_bf16(o[2 * np + 1], a, b[2], b[3]);
            }
        }
        __syncwarp();                                  // every lane is done with the tile before it is refilled
    }
    // a row's sum over the four lanes that share it; the warp's accumulators are the item's result
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        run_sum[half] += __shfl_xor_sync(0xffffffffu, run_sum[half], 1);
        run_sum[half] += __shfl_xor_sync(0xffffffffu, run_sum[half], 2);
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = g + half * 8;
        if (r >= group) continue;
        const float inv = 1.0f / run_sum[half];
        __nv_bfloat16* dst = p.out + ((size_t)t * p.q_heads + kvh * group + r) * d;
#pragma unroll
        for (int i = 0; i < kOTiles; ++i) {
            const int col = i * 8 + c2;
            if (col + 1 < d) {
                *reinterpret_cast<__nv_bfloat162*>(dst + col) = __floats2bfloat162_rn(o[i][half * 2] * inv, o[i][half * 2 + 1] * inv);
            } else if (col < d) {
                dst[col] = __float2bfloat16_rn(o[i][half * 2] * inv);
            }
        }
    }
}

}  // namespace celeg_b200
