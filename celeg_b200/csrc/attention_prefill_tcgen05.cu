// Paged causal grouped-query attention for prompt portions on Blackwell's fifth-generation tensor
// cores, for a head size of 64 (bfloat16):
//
//   grid = (query heads, query tiles); a query tile is up to 128 consecutive tokens of one span; tiles with
//   many keys come first in launch order, so that the grid drains with short ones.
//   Six warps. Warp 0 brings Q (one box of 128 rows x 64) and, per block of 64 keys, the K and V
//   rows page by page through the request's block table into a four-stage ring by TMA (128-byte
//   swizzle; a page is one box of page_tokens rows x 64): lane 0 waits for the stage, then lane 2 pg brings
//   page pg of K and lane 2 pg + 1 that of V, each looked up one block ahead (one thread issuing a block's
//   up to 16 copies in turn took longer than the block's softmax). Warp 1 issues the MMAs:
//       S[128 x 64] = Q K^T           (tcgen05.mma M128 N64 K16 x 4, both operands K-major)
//       O[128 x 64] += P V            (M128 N64 K16 x 4, P from tensor memory as the A operand, V as it lies
//                                      in the cache, keys x 64: the MN-major form of the B operand)
//   with S, P and O in tensor memory. S and P exist twice (even and odd blocks of keys): the scores of block
//   j+1 are being multiplied while the softmax threads work on block j, and P V of block j runs while they
//   work on block j+1. 256 columns of tensor memory and 81 KiB of shared memory a block: two blocks per SM.
//   Warps 2-5 are the softmax: a thread owns one query row (its TMEM lane), reads S with tcgen05.ld, masks
//   (causal, window, rows past the span; blocks that every row sees whole skip the mask), takes the maximum,
//   writes P = exp2(scaled S - maximum) as bfloat16 pairs into tensor memory with tcgen05.st and adds to its
//   denominator, all in float32 (packed f32x2 arithmetic, three-input maxima). O stays in tensor memory: the
//   maximum that P is relative to follows the true running maximum only when that has grown by more than 2^8,
//   and only then the warp rescales its rows of O (tcgen05.ld, multiply, tcgen05.st); at the end a thread
//   divides its row by the denominator and writes it. No shuffles: a row is one thread. Every tensor-memory
//   load, store and wait is taken by all lanes of a warp (they are .sync.aligned); only stores to global
//   memory are conditional.
//   Every wait on an mbarrier is bounded (tcgen05.cuh); a role that gives up records a code, and the
//   block leaves through the common exit (tensor memory released).
//
// Head sizes other than 64, pages that are no multiple of 8 tokens or do not divide 64, and float32
// go to attention_prefill.cu (mma.sync) or attention_generic.cu.
//
// Counterparts in celeg: see attention_prefill.cu.
#include "tcgen05.cuh"

namespace celeg_b200 {

constexpr int kFaThreads = 192;
constexpr int kFaM = 128;                 // query rows per tile
constexpr int kFaN = 64;                  // keys per block
constexpr int kFaD = 64;
constexpr unsigned kFaQBytes = kFaM * kFaD * 2;         // 16 KiB
constexpr unsigned kFaKvBytes = kFaN * kFaD * 2;        // 8 KiB each for K and V
constexpr int kFaStages = 4;
constexpr unsigned kFaSmemBytes = kFaQBytes + kFaStages * 2 * kFaKvBytes + 1024;
// Tensor memory: S of even and odd blocks at columns 0..63 and 64..127, O at 128..191, P (bfloat16, two keys a
// column) of even and odd blocks at 192..223 and 224..255
constexpr unsigned kFaTmemColumns = 256;
constexpr unsigned kFaOColumn = 2 * kFaN, kFaPColumn = 2 * kFaN + kFaD;

struct FaParams {
    __nv_bfloat16* out;            // [tokens, q_heads * 64]
    const int* positions;          // [tokens]
    const int* span_begin;         // [spans + 1]
    const int* block_table;        // [spans, table_stride]
    int table_stride;
    int spans, q_heads, kv_heads, page_tokens, window;
    float scale_log2;              // softmax scale * log2(e)
    int* error_flag;
};

__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive_one(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}

// The MN-major form of the instruction descriptor's B operand (bit 16): B is read as [k][n] with n contiguous.
__host__ __device__ constexpr unsigned instruction_descriptor_b_mn(int m, int n) {
    return instruction_descriptor(m, n) | (1u << 16);
}

__global__ void __launch_bounds__(kFaThreads)
attention_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                 const __grid_constant__ CUtensorMap map_v, const FaParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long q_full, kv_full[kFaStages], kv_empty[kFaStages], s_full[2], p_full[2],
        o_full[2];
    __shared__ unsigned tmem_base_slot;
    __shared__ int tile_span, tile_first;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        int seen = 0, found = -1, first = 0;
        for (int r = 0; r < p.spans; ++r) {
            const int len = p.span_begin[r + 1] - p.span_begin[r];
            const int tiles = (len + kFaM - 1) / kFaM;
            if ((int)blockIdx.y < seen + tiles) {
                // the last tile of a span has the most keys: it goes first, so that the blocks that are
                // still running when the grid drains are the short ones
                found = r;
                first = (tiles - 1 - ((int)blockIdx.y - seen)) * kFaM;
                break;
            }
            seen += tiles;
        }
        tile_span = found;
        tile_first = first;
        mbar_init(smem_u32(&q_full), 1);
        for (int s = 0; s < kFaStages; ++s) {
            mbar_init(smem_u32(&kv_full[s]), 1);
            mbar_init(smem_u32(&kv_empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&s_full[b]), 1);
            mbar_init(smem_u32(&p_full[b]), 128);
            mbar_init(smem_u32(&o_full[b]), 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) tmem_alloc(smem_u32(&tmem_base_slot), kFaTmemColumns);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const unsigned tmem_base = tmem_base_slot;
    const int span = tile_span;

    const unsigned smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const unsigned q_addr = smem_base;
    const unsigned kv_addr = q_addr + kFaQBytes;                       // stage s: K at +s*2*kv, V behind it

    int error = 0;
    if (span >= 0) {
        const int h = blockIdx.x;
        const int kvh = h / (p.q_heads / p.kv_heads);
        const int span_len = p.span_begin[span + 1] - p.span_begin[span];
        const int t0 = p.span_begin[span] + tile_first;
        const int rows = min(kFaM, span_len - tile_first);
        const int pos0 = p.positions[t0];
        const int pos_last = pos0 + rows - 1;
        const int first_key = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
        const int block_begin = first_key / kFaN;
        const int block_end = pos_last / kFaN + 1;

        if (warp == 0) {
            // ------------------------------------------------------------------ producer
            // Lane 0 waits for the stage; then lane 2 pg brings page pg of K and lane 2 pg + 1 that of V: one
            // thread issuing the up to 16 copies of a block one after the other took longer than the softmax
            // of a block. Every lane looks its page up one block ahead.
            const int* table = p.block_table + (size_t)span * p.table_stride;
            if (lane == 0) {
                mbar_expect_tx(smem_u32(&q_full), kFaQBytes);
                tma_load_2d(q_addr, &map_q, smem_u32(&q_full), h * kFaD, t0);
            }
            const int pages_per_block = kFaN / p.page_tokens;          // 1 to 8
            const unsigned page_bytes = (unsigned)p.page_tokens * kFaD * 2;
            const int pg = lane >> 1;
            const bool copies = pg < pages_per_block;
            const CUtensorMap* map = (lane & 1) ? &map_v : &map_k;
            auto lookup = [&](int kb) -> int {
                const int key0 = kb * kFaN + pg * p.page_tokens;
                // (keys nobody may see: any page of finite numbers will do)
                if (copies && kb < block_end && key0 <= pos_last && key0 + p.page_tokens > first_key)
                    return table[key0 / p.page_tokens];
                return 0;
            };
            int page_next = lookup(block_begin);
            for (int kb = block_begin; kb < block_end; ++kb) {
                const int i = kb - block_begin;
                const int s = i % kFaStages;
                int page = page_next;
                page_next = lookup(kb + 1);
                const unsigned bar = smem_u32(&kv_full[s]);
                int ok = 1;
                if (lane == 0) {
                    if (i >= kFaStages && !mbar_wait_suspended(smem_u32(&kv_empty[s]), ((i / kFaStages) - 1) & 1)) ok = 0;
                    if (ok) mbar_expect_tx(bar, 2 * kFaKvBytes);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) {
                    error = lane == 0 ? 61 : 0;
                    break;
                }
                if (copies) {
                    if (page < 0) {                       // the host never builds such a table
                        atomicExch(p.error_flag, 2);
                        page = 0;
                    }
                    const int row = (page * p.kv_heads + kvh) * p.page_tokens;
                    const unsigned dst = kv_addr + s * 2 * kFaKvBytes + ((lane & 1) ? kFaKvBytes : 0u) + pg * page_bytes;
                    tma_load_2d(dst, map, bar, 0, row);
                }
            }
        } else if (warp == 1 && lane == 0) {
            // ---------------------------------------------------------------- MMA issuer
            constexpr unsigned idesc_s = instruction_descriptor(kFaM, kFaN);
            constexpr unsigned idesc_o = instruction_descriptor_b_mn(kFaM, kFaD);
            const int blocks = block_end - block_begin;
            const unsigned long long desc_q = smem_descriptor(q_addr);
            // S of block i into its buffer, as soon as its keys are there
            auto scores = [&](int i) -> bool {
                const int s = i % kFaStages;
                if (!mbar_wait_suspended(smem_u32(&kv_full[s]), (i / kFaStages) & 1)) return false;
                tcgen05_fence_after();
                const unsigned long long desc_k = smem_descriptor(kv_addr + s * 2 * kFaKvBytes);
#pragma unroll
                for (int kk = 0; kk < kFaD / kUmmaK; ++kk)
                    umma_bf16(tmem_base + (unsigned)((i & 1) * kFaN), desc_q + 2 * kk, desc_k + 2 * kk, idesc_s, kk > 0 ? 1u : 0u);
                umma_commit(smem_u32(&s_full[i & 1]));
                return true;
            };
            if (!mbar_wait_suspended(smem_u32(&q_full), 0)) error = 62;
            if (!error && !scores(0)) error = 63;
            for (int i = 0; i < blocks && !error; ++i) {
                // the scores of the next block run while the softmax threads are busy with this one (they
                // have read the buffer's last content: P of block i-1 was complete before this point)
                if (i + 1 < blocks && !scores(i + 1)) {
                    error = 63;
                    break;
                }
                if (!mbar_wait_suspended(smem_u32(&p_full[i & 1]), (i >> 1) & 1)) {
                    error = 64;
                    break;
                }
                tcgen05_fence_after();
                const int s = i % kFaStages;
                const unsigned long long desc_v = smem_descriptor(kv_addr + s * 2 * kFaKvBytes + kFaKvBytes);
#pragma unroll
                for (int kk = 0; kk < kFaN / kUmmaK; ++kk) {
                    // P: 16 keys = 8 columns of tensor memory; V: 16 keys further = 16 rows of 128 bytes = 2 KiB
                    umma_bf16_a_tmem(tmem_base + kFaOColumn, tmem_base + kFaPColumn + (unsigned)((i & 1) * (kFaN / 2) + kk * 8),
                                     desc_v + (unsigned long long)(kk * 128), idesc_o, (i > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(smem_u32(&kv_empty[s]));
                umma_commit(smem_u32(&o_full[i & 1]));
            }
        } else if (warp >= 2) {
            // -------------------------------------------------------------------- softmax
            const int quarter = warp & 3;                           // the TMEM lanes this warp may touch
            const int row = quarter * 32 + lane;
            const unsigned lane_base = tmem_base + ((unsigned)(quarter * 32) << 16);
            const int qpos = pos0 + row;
            const bool live = row < rows;
            // The row's statistics. `used_max` is the maximum that P and the sum are relative to; it follows
            // the true running maximum only when that has grown by more than kFaSlack (in units of log2), so
            // that O, which accumulates in tensor memory, is rescaled rarely: exponentials stay below
            // 2^kFaSlack, which float32 sums and bfloat16 products hold without loss.
            constexpr float kFaSlack = 8.0f;
            float used_max = -INFINITY, run_sum = 0.0f;
            bool ok = true;
            const int blocks = block_end - block_begin;
            const unsigned o_taddr = lane_base + kFaOColumn;
            const unsigned long long scale2 = pack_f32x2(p.scale_log2, p.scale_log2);
            for (int i = 0; i < blocks; ++i) {
                // (S of block i complete also means: P V of block i-2 is complete, its P buffer is free)
                ok = ok && mbar_wait(smem_u32(&s_full[i & 1]), (i >> 1) & 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tcgen05_fence_after();
                const int key_base = (block_begin + i) * kFaN;
                const bool full = key_base + kFaN - 1 <= pos0 && rows == kFaM &&
                                  (p.window <= 0 || key_base > pos_last - p.window);
                // the whole row of scores in registers (one pass over tensor memory), not yet scaled
                float sc[kFaN];
                {
                    unsigned lo[32], hi[32];
                    tmem_load_32_issue(lane_base + (unsigned)((i & 1) * kFaN), lo);
                    tmem_load_32_issue(lane_base + (unsigned)((i & 1) * kFaN + 32), hi);
                    tmem_load_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        sc[j] = __uint_as_float(lo[j]);
                        sc[32 + j] = __uint_as_float(hi[j]);
                    }
                }
                if (!full) {
                    // keys key_base + [lo, hi] are the ones this row sees
                    const int hi = live ? min(kFaN - 1, qpos - key_base) : -1;
                    const int lo = p.window > 0 ? max(0, qpos - p.window + 1 - key_base) : 0;
#pragma unroll
                    for (int j = 0; j < kFaN; ++j) sc[j] = (j <= hi && j >= lo) ? sc[j] : -INFINITY;
                }
                // four independent chains of three-input maxima
                float part_max[4];
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) {
                    float m = max3_f32(sc[16 * c4], sc[16 * c4 + 1], sc[16 * c4 + 2]);
#pragma unroll
                    for (int j = 3; j < 15; j += 2) m = max3_f32(m, sc[16 * c4 + j], sc[16 * c4 + j + 1]);
                    part_max[c4] = fmaxf(m, sc[16 * c4 + 15]);
                }
                // (the scale is positive: the maximum commutes with it)
                const float block_max = fmaxf(max3_f32(part_max[0], part_max[1], part_max[2]), part_max[3]) * p.scale_log2;
                if (i == 0) {
                    used_max = block_max;
                } else {
                    const float new_max = fmaxf(used_max, block_max);
                    const bool grown = new_max > used_max + kFaSlack;          // (-inf + slack = -inf)
                    if (__any_sync(0xffffffffu, grown)) {
                        // O holds the sum up to block i-1 relative to used_max: wait for it, rescale the rows
                        // that grew (the warp's other rows by 1), put it back before P of this block is published
                        ok = mbar_wait(smem_u32(&o_full[(i - 1) & 1]), ((i - 1) >> 1) & 1);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                        tcgen05_fence_after();
                        const float factor = !grown ? 1.0f : (used_max == -INFINITY ? 0.0f : exp2f(used_max - new_max));
                        const unsigned long long factor2 = pack_f32x2(factor, factor);
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
                            unsigned part[32];
                            tmem_load_32_issue(o_taddr + (unsigned)(half * 32), part);
                            tmem_load_wait();
#pragma unroll
                            for (int j = 0; j < 32; j += 2) {
                                float a, b;
                                unpack_f32x2(mul_f32x2(pack_f32x2(__uint_as_float(part[j]), __uint_as_float(part[j + 1])), factor2), a, b);
                                part[j] = __float_as_uint(a);
                                part[j + 1] = __float_as_uint(b);
                            }
                            tmem_store_32(o_taddr + (unsigned)(half * 32), part);
                        }
                        tmem_store_wait();
                        run_sum *= factor;
                        if (grown) used_max = new_max;
                    }
                }
                const float safe_max = used_max == -INFINITY ? 0.0f : used_max;
                const unsigned long long neg_max2 = pack_f32x2(-safe_max, -safe_max);
                unsigned long long part_sum[4] = {0ull, 0ull, 0ull, 0ull};          // (0.0f, 0.0f) each
                unsigned p_packed[kFaN / 2];
#pragma unroll
                for (int j2 = 0; j2 < kFaN / 2; ++j2) {
                    float x0, x1, a, b;
                    unpack_f32x2(fma_f32x2(pack_f32x2(sc[2 * j2], sc[2 * j2 + 1]), scale2, neg_max2), x0, x1);
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(a) : "f"(x0));
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(b) : "f"(x1));
                    part_sum[j2 & 3] = add_f32x2(part_sum[j2 & 3], pack_f32x2(a, b));
                    const __nv_bfloat162 pair = __floats2bfloat162_rn(a, b);          // key 2 j2 in the lower half
                    p_packed[j2] = *reinterpret_cast<const unsigned*>(&pair);
                }
                tmem_store_32(lane_base + kFaPColumn + (unsigned)((i & 1) * (kFaN / 2)), p_packed);
                tmem_store_wait();
                {
                    float s0, s1;
                    unpack_f32x2(add_f32x2(add_f32x2(part_sum[0], part_sum[1]), add_f32x2(part_sum[2], part_sum[3])), s0, s1);
                    run_sum += s0 + s1;
                }
                tcgen05_fence_before();
                mbar_arrive_one(smem_u32(&p_full[i & 1]));
            }
            // the output: O of the last block complete, divided by the denominator
            float o[kFaD];
            if (ok && blocks > 0) {
                ok = mbar_wait(smem_u32(&o_full[(blocks - 1) & 1]), ((blocks - 1) >> 1) & 1);
                ok = __all_sync(0xffffffffu, ok);
                if (ok) {
                    tcgen05_fence_after();
                    unsigned lo[32], hi[32];
                    tmem_load_32_issue(o_taddr, lo);
                    tmem_load_32_issue(o_taddr + 32u, hi);
                    tmem_load_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        o[j] = __uint_as_float(lo[j]);
                        o[32 + j] = __uint_as_float(hi[j]);
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < kFaD; ++j) o[j] = 0.0f;
            }
            if (!ok) {
                if (lane == 0) atomicExch(p.error_flag, 65);
            } else if (live) {
                const float inv = run_sum > 0.0f ? 1.0f / run_sum : 0.0f;
                __nv_bfloat16* dst = p.out + ((size_t)(t0 + row) * p.q_heads + h) * kFaD;
#pragma unroll
                for (int c0 = 0; c0 < kFaD; c0 += 8) {
                    uint4 packed;
                    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                    for (int e2 = 0; e2 < 4; ++e2)
                        h2[e2] = __floats2bfloat162_rn(o[c0 + 2 * e2] * inv, o[c0 + 2 * e2 + 1] * inv);
                    *reinterpret_cast<uint4*>(dst + c0) = packed;
                }
            }
        }
        if (error) atomicExch(p.error_flag, error);
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, kFaTmemColumns);
}

}  // namespace celeg_b200

using namespace celeg_b200;

// Whether the shapes fit this kernel (the caller then uses celeg_attention_prefill or the general kernel).
CELEG_API int celeg_attention_prefill_tcgen05_supported(int q_heads, int kv_heads, int head_dim, int page_tokens) {
    return head_dim == kFaD && kv_heads > 0 && q_heads % kv_heads == 0 && page_tokens >= 8 && page_tokens % 8 == 0 &&
           kFaN % page_tokens == 0;
}

// q: [q_rows, q_row_stride] bfloat16 with head h at column h * 64 (q_rows: rows of the buffer that may be
// read, at least `tokens`); caches [pages, kv_heads, page_tokens, 64]. tile_count = sum over spans of
// ceil(length / 128), computed by the caller, who knows the lengths.
CELEG_API int celeg_attention_prefill_tcgen05(const void* q, int q_row_stride, int q_rows, void* out, const void* k_cache,
                                              const void* v_cache, int pages, const int* positions,
                                              const int* span_begin, const int* block_table, int table_stride,
                                              int tokens, int spans, int tile_count, int q_heads, int kv_heads,
                                              int head_dim, int page_tokens, int window, float scale, int* error_flag,
                                              cudaStream_t stream) {
    CELEG_REQUIRE(celeg_attention_prefill_tcgen05_supported(q_heads, kv_heads, head_dim, page_tokens),
                  "attention_prefill_tcgen05: head_dim=%d page_tokens=%d q_heads=%d kv_heads=%d are not taken here",
                  head_dim, page_tokens, q_heads, kv_heads);
    CELEG_REQUIRE(tokens >= 0 && spans >= 0 && tile_count >= 0 && pages > 0 && q_rows >= tokens && q_row_stride % 8 == 0 &&
                      ((size_t)q & 15) == 0 && error_flag,
                  "attention_prefill_tcgen05: invalid sizes tokens=%d spans=%d q_rows=%d q_row_stride=%d", tokens, spans,
                  q_rows, q_row_stride);
    if (tokens == 0 || tile_count == 0) return 0;
    CELEG_REQUIRE(tile_count <= 65535, "attention_prefill_tcgen05: %d query tiles exceed one launch (65535)", tile_count);
    CUtensorMap map_q, map_k, map_v;
    if (!tensor_map_for(q, q_rows, q_row_stride, q_row_stride, kFaM, &map_q)) return -2;
    const long long cache_rows = (long long)pages * kv_heads * page_tokens;
    if (!tensor_map_for(k_cache, cache_rows, kFaD, kFaD, page_tokens, &map_k)) return -2;
    if (!tensor_map_for(v_cache, cache_rows, kFaD, kFaD, page_tokens, &map_v)) return -2;
    FaParams p;
    p.out = (__nv_bfloat16*)out;
    p.positions = positions;
    p.span_begin = span_begin;
    p.block_table = block_table;
    p.table_stride = table_stride;
    p.spans = spans;
    p.q_heads = q_heads;
    p.kv_heads = kv_heads;
    p.page_tokens = page_tokens;
    p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.error_flag = error_flag;
    const cudaError_t status = cudaFuncSetAttribute(attention_prefill_tcgen05_kernel,
                                                    cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFaSmemBytes);
    if (status != cudaSuccess) {
        set_error("attention_prefill_tcgen05: %s", cudaGetErrorString(status));
        return -2;
    }
    attention_prefill_tcgen05_kernel<<<dim3(q_heads, tile_count), kFaThreads, kFaSmemBytes, stream>>>(map_q, map_k, map_v, p);
    return check_launch("attention_prefill_tcgen05");
}
