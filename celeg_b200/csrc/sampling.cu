// Sampling from float32 logits, one block per row, with celeg's rules
// (src/backend/cpu/sampler.cpp:26-101; CUDA twin packed_sample_topk_kernel,
// src/backend/cuda/kernels/sampling.cu:400-461):
//   * repetition penalty p > 1 on tokens the request has seen: l >= 0 ? l / p : l * p (also when greedy)
//   * temperature <= 0 or top_k == 1: arg-max, the first maximum wins
//   * else scores = l / temperature; the top_k best (score descending, then token ascending),
//     softmax over them in float32, top_p keeps the shortest prefix whose mass reaches p,
//     and one xorshift64* draw u = ((bits >> 11) + 0.5) / 2^53 walks that prefix.
// Each request has its own generator state and seen-table (indexed by its state slot), so its
// tokens do not depend on what else is in the batch. The sampled token is marked seen.
#include "common.cuh"

namespace celeg_b200 {

constexpr int kMaxTopK = 128;      // celeg's kMaxTopK (include/celeg/model/runtime_types.hpp:37)

struct Best {
    float score;
    int token;
};

__device__ __forceinline__ bool better(float sa, int ta, float sb, int tb) {
    return sa > sb || (sa == sb && ta < tb);
}

__device__ __forceinline__ Best warp_best(Best b) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float s = __shfl_xor_sync(0xffffffffu, b.score, offset);
        const int t = __shfl_xor_sync(0xffffffffu, b.token, offset);
        if (t >= 0 && (b.token < 0 || better(s, t, b.score, b.token))) {
            b.score = s;
            b.token = t;
        }
    }
    return b;
}

__device__ Best block_best(Best b, Best* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
    b = warp_best(b);
    __syncthreads();
    if (lane == 0) scratch[warp] = b;
    __syncthreads();
    if (warp == 0) {
        Best t = lane < warps ? scratch[lane] : Best{0.0f, -1};
        t = warp_best(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ float penalised(const float* logits, const uint8_t* seen, int token, float penalty) {
    float v = logits[token];
    if (seen && penalty > 1.0f && seen[token]) v = v >= 0.0f ? v / penalty : v * penalty;
    return v;
}

// Order-preserving key of a score: a larger float gives a larger unsigned key. NaN gives 0 and is never a
// candidate (no comparison with it holds in celeg's selection either).
__device__ __forceinline__ unsigned score_key(float v) {
    if (v != v) return 0u;
    if (v == 0.0f) return 0x80000000u;                 // -0 and +0 are one score
    const unsigned u = __float_as_uint(v);
    const unsigned key = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return key == 0u ? 1u : key;
}

// One block per row. The k best (score descending, then token ascending) are found by a radix selection over
// the scores' keys instead of k arg-max passes: four passes of 8 bits give the k-th largest key, a fifth pass
// gathers everything above it and the ties at it with the lowest token ids, and the k candidates are ranked
// among themselves. The vocabulary is read five or six times from the L2 instead of k times.
__global__ void sample_kernel(const float* logits, long long ld, int vocab,
                              const int* row_slot, uint8_t* seen_base,
                              unsigned long long* rng, const float* temperature,
                              const int* top_k, const float* top_p,
                              const float* penalty, int* out) {
    __shared__ Best scratch[33];
    __shared__ float cand_score[kMaxTopK];
    __shared__ int cand_token[kMaxTopK];
    __shared__ float sorted_score[kMaxTopK];
    __shared__ int sorted_token[kMaxTopK];
    __shared__ unsigned hist[256];
    __shared__ unsigned s_prefix, s_remaining, s_count, s_ties;
    chain_release();
    chain_wait();
    const int row = blockIdx.x;
    const float* l = logits + (size_t)row * ld;
    const int slot = row_slot ? row_slot[row] : row;
    uint8_t* seen = seen_base ? seen_base + (size_t)slot * vocab : nullptr;
    const float temp = temperature ? temperature[row] : 0.0f;
    const float pen = penalty ? penalty[row] : 1.0f;
    int k = top_k ? top_k[row] : 1;
    const bool greedy = temp <= 0.0f || k == 1;
    k = greedy ? 1 : min(min(k, kMaxTopK), vocab);
    auto score_of = [&](int token) {
        float v = penalised(l, seen, token, pen);
        if (!greedy) v = v / temp;
        return v;
    };

    // the k-th largest key, 8 bits at a time from the top
    if (threadIdx.x == 0) {
        s_prefix = 0u;
        s_remaining = (unsigned)k;
    }
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0u;
        __syncthreads();
        const unsigned prefix = s_prefix;
        for (int token = threadIdx.x; token < vocab; token += blockDim.x) {
            const unsigned key = score_key(score_of(token));
            if (key == 0u) continue;
            if (shift == 24 || (key >> (shift + 8)) == (prefix >> (shift + 8))) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned remaining = s_remaining, bin = 0u;
            if (shift == 24) {
                // fewer candidates than k (NaNs, or a tiny vocabulary): take all there are
                unsigned have = 0u;
                for (int i = 0; i < 256; ++i) have += hist[i];
                remaining = min(remaining, have);
            }
            if (remaining > 0u) {
                for (int i = 255; i >= 0; --i) {
                    if (hist[i] >= remaining) {
                        bin = (unsigned)i;
                        break;
                    }
                    remaining -= hist[i];
                }
            }
            s_prefix = prefix | (bin << shift);
            s_remaining = remaining;
            s_ties = hist[bin];
        }
        __syncthreads();
        if (shift == 24 && s_remaining == 0u) break;    // nothing but NaN in the row
    }
    const unsigned threshold = s_prefix;
    const unsigned need_ties = s_remaining;             // how many of the keys equal to the threshold belong to the k
    const unsigned ties = s_ties;
    __syncthreads();
    if (threadIdx.x == 0) s_count = 0u;
    __syncthreads();
    if (need_ties > 0u) {
        // everything above the threshold, and the ties when all of them are wanted
        for (int token = threadIdx.x; token < vocab; token += blockDim.x) {
            const float v = score_of(token);
            const unsigned key = score_key(v);
            if (key > threshold || (key == threshold && ties == need_ties)) {
                const unsigned at = atomicAdd(&s_count, 1u);
                if (at < (unsigned)kMaxTopK) {
                    cand_score[at] = v;
                    cand_token[at] = token;
                }
            }
        }
        __syncthreads();
        if (ties != need_ties) {
            // more equal scores at the threshold than places left: the lowest token ids among them, one by one
            int previous = -1;
            for (unsigned pick = 0; pick < need_ties; ++pick) {
                Best mine{0.0f, -1};
                for (int token = threadIdx.x; token < vocab; token += blockDim.x) {
                    if (token <= previous) continue;
                    const float v = score_of(token);
                    if (score_key(v) != threshold) continue;
                    if (mine.token < 0 || token < mine.token) {
                        mine.score = v;
                        mine.token = token;
                    }
                }
                // block_best orders by score first; the scores are equal here, so the lower token wins
                const Best best = block_best(mine, scratch);
                if (threadIdx.x == 0 && best.token >= 0) {
                    const unsigned at = s_count++;
                    if (at < (unsigned)kMaxTopK) {
                        cand_score[at] = best.score;
                        cand_token[at] = best.token;
                    }
                }
                previous = best.token;
                if (best.token < 0) break;
            }
            __syncthreads();
        }
    }
    k = min((int)s_count, kMaxTopK);
    // rank the candidates among themselves: score descending, then token ascending
    for (int i = threadIdx.x; i < k; i += blockDim.x) {
        const float sc = cand_score[i];
        const int tk = cand_token[i];
        int rank = 0;
        for (int j = 0; j < k; ++j) rank += better(cand_score[j], cand_token[j], sc, tk) ? 1 : 0;
        sorted_score[rank] = sc;
        sorted_token[rank] = tk;
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    int chosen;
    if (greedy || k <= 1) {
        chosen = k >= 1 ? sorted_token[0] : 0;
    } else {
        const float maximum = sorted_score[0];
        float total = 0.0f;
        for (int i = 0; i < k; ++i) {
            sorted_score[i] = expf(sorted_score[i] - maximum);
            total += sorted_score[i];
        }
        for (int i = 0; i < k; ++i) sorted_score[i] /= total;
        int active = k;
        const float p = top_p ? top_p[row] : 1.0f;
        if (p < 1.0f) {
            float cumulative = 0.0f;
            active = 0;
            do {
                cumulative += sorted_score[active++];
            } while (active < k && cumulative < p);
            total = 0.0f;
            for (int i = 0; i < active; ++i) total += sorted_score[i];
        } else {
            total = 1.0f;
        }
        unsigned long long state = rng[slot];
        state ^= state >> 12;
        state ^= state << 25;
        state ^= state >> 27;
        rng[slot] = state;
        const unsigned long long bits = state * 2685821657736338717ULL;
        const float unit = (float)(((double)(bits >> 11) + 0.5) * (1.0 / 9007199254740992.0));
        float target = unit * total;
        chosen = sorted_token[active - 1];
        for (int i = 0; i < active; ++i) {
            target -= sorted_score[i];
            if (target <= 0.0f) {
                chosen = sorted_token[i];
                break;
            }
        }
    }
    out[row] = chosen;
    if (seen) seen[chosen] = 1;
}

// Marks the tokens of a step as seen by their requests: slot = span_slot[token_span[i]].
// Greedy rows only (every row of the call has temperature <= 0 or top_k == 1): the vocabulary is
// cut into `chunks` pieces so that a few rows still use many SMs; a second, tiny kernel picks the
// best piece per row. The first maximum wins, as in the general kernel.
__global__ void argmax_partial_kernel(const float* logits, long long ld, int vocab, const int* row_slot,
                                      const uint8_t* seen_base, const float* penalty, int chunks,
                                      float* partial_score, int* partial_token) {
    __shared__ Best scratch[33];
    chain_release();
    chain_wait();
    const int row = blockIdx.y, chunk = blockIdx.x;
    const float* l = logits + (size_t)row * ld;
    const int slot = row_slot ? row_slot[row] : row;
    const float pen = penalty ? penalty[row] : 1.0f;
    const uint8_t* seen = (seen_base && pen > 1.0f) ? seen_base + (size_t)slot * vocab : nullptr;
    const int per = (vocab + chunks - 1) / chunks;
    const int begin = chunk * per, end = min(vocab, begin + per);
    Best mine{0.0f, -1};
    constexpr int kBatch = 8;
    for (int base = begin + threadIdx.x; base < end; base += blockDim.x * kBatch) {
        float v[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int token = base + u * blockDim.x;
            v[u] = token < end ? l[token] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int token = base + u * blockDim.x;
            if (token >= end) continue;
            float value = v[u];
            if (seen && seen[token]) value = value >= 0.0f ? value / pen : value * pen;
            if (mine.token < 0 || better(value, token, mine.score, mine.token)) {
                mine.score = value;
                mine.token = token;
            }
        }
    }
    const Best best = block_best(mine, scratch);
    if (threadIdx.x == 0) {
        partial_score[row * chunks + chunk] = best.score;
        partial_token[row * chunks + chunk] = best.token;
    }
}

__global__ void argmax_final_kernel(const float* partial_score, const int* partial_token, int chunks, int vocab,
                                    const int* row_slot, uint8_t* seen_base, int* out) {
    chain_release();
    chain_wait();
    const int row = blockIdx.x;
    Best mine{0.0f, -1};
    for (int i = threadIdx.x; i < chunks; i += 32) {
        const float s = partial_score[row * chunks + i];
        const int t = partial_token[row * chunks + i];
        if (t >= 0 && (mine.token < 0 || better(s, t, mine.score, mine.token))) {
            mine.score = s;
            mine.token = t;
        }
    }
    mine = warp_best(mine);
    if (threadIdx.x == 0) {
        const int chosen = mine.token < 0 ? 0 : mine.token;
        out[row] = chosen;
        if (seen_base) seen_base[(size_t)(row_slot ? row_slot[row] : row) * vocab + chosen] = 1;
    }
}

__global__ void mark_seen_kernel(uint8_t* seen_base, int vocab, const int* tokens,
                                 const int* token_span, const int* span_slot,
                                 int count) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const int token = tokens[i];
    if (token >= 0 && token < vocab) seen_base[(size_t)span_slot[token_span[i]] * vocab + token] = 1;
}

}  // namespace celeg_b200

using namespace celeg_b200;

CELEG_API int celeg_sample(const float* logits, long long ld, int vocab, int rows, const int* row_slot,
                           uint8_t* seen, unsigned long long* rng, const float* temperature, const int* top_k,
                           const float* top_p, const float* penalty, int* out, cudaStream_t stream) {
    CELEG_REQUIRE(rows >= 0 && vocab > 0 && ld >= vocab, "sample: invalid sizes rows=%d vocab=%d ld=%lld", rows,
                  vocab, ld);
    CELEG_REQUIRE(rng != nullptr || temperature == nullptr, "sample: temperature sampling needs generator states");
    if (rows == 0) return 0;
    const int threads = vocab >= 16384 ? 1024 : 256;
    launch_chained(sample_kernel, rows, threads, 0, stream, logits, ld, vocab, row_slot, seen, rng, temperature,
                   top_k, top_p, penalty, out);
    return check_launch("sample");
}

// All rows greedy. partial_score / partial_token: scratch of rows * 64 elements each.
CELEG_API int celeg_sample_greedy(const float* logits, long long ld, int vocab, int rows, const int* row_slot,
                                  uint8_t* seen, const float* penalty, int* out, float* partial_score,
                                  int* partial_token, cudaStream_t stream) {
    CELEG_REQUIRE(rows >= 0 && vocab > 0 && ld >= vocab, "sample_greedy: invalid sizes rows=%d vocab=%d ld=%lld", rows,
                  vocab, ld);
    CELEG_REQUIRE(rows <= 65535, "sample_greedy: %d rows exceed one launch", rows);
    if (rows == 0) return 0;
    int chunks = (vocab + 2047) / 2048;
    chunks = chunks < 1 ? 1 : chunks > 64 ? 64 : chunks;
    launch_chained(argmax_partial_kernel, dim3(chunks, rows), 256, 0, stream, logits, ld, vocab, row_slot,
                   (const uint8_t*)seen, penalty, chunks, partial_score, partial_token);
    int status = check_launch("sample_greedy (partial)");
    if (status != 0) return status;
    launch_chained(argmax_final_kernel, rows, 32, 0, stream, (const float*)partial_score, (const int*)partial_token,
                   chunks, vocab, row_slot, seen, out);
    return check_launch("sample_greedy (final)");
}

CELEG_API int celeg_mark_seen(uint8_t* seen, int vocab, const int* tokens, const int* token_span,
                              const int* span_slot, int count, cudaStream_t stream) {
    CELEG_REQUIRE(count >= 0 && vocab > 0, "mark_seen: invalid sizes count=%d vocab=%d", count, vocab);
    if (count == 0) return 0;
    mark_seen_kernel<<<(count + 255) / 256, 256, 0, stream>>>(seen, vocab, tokens, token_span, span_slot, count);
    return check_launch("mark_seen");
}
