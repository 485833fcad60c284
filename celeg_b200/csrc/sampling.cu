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

__global__ void sample_kernel(const float* logits, long long ld, int vocab,
                              const int* row_slot, uint8_t* seen_base,
                              unsigned long long* rng, const float* temperature,
                              const int* top_k, const float* top_p,
                              const float* penalty, int* out) {
    __shared__ Best scratch[33];
    __shared__ float cand_score[kMaxTopK];
    __shared__ int cand_token[kMaxTopK];
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

    float prev_score = INFINITY;
    int prev_token = -1;
    for (int pick = 0; pick < k; ++pick) {
        Best mine{0.0f, -1};
        for (int token = threadIdx.x; token < vocab; token += blockDim.x) {
            float v = penalised(l, seen, token, pen);
            if (!greedy) v = v / temp;
            // only candidates that come after the previous pick in (score desc, token asc) order
            if (pick > 0 && !better(prev_score, prev_token, v, token)) continue;
            if (mine.token < 0 || better(v, token, mine.score, mine.token)) {
                mine.score = v;
                mine.token = token;
            }
        }
        const Best best = block_best(mine, scratch);
        if (threadIdx.x == 0) {
            cand_score[pick] = best.score;
            cand_token[pick] = best.token;
        }
        prev_score = best.score;
        prev_token = best.token;
        if (best.token < 0) {            // fewer distinct candidates than k (NaNs): stop here
            k = pick;
            break;
        }
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    int chosen;
    if (greedy || k <= 1) {
        chosen = k >= 1 ? cand_token[0] : 0;
    } else {
        const float maximum = cand_score[0];
        float total = 0.0f;
        for (int i = 0; i < k; ++i) {
            cand_score[i] = expf(cand_score[i] - maximum);
            total += cand_score[i];
        }
        for (int i = 0; i < k; ++i) cand_score[i] /= total;
        int active = k;
        const float p = top_p ? top_p[row] : 1.0f;
        if (p < 1.0f) {
            float cumulative = 0.0f;
            active = 0;
            do {
                cumulative += cand_score[active++];
            } while (active < k && cumulative < p);
            total = 0.0f;
            for (int i = 0; i < active; ++i) total += cand_score[i];
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
        chosen = cand_token[active - 1];
        for (int i = 0; i < active; ++i) {
            target -= cand_score[i];
            if (target <= 0.0f) {
                chosen = cand_token[i];
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
