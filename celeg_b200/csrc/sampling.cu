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

// The same for tokens token .. token + 3 (token a multiple of 4, logits + token 16-byte aligned, seen + token 4-byte
// aligned), with the division by the temperature that the callers apply to a score: one operation after the
// other as for a single token, so that both ways give the same bits.
__device__ __forceinline__ float4 penalised_quad(const float* logits, const uint8_t* seen, int token, float penalty,
                                                 bool greedy, float temperature) {
    float4 v = *reinterpret_cast<const float4*>(logits + token);
    if (seen && penalty > 1.0f) {
        const uchar4 marks = *reinterpret_cast<const uchar4*>(seen + token);
        if (marks.x) v.x = v.x >= 0.0f ? v.x / penalty : v.x * penalty;
        if (marks.y) v.y = v.y >= 0.0f ? v.y / penalty : v.y * penalty;
        if (marks.z) v.z = v.z >= 0.0f ? v.z / penalty : v.z * penalty;
        if (marks.w) v.w = v.w >= 0.0f ? v.w / penalty : v.w * penalty;
    }
    if (!greedy) {
        v.x = v.x / temperature;
        v.y = v.y / temperature;
        v.z = v.z / temperature;
        v.w = v.w / temperature;
    }
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

constexpr int kSelectPool = 1024;   // most candidates the first stage may leave for the exact selection
constexpr int kSelectByRank = 256;  // up to this many pairs are ranked by counting instead of by a radix selection
constexpr int kSelectGroups = 128;  // the first stage bounds the k-th score by the k-th of this many group maxima (>= kMaxTopK)

struct SelectShared {
    Best scratch[33];
    float cand_score[kMaxTopK];
    int cand_token[kMaxTopK];
    float sorted_score[kMaxTopK];
    int sorted_token[kMaxTopK];
    unsigned hist[256];
    unsigned warp_hist[32][256];     // a histogram per warp: scores crowd into a few bins of the top digits, one
    unsigned prefix, remaining, count, ties;   // shared histogram would serialise on them
    float thread_max[1024];
    float pool_score[kSelectPool];
    int pool_token[kSelectPool];
    unsigned pool_count;
};

// The k best of n (score, token) pairs, score descending, then token ascending, into sm.sorted_*; returns how
// many there are (fewer than k if fewer pairs have a score that is a number). All threads of the block call
// it. A radix selection over the scores' keys: four passes of 8 bits give the k-th largest key, a fifth pass
// gathers everything above it and the ties at it with the lowest token ids, and the candidates are ranked
// among themselves.
template <typename ScoreAt, typename TokenAt>
__device__ int select_top_k(SelectShared& sm, const int n, const int k, ScoreAt score_at, TokenAt token_at) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    constexpr int kBatch = 8;
    __syncthreads();
    if (n <= kSelectByRank) {
        // Few pairs (the pool that the first stage of range_top_k leaves, its group maxima): every pair counts
        // the pairs that come before it in the order and, if fewer than k do, takes that place. The order is
        // total (tokens differ), so the places are a permutation. No histogram, two barriers.
        if (threadIdx.x == 0) sm.count = 0u;
        __syncthreads();
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const float sc = score_at(i);
            if (sc != sc) continue;                          // not a number: never a candidate
            const int tk = token_at(i);
            int rank = 0;
            for (int j = 0; j < n; ++j) {
                const float other = score_at(j);
                rank += (other == other && better(other, token_at(j), sc, tk)) ? 1 : 0;
            }
            atomicAdd(&sm.count, 1u);
            if (rank < k) {
                sm.sorted_score[rank] = sc;
                sm.sorted_token[rank] = tk;
            }
        }
        __syncthreads();
        return min((int)sm.count, k);
    }
    if (threadIdx.x == 0) {
        sm.prefix = 0u;
        sm.remaining = (unsigned)k;
        sm.ties = 0u;
    }
    __syncthreads();
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = lane; i < 256; i += 32) sm.warp_hist[warp][i] = 0u;
        __syncwarp();
        const unsigned prefix = sm.prefix;
        // every lane runs the same number of rounds, so that the warp-wide match below sees all lanes; eight
        // scores per lane and round are loaded before any is used
        for (int base = warp * 32; base < n; base += blockDim.x * kBatch) {
            float v[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int i = base + u * blockDim.x + lane;
                v[u] = i < n ? score_at(i) : __int_as_float(0x7fc00000);      // NaN: no contribution
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                if (base + u * (int)blockDim.x >= n) break;                 // (the same for all lanes)
                unsigned bin = 0xffffffffu;
                const unsigned key = score_key(v[u]);
                if (key != 0u && (shift == 24 || (key >> (shift + 8)) == (prefix >> (shift + 8))))
                    bin = (key >> shift) & 255u;
                // lanes with the same bin: the lowest of them adds their number, no two lanes write one counter
                const unsigned peers = __match_any_sync(0xffffffffu, bin);
                if (bin != 0xffffffffu && lane == __ffs(peers) - 1) sm.warp_hist[warp][bin] += __popc(peers);
                __syncwarp();
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < 256; i += blockDim.x) {
            unsigned total = 0u;
            for (int w = 0; w < warps; ++w) total += sm.warp_hist[w][i];
            sm.hist[i] = total;
        }
        __syncthreads();
        if (warp == 0) {
            // the bin in which the count from the top reaches what is still wanted: lane l holds bins 8l..8l+7
            unsigned local[8], sum = 0u;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                local[j] = sm.hist[lane * 8 + j];
                sum += local[j];
            }
            unsigned from_top = sum;                                   // this lane's bins and all higher ones
#pragma unroll
            for (int offset = 1; offset < 32; offset <<= 1) {
                const unsigned other = __shfl_down_sync(0xffffffffu, from_top, offset);
                if (lane + offset < 32) from_top += other;
            }
            const unsigned total = __shfl_sync(0xffffffffu, from_top, 0);
            unsigned remaining = sm.remaining;
            if (shift == 24) remaining = min(remaining, total);       // fewer candidates than k: take all there are
            const unsigned above = from_top - sum;
            __syncwarp();
            if (remaining == 0u) {
                if (lane == 0) {
                    sm.remaining = 0u;
                    sm.ties = 0u;
                }
            } else if (above < remaining && remaining <= above + sum) {
                unsigned left = remaining - above;
                int chosen_bin = 0;
#pragma unroll
                for (int j = 7; j >= 0; --j) {
                    if (left != 0u) {
                        if (local[j] >= left) {
                            chosen_bin = j;
                            sm.ties = local[j];
                            sm.remaining = left;
                            left = 0u;
                        } else {
                            left -= local[j];
                        }
                    }
                }
                sm.prefix = prefix | ((unsigned)(lane * 8 + chosen_bin) << shift);
            }
        }
        __syncthreads();
        if (shift == 24 && sm.remaining == 0u) break;    // not one score that is a number
    }
    const unsigned threshold = sm.prefix;
    const unsigned need_ties = sm.remaining;             // how many of the keys equal to the threshold belong to the k
    const unsigned ties = sm.ties;
    __syncthreads();
    if (threadIdx.x == 0) sm.count = 0u;
    __syncthreads();
    if (need_ties > 0u) {
        // everything above the threshold, and the ties when all of them are wanted
        for (int base = threadIdx.x; base < n; base += blockDim.x * kBatch) {
            float v[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int i = base + u * blockDim.x;
                v[u] = i < n ? score_at(i) : __int_as_float(0x7fc00000);
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const unsigned key = score_key(v[u]);
                if (key != 0u && (key > threshold || (key == threshold && ties == need_ties))) {
                    const unsigned at = atomicAdd(&sm.count, 1u);
                    if (at < (unsigned)kMaxTopK) {
                        sm.cand_score[at] = v[u];
                        sm.cand_token[at] = token_at(base + u * blockDim.x);
                    }
                }
            }
        }
        __syncthreads();
        if (ties != need_ties) {
            // more equal scores at the threshold than places left: the lowest token ids among them, one by one
            int previous = -1;
            for (unsigned pick = 0; pick < need_ties; ++pick) {
                Best mine{0.0f, -1};
                for (int i = threadIdx.x; i < n; i += blockDim.x) {
                    const int token = token_at(i);
                    if (token <= previous) continue;
                    const float v = score_at(i);
                    if (score_key(v) != threshold) continue;
                    if (mine.token < 0 || token < mine.token) {
                        mine.score = v;
                        mine.token = token;
                    }
                }
                // block_best orders by score first; the scores are equal here, so the lower token wins
                const Best best = block_best(mine, sm.scratch);
                if (threadIdx.x == 0 && best.token >= 0) {
                    const unsigned at = sm.count++;
                    if (at < (unsigned)kMaxTopK) {
                        sm.cand_score[at] = best.score;
                        sm.cand_token[at] = best.token;
                    }
                }
                previous = best.token;
                if (best.token < 0) break;
            }
            __syncthreads();
        }
    }
    const int found = min((int)sm.count, kMaxTopK);
    // rank the candidates among themselves: score descending, then token ascending
    for (int i = threadIdx.x; i < found; i += blockDim.x) {
        const float sc = sm.cand_score[i];
        const int tk = sm.cand_token[i];
        int rank = 0;
        for (int j = 0; j < found; ++j) rank += better(sm.cand_score[j], sm.cand_token[j], sc, tk) ? 1 : 0;
        sm.sorted_score[rank] = sc;
        sm.sorted_token[rank] = tk;
    }
    __syncthreads();
    return found;
}

// The k best scores of tokens [begin, end) of a row, into sm.sorted_*, in two stages. First every thread keeps
// the largest score of its share and groups of threads the largest of theirs; the k-th largest of these 128
// maxima is a lower bound of the k-th largest score (k different tokens reach it), so one more pass that keeps
// every token at or above it leaves a pool of about twice k candidates for the exact selection. A pool that overflows (scores that are equal by the thousand)
// sends the range to the exact selection over all of it instead. The range is read twice where the plain form
// reads it k times. Returns how many were found.
template <typename ScoreOf, typename QuadOf>
__device__ int range_top_k(SelectShared& sm, const int begin, const int end, const int k, ScoreOf score_of,
                           QuadOf quad_of, const bool quads) {
    constexpr int kBatch = 8;
    constexpr int kQuads = 4;                            // 16-byte loads in flight per thread and round
    // with `quads`, the scores of tokens begin + 4 q .. + 3 come from quad_of(begin + 4 q) (16-byte loads of
    // the logits, 4-byte loads of the seen marks; the same arithmetic per score); the rest one by one
    const int n4 = quads ? (end - begin) / 4 : 0;
    const int scalar_begin = begin + 4 * n4;
    float mine = -INFINITY;
    bool any = false;
    for (int q0 = threadIdx.x; q0 < n4; q0 += blockDim.x * kQuads) {
        float4 v[kQuads];
#pragma unroll
        for (int u = 0; u < kQuads; ++u) {
            const int q = q0 + u * blockDim.x;
            const float nan = __int_as_float(0x7fc00000);
            v[u] = q < n4 ? quad_of(begin + 4 * q) : make_float4(nan, nan, nan, nan);
        }
#pragma unroll
        for (int u = 0; u < kQuads; ++u) {
            const float part[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (part[c] == part[c]) {
                    mine = any ? fmaxf(mine, part[c]) : part[c];
                    any = true;
                }
            }
        }
    }
    for (int base = scalar_begin + threadIdx.x; base < end; base += blockDim.x * kBatch) {
        float v[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int token = base + u * blockDim.x;
            v[u] = token < end ? score_of(token) : __int_as_float(0x7fc00000);
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            if (v[u] == v[u]) {
                mine = any ? fmaxf(mine, v[u]) : v[u];
                any = true;
            }
        }
    }
    // the maxima of groups of neighbouring threads, kSelectGroups of them (a maximum ignores what is not a number)
    float group_max = any ? mine : __int_as_float(0x7fc00000);
    const int group = max(1, (int)blockDim.x / kSelectGroups);          // 8, 4 or 2 threads: a power of two within a warp
    for (int offset = group >> 1; offset > 0; offset >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, group_max, offset);
        group_max = group_max != group_max ? other : (other != other ? group_max : fmaxf(group_max, other));
    }
    __syncthreads();                                   // (sm.thread_max may still be read by an earlier selection)
    if (threadIdx.x % group == 0) sm.thread_max[threadIdx.x / group] = group_max;
    const int groups = (int)blockDim.x / group;
    int found = select_top_k(sm, groups, k, [&](int i) { return sm.thread_max[i]; }, [](int i) { return i; });
    if (found == 0) return 0;                          // not one score that is a number
    // k groups hold a score each at or above the k-th largest maximum: a lower bound of the k-th largest score.
    // Fewer groups with a score than k (a short range, scores that are no numbers): no bound, every score is pooled.
    const float bound = found >= k ? sm.sorted_score[k - 1] : -INFINITY;
    __syncthreads();
    if (threadIdx.x == 0) sm.pool_count = 0u;
    __syncthreads();
    for (int q0 = threadIdx.x; q0 < n4; q0 += blockDim.x * kQuads) {
        float4 v[kQuads];
#pragma unroll
        for (int u = 0; u < kQuads; ++u) {
            const int q = q0 + u * blockDim.x;
            const float nan = __int_as_float(0x7fc00000);
            v[u] = q < n4 ? quad_of(begin + 4 * q) : make_float4(nan, nan, nan, nan);
        }
#pragma unroll
        for (int u = 0; u < kQuads; ++u) {
            const float part[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (part[c] >= bound) {
                    const unsigned at = atomicAdd(&sm.pool_count, 1u);
                    if (at < (unsigned)kSelectPool) {
                        sm.pool_score[at] = part[c];
                        sm.pool_token[at] = begin + 4 * (q0 + u * (int)blockDim.x) + c;
                    }
                }
            }
        }
    }
    for (int base = scalar_begin + threadIdx.x; base < end; base += blockDim.x * kBatch) {
        float v[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int token = base + u * blockDim.x;
            v[u] = token < end ? score_of(token) : __int_as_float(0x7fc00000);
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            if (v[u] >= bound) {
                const unsigned at = atomicAdd(&sm.pool_count, 1u);
                if (at < (unsigned)kSelectPool) {
                    sm.pool_score[at] = v[u];
                    sm.pool_token[at] = base + u * blockDim.x;
                }
            }
        }
    }
    __syncthreads();
    const unsigned pooled = sm.pool_count;
    if (pooled <= (unsigned)kSelectPool)
        return select_top_k(sm, (int)pooled, k, [&](int i) { return sm.pool_score[i]; },
                            [&](int i) { return sm.pool_token[i]; });
    return select_top_k(sm, end - begin, k, [&](int i) { return score_of(begin + i); }, [&](int i) { return begin + i; });
}

// What one thread does with the k candidates in sm.sorted_*: arg-max, or softmax, top-p and the draw.
__device__ int draw_from_sorted(SelectShared& sm, const int k, const bool greedy, const float p,
                                unsigned long long* rng_state) {
    float* sorted_score = sm.sorted_score;
    const int* sorted_token = sm.sorted_token;
    if (greedy || k <= 1) return k >= 1 ? sorted_token[0] : 0;
    const float maximum = sorted_score[0];
    float total = 0.0f;
    for (int i = 0; i < k; ++i) {
        sorted_score[i] = expf(sorted_score[i] - maximum);
        total += sorted_score[i];
    }
    for (int i = 0; i < k; ++i) sorted_score[i] /= total;
    int active = k;
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
    unsigned long long state = *rng_state;
    state ^= state >> 12;
    state ^= state << 25;
    state ^= state >> 27;
    *rng_state = state;
    const unsigned long long bits = state * 2685821657736338717ULL;
    const float unit = (float)(((double)(bits >> 11) + 0.5) * (1.0 / 9007199254740992.0));
    float target = unit * total;
    int chosen = sorted_token[active - 1];
    for (int i = 0; i < active; ++i) {
        target -= sorted_score[i];
        if (target <= 0.0f) {
            chosen = sorted_token[i];
            break;
        }
    }
    return chosen;
}

struct SampleRow {
    const float* logits;
    uint8_t* seen;
    int slot;
    float temperature, penalty;
    int k;
    bool greedy;
};

__device__ __forceinline__ SampleRow sample_row(const float* logits, long long ld, int vocab, const int* row_slot,
                                                uint8_t* seen_base, const float* temperature, const int* top_k,
                                                const float* penalty, int row) {
    SampleRow r;
    r.logits = logits + (size_t)row * ld;
    r.slot = row_slot ? row_slot[row] : row;
    r.seen = seen_base ? seen_base + (size_t)r.slot * vocab : nullptr;
    r.temperature = temperature ? temperature[row] : 0.0f;
    r.penalty = penalty ? penalty[row] : 1.0f;
    const int k = top_k ? top_k[row] : 1;
    r.greedy = r.temperature <= 0.0f || k == 1;
    r.k = r.greedy ? 1 : min(min(k, kMaxTopK), vocab);
    return r;
}

// One block per row: selection over the whole vocabulary and the draw (many rows).
__global__ void sample_kernel(const float* logits, long long ld, int vocab,
                              const int* row_slot, uint8_t* seen_base,
                              unsigned long long* rng, const float* temperature,
                              const int* top_k, const float* top_p,
                              const float* penalty, int* out) {
    __shared__ SelectShared sm;
    chain_release();
    chain_wait();
    const int row = blockIdx.x;
    const SampleRow r = sample_row(logits, ld, vocab, row_slot, seen_base, temperature, top_k, penalty, row);
    auto score_of = [&](int token) {
        float v = penalised(r.logits, r.seen, token, r.penalty);
        if (!r.greedy) v = v / r.temperature;
        return v;
    };
    auto quad_of = [&](int token) { return penalised_quad(r.logits, r.seen, token, r.penalty, r.greedy, r.temperature); };
    const bool quads = (((size_t)r.logits) & 15) == 0 && (r.seen == nullptr || (((size_t)r.seen) & 3) == 0);
    const int found = range_top_k(sm, 0, vocab, r.k, score_of, quad_of, quads);
    if (threadIdx.x != 0) return;
    const int chosen = draw_from_sorted(sm, found, r.greedy, top_p ? top_p[row] : 1.0f, rng ? rng + r.slot : nullptr);
    out[row] = chosen;
    if (r.seen) r.seen[chosen] = 1;
}

// Few rows: a row's vocabulary is cut into `chunks` pieces, one block each, so that a handful of rows still
// uses many SMs; every piece leaves its own k best (part_score / part_token [rows, chunks, kMaxTopK], entries
// past part_count are unused), and sample_merge_kernel selects among those and draws.
__global__ void sample_chunks_kernel(const float* logits, long long ld, int vocab, const int* row_slot,
                                     uint8_t* seen_base, const float* temperature, const int* top_k,
                                     const float* penalty, int chunks, float* part_score, int* part_token,
                                     int* part_count) {
    __shared__ SelectShared sm;
    chain_release();
    chain_wait();
    const int row = blockIdx.y, chunk = blockIdx.x;
    const SampleRow r = sample_row(logits, ld, vocab, row_slot, seen_base, temperature, top_k, penalty, row);
    auto score_of = [&](int token) {
        float v = penalised(r.logits, r.seen, token, r.penalty);
        if (!r.greedy) v = v / r.temperature;
        return v;
    };
    auto quad_of = [&](int token) { return penalised_quad(r.logits, r.seen, token, r.penalty, r.greedy, r.temperature); };
    const bool quads = (((size_t)r.logits) & 15) == 0 && (r.seen == nullptr || (((size_t)r.seen) & 3) == 0);
    const int per = (vocab + chunks - 1) / chunks;
    const int begin = min(vocab, chunk * per), end = min(vocab, begin + per);
    const int found = end > begin ? range_top_k(sm, begin, end, min(r.k, end - begin), score_of, quad_of,
                                                quads && (begin & 3) == 0) : 0;
    const size_t base = ((size_t)row * chunks + chunk) * kMaxTopK;
    for (int i = threadIdx.x; i < found; i += blockDim.x) {
        part_score[base + i] = sm.sorted_score[i];
        part_token[base + i] = sm.sorted_token[i];
    }
    if (threadIdx.x == 0) part_count[row * chunks + chunk] = found;
}

__global__ void sample_merge_kernel(int vocab, const int* row_slot, uint8_t* seen_base, unsigned long long* rng,
                                    const float* temperature, const int* top_k, const float* top_p, int chunks,
                                    const float* part_score, const int* part_token, const int* part_count,
                                    int* out) {
    __shared__ SelectShared sm;
    chain_release();
    chain_wait();
    const int row = blockIdx.x;
    const SampleRow r = sample_row(nullptr, 0, vocab, row_slot, seen_base, temperature, top_k, nullptr, row);
    const size_t base = (size_t)row * chunks * kMaxTopK;
    const int* counts = part_count + row * chunks;
    auto score_at = [&](int i) {
        return (i % kMaxTopK) < counts[i / kMaxTopK] ? part_score[base + i] : __int_as_float(0x7fc00000);
    };
    auto token_at = [&](int i) { return part_token[base + i]; };
    const int found = select_top_k(sm, chunks * kMaxTopK, r.k, score_at, token_at);
    if (threadIdx.x != 0) return;
    const int chosen = draw_from_sorted(sm, found, r.greedy, top_p ? top_p[row] : 1.0f, rng ? rng + r.slot : nullptr);
    out[row] = chosen;
    if (r.seen) r.seen[chosen] = 1;
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
    // whole groups of four tokens with one 16-byte load of the logits and one 4-byte load of the seen marks
    // (the same comparison per token, tokens in rising order within a thread as below), the rest one by one
    const bool quads = ((((size_t)l) & 15) == 0) && (begin & 3) == 0 && (seen == nullptr || (((size_t)seen) & 3) == 0);
    const int n4 = quads ? (end - begin) / 4 : 0;
    for (int q = threadIdx.x; q < n4; q += blockDim.x) {
        const int token0 = begin + 4 * q;
        const float4 four = *reinterpret_cast<const float4*>(l + token0);
        uchar4 marks = make_uchar4(0, 0, 0, 0);
        if (seen) marks = *reinterpret_cast<const uchar4*>(seen + token0);
        const float part[4] = {four.x, four.y, four.z, four.w};
        const unsigned char mark[4] = {marks.x, marks.y, marks.z, marks.w};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float value = part[c];
            if (mark[c]) value = value >= 0.0f ? value / pen : value * pen;
            if (mine.token < 0 || better(value, token0 + c, mine.score, mine.token)) {
                mine.score = value;
                mine.token = token0 + c;
            }
        }
    }
    for (int base = begin + 4 * n4 + threadIdx.x; base < end; base += blockDim.x * kBatch) {
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

constexpr int kSampleChunks = 16;        // pieces a row is cut into when there are few rows
constexpr int kSampleChunkedRows = 32;   // ... which is when there are at most this many

// Elements of part_score / part_token (and, divided by 128, of part_count) that celeg_sample wants as scratch to
// cut the rows of a small batch into pieces: kSampleChunkedRows * kSampleChunks * 128.
CELEG_API int celeg_sample_scratch_elements() { return kSampleChunkedRows * kSampleChunks * kMaxTopK; }

// part_score / part_token / part_count may be null: then every row is one block whatever the number of rows.
CELEG_API int celeg_sample(const float* logits, long long ld, int vocab, int rows, const int* row_slot,
                           uint8_t* seen, unsigned long long* rng, const float* temperature, const int* top_k,
                           const float* top_p, const float* penalty, int* out, float* part_score, int* part_token,
                           int* part_count, cudaStream_t stream) {
    CELEG_REQUIRE(rows >= 0 && vocab > 0 && ld >= vocab, "sample: invalid sizes rows=%d vocab=%d ld=%lld", rows,
                  vocab, ld);
    CELEG_REQUIRE(rng != nullptr || temperature == nullptr, "sample: temperature sampling needs generator states");
    if (rows == 0) return 0;
    // (more rows than SMs: blocks of 512 threads, of which two run on an SM at a time (registers), so that 256 rows
    // are one wave of blocks instead of two)
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (sms <= 0) sms = 148;
    }
    const int threads = vocab >= 16384 ? (rows > sms ? 512 : 1024) : 256;
    if (part_score && part_token && part_count && rows <= kSampleChunkedRows && vocab >= kSampleChunks * 1024) {
        launch_chained(sample_chunks_kernel, dim3(kSampleChunks, rows), 256, 0, stream, logits, ld, vocab, row_slot,
                       seen, temperature, top_k, penalty, kSampleChunks, part_score, part_token, part_count);
        const int status = check_launch("sample (pieces)");
        if (status != 0) return status;
        launch_chained(sample_merge_kernel, rows, 256, 0, stream, vocab, row_slot, seen, rng, temperature, top_k,
                       top_p, kSampleChunks, (const float*)part_score, (const int*)part_token,
                       (const int*)part_count, out);
        return check_launch("sample (merge)");
    }
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
