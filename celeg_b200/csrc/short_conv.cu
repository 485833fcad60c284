// The short-convolution mixer's inner step for a batch of spans (a span = the tokens one
// request brings to this step; a single decoded token is a span of length 1):
//
//   [B | C | X] = proj[t, 0:H | H:2H | 2H:3H]     bx_t = B_t * X_t
//   conv_t[c]   = sum_{tap<L} kernel[c, tap] * bx_{t-(L-1)+tap}[c]      (tap L-1 = current token)
//   out_t       = C_t * conv_t
//
// bx of positions before the span comes from the request's state slot, which keeps the last
// L-1 values of bx per channel, oldest first, in float32. Positions before the sequence are
// zero (a slot is zeroed when a request takes it).
//
// Work split, two launches. Tokens whose taps all lie inside the span (index in span >= L-1) are
// independent: one block row per token (eight channels per thread for bfloat16). Everything that
// touches the slot - the first L-1 tokens of a span and the slot's new content - is done by ONE
// thread per (span, channel), which reads the old state into registers before it writes, so the
// update is in place without a second buffer.
// Both paths add the taps in the same order, so a token's result does not depend on where the
// span was cut.
//
// Counterparts in celeg: conv_decode_batch_ptrs_kernel and conv_ragged_prefill_kernel
// (src/backend/cuda/kernels/shortconv.cuh:1-33, 34-), where one thread walks a whole span
// serially and the state is a bf16 ring indexed by position % L.
#include "common.cuh"

namespace celeg_b200 {

constexpr int kMaxTaps = 16;

// Tokens whose taps all lie inside their span (index in span >= taps-1): one block row per token,
// one channel per thread.
template <typename A>
__global__ void short_conv_tokens_kernel(const A* proj, const float* __restrict__ kernel, A* out,
                                         const int* token_span, const int* span_begin, int hidden, int taps) {
    chain_release();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= hidden) return;
    float w[kMaxTaps];
#pragma unroll
    for (int i = 0; i < kMaxTaps; ++i) w[i] = i < taps ? kernel[(size_t)c * taps + i] : 0.0f;   // constant data
    chain_wait();
    const int t = blockIdx.y;
    const size_t row = (size_t)3 * hidden;
    const int first = span_begin[token_span[t]];
    if (t - first < taps - 1) return;               // handled with the state by the span kernel
    float conv = 0.0f;
    for (int tap = 0; tap < taps; ++tap) {
        const A* p = proj + (size_t)(t - (taps - 1) + tap) * row;
        conv += w[tap] * (to_float(p[c]) * to_float(p[2 * hidden + c]));
    }
    out[(size_t)t * hidden + c] = from_float<A>(to_float(proj[(size_t)t * row + hidden + c]) * conv);
}

// The same for bfloat16 and a width that is a multiple of 8: eight channels per thread, 16-byte loads.
__global__ void short_conv_tokens_bf16x8_kernel(const __nv_bfloat16* proj, const float* __restrict__ kernel,
                                                __nv_bfloat16* out, const int* token_span, const int* span_begin,
                                                int hidden, int taps) {
    chain_release();
    chain_wait();
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= hidden) return;
    const int t = blockIdx.y;
    const size_t row = (size_t)3 * hidden;
    const int first = span_begin[token_span[t]];
    if (t - first < taps - 1) return;
    float conv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) conv[i] = 0.0f;
    for (int tap = 0; tap < taps; ++tap) {
        const __nv_bfloat16* p = proj + (size_t)(t - (taps - 1) + tap) * row + c;
        const uint4 b4 = *reinterpret_cast<const uint4*>(p);
        const uint4 x4 = *reinterpret_cast<const uint4*>(p + 2 * hidden);
        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b4);
        const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&x4);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 b = __bfloat1622float2(b2[i]);
            const float2 x = __bfloat1622float2(x2[i]);
            conv[2 * i] += kernel[(size_t)(c + 2 * i) * taps + tap] * (b.x * x.x);
            conv[2 * i + 1] += kernel[(size_t)(c + 2 * i + 1) * taps + tap] * (b.y * x.y);
        }
    }
    const uint4 c4 = *reinterpret_cast<const uint4*>(proj + (size_t)t * row + hidden + c);
    const __nv_bfloat162* c2 = reinterpret_cast<const __nv_bfloat162*>(&c4);
    uint4 r;
    __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 cc = __bfloat1622float2(c2[i]);
        r2[i] = __floats2bfloat162_rn(cc.x * conv[2 * i], cc.y * conv[2 * i + 1]);
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * hidden + c) = r;
}

// The same again for kernels of at most four taps (LFM2 has three): a thread keeps the weights of its
// eight channels in registers and walks over kTokensPerThread consecutive tokens with a sliding
// window of B*X, so a row of the projection is read 1.4 times instead of `taps` times and all loads of a
// thread are in flight together. Taps are added in the same order as in the kernels above.
constexpr int kTokensPerThread = 8;
constexpr int kFewTaps = 4;

__device__ __forceinline__ void short_conv_window_body(const __nv_bfloat16* proj, const float* __restrict__ kernel,
                                                       __nv_bfloat16* out, const int* token_span, const int* span_begin,
                                                       int hidden, int taps, int tokens, const int c, const int group) {
    if (c >= hidden) return;
    float w[kFewTaps][8];                        // w[e]: the tap that meets the token e places back (tap taps-1-e)
#pragma unroll
    for (int e = 0; e < kFewTaps; ++e)
#pragma unroll
        for (int i = 0; i < 8; ++i) w[e][i] = e < taps ? kernel[(size_t)(c + i) * taps + (taps - 1 - e)] : 0.0f;
    chain_wait();
    const int t0 = group * kTokensPerThread;
    const size_t row = (size_t)3 * hidden;
    const int keep = taps - 1;
    constexpr int kRows = kTokensPerThread + kFewTaps - 1;
    // rows t0 - keep .. t0 + kTokensPerThread - 1 of B and X (rows before the batch or past it: not loaded)
    uint4 b4[kRows], x4[kRows], c4[kTokensPerThread];
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        const int t = t0 - (kFewTaps - 1) + r;
        const bool wanted = t >= t0 - keep && t >= 0 && t < tokens;
        b4[r] = wanted ? *reinterpret_cast<const uint4*>(proj + (size_t)t * row + c) : zero;
        x4[r] = wanted ? *reinterpret_cast<const uint4*>(proj + (size_t)t * row + 2 * hidden + c) : zero;
    }
    int first[kTokensPerThread];
#pragma unroll
    for (int j = 0; j < kTokensPerThread; ++j) {
        const int t = t0 + j;
        c4[j] = t < tokens ? *reinterpret_cast<const uint4*>(proj + (size_t)t * row + hidden + c) : zero;
        first[j] = t < tokens ? span_begin[token_span[t]] : t + 1;
    }
    float bx[kRows][8];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b4[r]);
        const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&x4[r]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 b = __bfloat1622float2(b2[i]);
            const float2 x = __bfloat1622float2(x2[i]);
            bx[r][2 * i] = b.x * x.x;
            bx[r][2 * i + 1] = b.y * x.y;
        }
    }
#pragma unroll
    for (int j = 0; j < kTokensPerThread; ++j) {
        const int t = t0 + j;
        if (t >= tokens || t - first[j] < keep) continue;      // the span kernel's tokens
        float conv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) conv[i] = 0.0f;
        // oldest tap first, as everywhere: the token e places back is row j + (kFewTaps - 1) - e
#pragma unroll
        for (int e = kFewTaps - 1; e >= 0; --e) {
            if (e < taps) {
#pragma unroll
                for (int i = 0; i < 8; ++i) conv[i] += w[e][i] * bx[j + (kFewTaps - 1) - e][i];
            }
        }
        const __nv_bfloat162* c2 = reinterpret_cast<const __nv_bfloat162*>(&c4[j]);
        uint4 result;
        __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&result);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 cc = __bfloat1622float2(c2[i]);
            r2[i] = __floats2bfloat162_rn(cc.x * conv[2 * i], cc.y * conv[2 * i + 1]);
        }
        *reinterpret_cast<uint4*>(out + (size_t)t * hidden + c) = result;
    }
}

// Everything that touches a request's state: the first taps-1 tokens of its span and the slot's new
// content, one thread per (span, channel), which reads the old state into registers before it writes.
template <typename A>
__device__ __forceinline__ void short_conv_spans_body(const A* proj, const float* __restrict__ kernel, float* state,
                                                      long long slot_stride, A* out, const int* span_begin,
                                                      const int* span_slot, int hidden, int taps, const int c,
                                                      const int s) {
    if (c >= hidden) return;
    const size_t row = (size_t)3 * hidden;
    float w[kMaxTaps];
#pragma unroll
    for (int i = 0; i < kMaxTaps; ++i) w[i] = i < taps ? kernel[(size_t)c * taps + i] : 0.0f;   // constant data
    chain_wait();
    const int first = span_begin[s];
    const int count = span_begin[s + 1] - first;
    const int keep = taps - 1;
    float* st = state + (size_t)span_slot[s] * slot_stride;     // [keep][hidden]
    if (count == 1 && keep >= 1) {
        // a decoded token: its three values and the carried taps are asked for together (in the general
        // form below C is loaded only after the convolution is summed), same arithmetic in the same order
        const A* p = proj + (size_t)first * row;
        const A b_raw = p[c], c_raw = p[hidden + c], x_raw = p[2 * hidden + c];
        float old_taps[kMaxTaps];
#pragma unroll
        for (int i = 0; i < kMaxTaps; ++i) old_taps[i] = i < keep ? st[(size_t)i * hidden + c] : 0.0f;
        const float bx = to_float(b_raw) * to_float(x_raw);
        float conv = 0.0f;
#pragma unroll
        for (int tap = 0; tap < kMaxTaps; ++tap) {
            if (tap < keep) conv += w[tap] * old_taps[tap];
            else if (tap == keep) conv += w[tap] * bx;
        }
        out[(size_t)first * hidden + c] = from_float<A>(to_float(c_raw) * conv);
#pragma unroll
        for (int i = 0; i < kMaxTaps; ++i) {
            if (i + 1 < keep) st[(size_t)i * hidden + c] = old_taps[i + 1];
            else if (i + 1 == keep) st[(size_t)i * hidden + c] = bx;
        }
        return;
    }
    // history[i], i < keep: bx of the keep positions before the span; history[keep + j]: bx of span token j
    float history[2 * kMaxTaps];
#pragma unroll
    for (int i = 0; i < kMaxTaps; ++i) history[i] = i < keep ? st[(size_t)i * hidden + c] : 0.0f;
    const int head = count < keep ? count : keep;
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j) {
        if (j < head) {
            const A* p = proj + (size_t)(first + j) * row;
            history[keep + j] = to_float(p[c]) * to_float(p[2 * hidden + c]);
        }
    }
    for (int j = 0; j < head; ++j) {
        float conv = 0.0f;
        for (int tap = 0; tap < taps; ++tap) conv += w[tap] * history[j + tap];
        const int t = first + j;
        out[(size_t)t * hidden + c] = from_float<A>(to_float(proj[(size_t)t * row + hidden + c]) * conv);
    }
    // new state: the last `keep` values of (old state ++ bx of the span)
    for (int i = 0; i < keep; ++i) {
        const int source = count + i;               // index into the sequence old(keep) ++ span(count)
        float v;
        if (source < keep + head) {
            v = history[source];
        } else {
            const A* p = proj + (size_t)(first + source - keep) * row;
            v = to_float(p[c]) * to_float(p[2 * hidden + c]);
        }
        st[(size_t)i * hidden + c] = v;
    }
}

// A step in which every request brings one token (many requests decoding), bfloat16, at most kFewTaps taps: a
// thread serves eight neighbouring channels of one request with 16-byte loads (the span kernel's decoded-token
// path loads two bytes at a time). The same arithmetic in the same order per channel, so the same bits.
__global__ void __launch_bounds__(128)
short_conv_decode_bf16x8_kernel(const __nv_bfloat16* proj, const float* __restrict__ kernel, float* state,
                                long long slot_stride, __nv_bfloat16* out, const int* span_begin, const int* span_slot,
                                int hidden, int taps) {
    chain_release();
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= hidden) return;
    const int keep = taps - 1;
    float w[8][kFewTaps];                           // constant data first
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int tap = 0; tap < kFewTaps; ++tap) w[j][tap] = tap < taps ? kernel[(size_t)(c + j) * taps + tap] : 0.0f;
    chain_wait();
    const int s = blockIdx.y;
    const int t = span_begin[s];
    float* st = state + (size_t)span_slot[s] * slot_stride + c;      // [keep][hidden]
    const __nv_bfloat16* p = proj + (size_t)t * 3 * hidden + c;
    const uint4 b_raw = *reinterpret_cast<const uint4*>(p);
    const uint4 c_raw = *reinterpret_cast<const uint4*>(p + hidden);
    const uint4 x_raw = *reinterpret_cast<const uint4*>(p + 2 * hidden);
    float old_taps[kFewTaps - 1][8];
#pragma unroll
    for (int tap = 0; tap < kFewTaps - 1; ++tap) {
        float4 lo = make_float4(0.0f, 0.0f, 0.0f, 0.0f), hi = lo;
        if (tap < keep) {
            lo = *reinterpret_cast<const float4*>(st + (size_t)tap * hidden);
            hi = *reinterpret_cast<const float4*>(st + (size_t)tap * hidden + 4);
        }
        old_taps[tap][0] = lo.x; old_taps[tap][1] = lo.y; old_taps[tap][2] = lo.z; old_taps[tap][3] = lo.w;
        old_taps[tap][4] = hi.x; old_taps[tap][5] = hi.y; old_taps[tap][6] = hi.z; old_taps[tap][7] = hi.w;
    }
    const __nv_bfloat16* bb = reinterpret_cast<const __nv_bfloat16*>(&b_raw);
    const __nv_bfloat16* cc = reinterpret_cast<const __nv_bfloat16*>(&c_raw);
    const __nv_bfloat16* xx = reinterpret_cast<const __nv_bfloat16*>(&x_raw);
    float bx[8];
    uint4 packed;
    __nv_bfloat16* result = reinterpret_cast<__nv_bfloat16*>(&packed);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        bx[j] = to_float(bb[j]) * to_float(xx[j]);
        float conv = 0.0f;
#pragma unroll
        for (int tap = 0; tap < kFewTaps; ++tap) {
            if (tap < keep) conv += w[j][tap] * old_taps[tap < kFewTaps - 1 ? tap : 0][j];
            else if (tap == keep) conv += w[j][tap] * bx[j];
        }
        result[j] = from_float<__nv_bfloat16>(to_float(cc[j]) * conv);
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * hidden + c) = packed;
#pragma unroll
    for (int tap = 0; tap < kFewTaps - 1; ++tap) {
        if (tap + 1 < keep) {
            *reinterpret_cast<float4*>(st + (size_t)tap * hidden) =
                make_float4(old_taps[tap + 1 < kFewTaps - 1 ? tap + 1 : 0][0], old_taps[tap + 1 < kFewTaps - 1 ? tap + 1 : 0][1],
                            old_taps[tap + 1 < kFewTaps - 1 ? tap + 1 : 0][2], old_taps[tap + 1 < kFewTaps - 1 ? tap + 1 : 0][3]);
            *reinterpret_cast<float4*>(st + (size_t)tap * hidden + 4) =
                make_float4(old_taps[tap + 1 < kFewTaps - 1 ? tap + 1 : 0][4], old_taps[tap + 1 < kFewTaps - 1 ? tap + 1 : 0][5],
                            old_taps[tap + 1 < kFewTaps - 1 ? tap + 1 : 0][6], old_taps[tap + 1 < kFewTaps - 1 ? tap + 1 : 0][7]);
        } else if (tap + 1 == keep) {
            *reinterpret_cast<float4*>(st + (size_t)tap * hidden) = make_float4(bx[0], bx[1], bx[2], bx[3]);
            *reinterpret_cast<float4*>(st + (size_t)tap * hidden + 4) = make_float4(bx[4], bx[5], bx[6], bx[7]);
        }
    }
}

template <typename A>
__global__ void short_conv_spans_kernel(const A* proj, const float* __restrict__ kernel, float* state,
                                        long long slot_stride, A* out, const int* span_begin, const int* span_slot,
                                        int hidden, int taps) {
    chain_release();
    short_conv_spans_body<A>(proj, kernel, state, slot_stride, out, span_begin, span_slot, hidden, taps,
                             blockIdx.x * blockDim.x + threadIdx.x, blockIdx.y);
}

__global__ void __launch_bounds__(128)
short_conv_tokens_window_kernel(const __nv_bfloat16* proj, const float* __restrict__ kernel, __nv_bfloat16* out,
                                const int* token_span, const int* span_begin, int hidden, int taps, int tokens) {
    chain_release();
    short_conv_window_body(proj, kernel, out, token_span, span_begin, hidden, taps, tokens,
                           (blockIdx.x * blockDim.x + threadIdx.x) * 8, blockIdx.y);
}

// Both of them in one launch for prompt portions (bfloat16, at most four taps): the first blocks do the spans'
// work, which is a chain of dependent loads per thread and would otherwise stand alone on the GPU for
// several microseconds, the others the sliding windows; the two write different tokens.
__global__ void __launch_bounds__(128)
short_conv_prompt_kernel(const __nv_bfloat16* proj, const float* __restrict__ kernel, float* state, long long slot_stride,
                         __nv_bfloat16* out, const int* token_span, const int* span_begin, const int* span_slot,
                         int hidden, int taps, int tokens, int spans, int span_blocks_x, int window_blocks_x) {
    chain_release();
    int block = blockIdx.x;
    const int span_blocks = span_blocks_x * spans;
    if (block < span_blocks) {
        short_conv_spans_body<__nv_bfloat16>(proj, kernel, state, slot_stride, out, span_begin, span_slot, hidden, taps,
                                             (block % span_blocks_x) * blockDim.x + threadIdx.x, block / span_blocks_x);
    } else {
        block -= span_blocks;
        short_conv_window_body(proj, kernel, out, token_span, span_begin, hidden, taps, tokens,
                               ((block % window_blocks_x) * blockDim.x + threadIdx.x) * 8, block / window_blocks_x);
    }
}

}  // namespace celeg_b200

using namespace celeg_b200;

CELEG_API int celeg_short_conv(const void* proj, const float* kernel, float* state, long long slot_stride,
                               void* out, const int* token_span, const int* span_begin, const int* span_slot,
                               int tokens, int spans, int hidden, int taps, int max_span, int act_dtype,
                               cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && spans >= 0 && hidden > 0, "short_conv: invalid sizes tokens=%d spans=%d hidden=%d",
                  tokens, spans, hidden);
    CELEG_REQUIRE(taps >= 1 && taps <= kMaxTaps, "short_conv: kernel length %d is outside 1..%d", taps, kMaxTaps);
    CELEG_REQUIRE(act_dtype == kFloat32 || act_dtype == kBFloat16, "short_conv: unknown dtype code %d", act_dtype);
    if (tokens == 0) return 0;
    CELEG_REQUIRE(tokens <= 65535 && spans <= 65535, "short_conv: %d tokens or %d spans exceed one launch (65535)",
                  tokens, spans);
    const bool windows = act_dtype == kBFloat16 && hidden % 8 == 0 && ((((size_t)proj) | ((size_t)out)) & 15) == 0 &&
                         taps <= kFewTaps && tokens >= 4 * kTokensPerThread && max_span > taps - 1;
    if (windows) {
        const int span_blocks_x = (hidden + 127) / 128, window_blocks_x = (hidden / 8 + 127) / 128;
        const long long blocks = (long long)span_blocks_x * spans +
                                 (long long)window_blocks_x * ((tokens + kTokensPerThread - 1) / kTokensPerThread);
        if (blocks <= 0x7fffffffLL) {
            launch_chained(short_conv_prompt_kernel, (unsigned)blocks, 128, 0, stream, (const __nv_bfloat16*)proj, kernel,
                           state, slot_stride, (__nv_bfloat16*)out, token_span, span_begin, span_slot, hidden, taps,
                           tokens, spans, span_blocks_x, window_blocks_x);
            return check_launch("short_conv (prompt portions)");
        }
    }
    if (act_dtype == kBFloat16 && max_span == 1 && tokens == spans && spans >= 16 && taps >= 2 && taps <= kFewTaps &&
        hidden % 8 == 0 && (slot_stride & 3) == 0 &&
        ((((size_t)proj) | ((size_t)out) | ((size_t)state) | ((size_t)kernel)) & 15) == 0) {
        // every request brings one token, and there are many of them: eight channels a thread
        const int vec_threads = hidden / 8 >= 128 ? 128 : ((hidden / 8 + 31) / 32) * 32;
        dim3 grid((hidden / 8 + vec_threads - 1) / vec_threads, spans);
        launch_chained(short_conv_decode_bf16x8_kernel, grid, vec_threads, 0, stream, (const __nv_bfloat16*)proj, kernel,
                       state, slot_stride, (__nv_bfloat16*)out, span_begin, span_slot, hidden, taps);
        return check_launch("short_conv (decoded tokens)");
    }
    const int threads = hidden >= 256 ? 256 : ((hidden + 31) / 32) * 32;
    dim3 span_grid((hidden + threads - 1) / threads, spans);
    if (act_dtype == kFloat32)
        launch_chained(short_conv_spans_kernel<float>, span_grid, threads, 0, stream, (const float*)proj, kernel, state,
                       slot_stride, (float*)out, span_begin, span_slot, hidden, taps);
    else
        launch_chained(short_conv_spans_kernel<__nv_bfloat16>, span_grid, threads, 0, stream,
                       (const __nv_bfloat16*)proj, kernel, state, slot_stride, (__nv_bfloat16*)out, span_begin,
                       span_slot, hidden, taps);
    int status = check_launch("short_conv (spans)");
    if (status != 0 || max_span <= taps - 1) return status;       // no token lies past the first taps-1 of its span
    if (act_dtype == kBFloat16 && hidden % 8 == 0 && ((((size_t)proj) | ((size_t)out)) & 15) == 0 && taps <= kFewTaps &&
        tokens >= 4 * kTokensPerThread) {
        const int vec_threads = hidden / 8 >= 128 ? 128 : ((hidden / 8 + 31) / 32) * 32;
        dim3 grid((hidden / 8 + vec_threads - 1) / vec_threads, (tokens + kTokensPerThread - 1) / kTokensPerThread);
        launch_chained(short_conv_tokens_window_kernel, grid, vec_threads, 0, stream, (const __nv_bfloat16*)proj, kernel,
                       (__nv_bfloat16*)out, token_span, span_begin, hidden, taps, tokens);
    } else if (act_dtype == kBFloat16 && hidden % 8 == 0 && ((((size_t)proj) | ((size_t)out)) & 15) == 0) {
        const int vec_threads = hidden / 8 >= 128 ? 128 : ((hidden / 8 + 31) / 32) * 32;
        dim3 grid((hidden / 8 + vec_threads - 1) / vec_threads, tokens);
        launch_chained(short_conv_tokens_bf16x8_kernel, grid, vec_threads, 0, stream, (const __nv_bfloat16*)proj, kernel,
                       (__nv_bfloat16*)out, token_span, span_begin, hidden, taps);
    } else {
        dim3 grid((hidden + threads - 1) / threads, tokens);
        if (act_dtype == kFloat32)
            launch_chained(short_conv_tokens_kernel<float>, grid, threads, 0, stream, (const float*)proj, kernel,
                           (float*)out, token_span, span_begin, hidden, taps);
        else
            launch_chained(short_conv_tokens_kernel<__nv_bfloat16>, grid, threads, 0, stream,
                           (const __nv_bfloat16*)proj, kernel, (__nv_bfloat16*)out, token_span, span_begin, hidden,
                           taps);
    }
    return check_launch("short_conv (tokens)");
}
