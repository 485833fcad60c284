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
// Work split. Tokens whose taps all lie inside the span (index in span >= L-1) are independent:
// one block row per token. Everything that touches the slot - the first L-1 tokens of a span
// and the slot's new content - is done by ONE thread per (span, channel), which reads the old
// state into registers before it writes, so the update is in place without a second buffer.
// Both paths add the taps in the same order, so a token's result does not depend on where the
// span was cut.
//
// Counterparts in celeg: conv_decode_batch_ptrs_kernel and conv_ragged_prefill_kernel
// (src/backend/cuda/kernels/shortconv.cuh:1-33, 34-), where one thread walks a whole span
// serially and the state is a bf16 ring indexed by position % L.
#include "common.cuh"

namespace celeg_b200 {

constexpr int kMaxTaps = 16;

template <typename A>
__global__ void short_conv_kernel(const A* proj, const float* __restrict__ kernel,
                                  float* state, long long slot_stride, A* out,
                                  const int* token_span, const int* span_begin,
                                  const int* span_slot, int tokens, int spans, int hidden,
                                  int taps) {
    chain_release();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= hidden) return;
    const int y = blockIdx.y;
    const size_t row = (size_t)3 * hidden;
    float w[kMaxTaps];
#pragma unroll
    for (int i = 0; i < kMaxTaps; ++i) w[i] = i < taps ? kernel[(size_t)c * taps + i] : 0.0f;   // constant data
    chain_wait();

    if (y < tokens) {
        const int t = y;
        const int first = span_begin[token_span[t]];
        if (t - first < taps - 1) return;           // handled with the slot below
        float conv = 0.0f;
        for (int tap = 0; tap < taps; ++tap) {
            const A* p = proj + (size_t)(t - (taps - 1) + tap) * row;
            conv += w[tap] * (to_float(p[c]) * to_float(p[2 * hidden + c]));
        }
        out[(size_t)t * hidden + c] = from_float<A>(to_float(proj[(size_t)t * row + hidden + c]) * conv);
        return;
    }

    const int s = y - tokens;
    if (s >= spans) return;
    const int first = span_begin[s];
    const int count = span_begin[s + 1] - first;
    const int keep = taps - 1;
    float* st = state + (size_t)span_slot[s] * slot_stride;     // [keep][hidden]
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

}  // namespace celeg_b200

using namespace celeg_b200;

CELEG_API int celeg_short_conv(const void* proj, const float* kernel, float* state, long long slot_stride,
                               void* out, const int* token_span, const int* span_begin, const int* span_slot,
                               int tokens, int spans, int hidden, int taps, int act_dtype,
                               cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && spans >= 0 && hidden > 0, "short_conv: invalid sizes tokens=%d spans=%d hidden=%d",
                  tokens, spans, hidden);
    CELEG_REQUIRE(taps >= 1 && taps <= kMaxTaps, "short_conv: kernel length %d is outside 1..%d", taps, kMaxTaps);
    if (tokens == 0) return 0;
    CELEG_REQUIRE(tokens + spans <= 65535, "short_conv: %d tokens + %d spans exceed one launch (65535)", tokens,
                  spans);
    const int threads = hidden >= 256 ? 256 : ((hidden + 31) / 32) * 32;
    dim3 grid((hidden + threads - 1) / threads, tokens + spans);
    if (act_dtype == kFloat32)
        launch_chained(short_conv_kernel<float>, grid, threads, 0, stream, (const float*)proj, kernel, state,
                       slot_stride, (float*)out, token_span, span_begin, span_slot, tokens, spans, hidden, taps);
    else if (act_dtype == kBFloat16)
        launch_chained(short_conv_kernel<__nv_bfloat16>, grid, threads, 0, stream, (const __nv_bfloat16*)proj,
                       kernel, state, slot_stride, (__nv_bfloat16*)out, token_span, span_begin, span_slot, tokens,
                       spans, hidden, taps);
    else
        CELEG_REQUIRE(false, "short_conv: unknown dtype code %d", act_dtype);
    return check_launch("short_conv");
}
