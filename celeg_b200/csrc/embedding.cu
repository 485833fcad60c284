// Embedding gather: residual[t, :] = multiplier * table[token[t], :], written as float32
// (the residual stream is kept in 32-bit on both precision paths).
// Counterpart in celeg: embedding_batch_kernel (src/backend/cuda/kernels/embedding.cu:26).
#include "common.cuh"

namespace celeg_b200 {

// next_w != null: the first half of a split RMSNorm (gemv_bf16.cu) for the norm that follows:
// xw_out[t, :] = bf16(residual * next_w) and sumsq_out[t] = sum(residual^2).
template <typename W>
__global__ void embedding_kernel(const W* __restrict__ table, const int* tokens,
                                 float* out, int hidden, int vocab, float multiplier, const float* next_w,
                                 __nv_bfloat16* xw_out, float* sumsq_out, int sumsq_stride) {
    __shared__ float scratch[33];
    chain_release();
    chain_wait();
    const int row = blockIdx.x;
    const int token = tokens[row];
    float* dst = out + (size_t)row * hidden;
    const bool valid = token >= 0 && token < vocab;          // the host refuses other ids before launch
    const W* src = table + (size_t)(valid ? token : 0) * hidden;
    float squares = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = valid ? to_float(src[i]) * multiplier : 0.0f;
        dst[i] = v;
        if (next_w) {
            xw_out[(size_t)row * hidden + i] = __float2bfloat16_rn(v * next_w[i]);
            squares += v * v;
        }
    }
    if (next_w) {
        squares = block_sum(squares, scratch);
        if (threadIdx.x == 0) sumsq_out[(size_t)row * sumsq_stride] = squares;
    }
}

}  // namespace celeg_b200

using namespace celeg_b200;

static int embedding_checked(const void* table, int table_dtype, const int* tokens, float* out, int rows, int hidden,
                             int vocab, float multiplier, const float* next_w, void* xw_out, float* sumsq_out,
                             int sumsq_stride, cudaStream_t stream) {
    CELEG_REQUIRE(rows >= 0 && hidden > 0 && vocab > 0, "embedding: invalid sizes rows=%d hidden=%d vocab=%d",
                  rows, hidden, vocab);
    CELEG_REQUIRE(!next_w || (xw_out && sumsq_out && sumsq_stride >= 1),
                  "embedding: preparing the norm that follows needs its two outputs");
    if (rows == 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == kFloat32)
        launch_chained(embedding_kernel<float>, rows, threads, 0, stream, (const float*)table, tokens, out, hidden,
                       vocab, multiplier, next_w, (__nv_bfloat16*)xw_out, sumsq_out, sumsq_stride);
    else if (table_dtype == kBFloat16)
        launch_chained(embedding_kernel<__nv_bfloat16>, rows, threads, 0, stream, (const __nv_bfloat16*)table,
                       tokens, out, hidden, vocab, multiplier, next_w, (__nv_bfloat16*)xw_out, sumsq_out, sumsq_stride);
    else
        CELEG_REQUIRE(false, "embedding: unknown dtype code %d", table_dtype);
    return check_launch("embedding");
}

CELEG_API int celeg_embedding(const void* table, int table_dtype, const int* tokens, float* out, int rows,
                              int hidden, int vocab, float multiplier, cudaStream_t stream) {
    return embedding_checked(table, table_dtype, tokens, out, rows, hidden, vocab, multiplier, nullptr, nullptr,
                             nullptr, 0, stream);
}

// The gather and, for the RMSNorm that follows, the first half of a split norm: xw_out [rows, hidden]
// bfloat16 = residual * next_w, sumsq_out[row * sumsq_stride] = sum of the row's squares.
CELEG_API int celeg_embedding_split_norm(const void* table, int table_dtype, const int* tokens, float* out, int rows,
                                         int hidden, int vocab, float multiplier, const float* next_w, void* xw_out,
                                         float* sumsq_out, int sumsq_stride, cudaStream_t stream) {
    return embedding_checked(table, table_dtype, tokens, out, rows, hidden, vocab, multiplier, next_w, xw_out,
                             sumsq_out, sumsq_stride, stream);
}
