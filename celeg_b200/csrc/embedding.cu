// Embedding gather: residual[t, :] = multiplier * table[token[t], :], written as float32
// (the residual stream is kept in 32-bit on both precision paths).
// Counterpart in celeg: embedding_batch_kernel (src/backend/cuda/kernels/embedding.cu:26).
#include "common.cuh"

namespace celeg_b200 {

template <typename W>
__global__ void embedding_kernel(const W* __restrict__ table, const int* tokens,
                                 float* out, int hidden, int vocab, float multiplier) {
    chain_release();
    chain_wait();
    const int row = blockIdx.x;
    const int token = tokens[row];
    float* dst = out + (size_t)row * hidden;
    if (token < 0 || token >= vocab) {          // the host refuses such ids before launch
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.0f;
        return;
    }
    const W* src = table + (size_t)token * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_float(src[i]) * multiplier;
}

}  // namespace celeg_b200

using namespace celeg_b200;

CELEG_API int celeg_embedding(const void* table, int table_dtype, const int* tokens, float* out, int rows,
                              int hidden, int vocab, float multiplier, cudaStream_t stream) {
    CELEG_REQUIRE(rows >= 0 && hidden > 0 && vocab > 0, "embedding: invalid sizes rows=%d hidden=%d vocab=%d",
                  rows, hidden, vocab);
    if (rows == 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == kFloat32)
        launch_chained(embedding_kernel<float>, rows, threads, 0, stream, (const float*)table, tokens, out, hidden,
                       vocab, multiplier);
    else if (table_dtype == kBFloat16)
        launch_chained(embedding_kernel<__nv_bfloat16>, rows, threads, 0, stream, (const __nv_bfloat16*)table,
                       tokens, out, hidden, vocab, multiplier);
    else
        CELEG_REQUIRE(false, "embedding: unknown dtype code %d", table_dtype);
    return check_launch("embedding");
}
