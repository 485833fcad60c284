// SwiGLU activation on the fused gate|up projection: out[t, i] = silu(g[t, i]) * u[t, i] with
// g = in[t, 0:I], u = in[t, I:2I], silu(g) = g / (1 + exp(-g)), computed in float32 and rounded
// once. Counterpart in celeg: swiglu_interleaved_kernel (src/backend/cuda/kernels/qkv_rope.cuh:24-39),
// which rounds silu(g) to bf16 before the product.
#include "common.cuh"

namespace celeg_b200 {

template <typename A>
__global__ void swiglu_kernel(const A* in, A* out, long long total, int inner) {
    chain_release();
    chain_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const long long t = idx / inner;
        const int i = (int)(idx % inner);
        const A* row = in + t * 2 * inner;
        const float g = to_float(row[i]);
        const float u = to_float(row[inner + i]);
        out[idx] = from_float<A>(g / (1.0f + expf(-g)) * u);
    }
}

}  // namespace celeg_b200

using namespace celeg_b200;

CELEG_API int celeg_swiglu(const void* gate_up, void* out, int tokens, int inner, int act_dtype,
                           cudaStream_t stream) {
    CELEG_REQUIRE(tokens >= 0 && inner > 0, "swiglu: invalid sizes tokens=%d inner=%d", tokens, inner);
    if (tokens == 0) return 0;
    const long long total = (long long)tokens * inner;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads < 148LL * 16 ? (total + threads - 1) / threads
                                                                                      : 148LL * 16);
    if (act_dtype == kFloat32)
        launch_chained(swiglu_kernel<float>, blocks, threads, 0, stream, (const float*)gate_up, (float*)out, total,
                       inner);
    else if (act_dtype == kBFloat16)
        launch_chained(swiglu_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (const __nv_bfloat16*)gate_up,
                       (__nv_bfloat16*)out, total, inner);
    else
        CELEG_REQUIRE(false, "swiglu: unknown dtype code %d", act_dtype);
    return check_launch("swiglu");
}
