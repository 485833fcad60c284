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

// bfloat16 with a width that is a multiple of 8: eight elements per thread, 16-byte loads and stores.
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* in, __nv_bfloat16* out, long long total_vecs,
                                     int inner_vecs) {
    chain_release();
    chain_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total_vecs; idx += stride) {
        const long long t = idx / inner_vecs;
        const int v = (int)(idx % inner_vecs);
        const uint4* row = reinterpret_cast<const uint4*>(in) + t * 2 * inner_vecs;
        const uint4 g4 = row[v];
        const uint4 u4 = row[inner_vecs + v];
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
        uint4 r;
        __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 g = __bfloat1622float2(g2[i]);
            const float2 u = __bfloat1622float2(u2[i]);
            r2[i] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
        }
        reinterpret_cast<uint4*>(out)[idx] = r;
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
    else if (act_dtype == kBFloat16 && inner % 8 == 0 && ((((size_t)gate_up) | ((size_t)out)) & 15) == 0) {
        const long long vecs = total / 8;
        const unsigned vec_blocks = (unsigned)((vecs + threads - 1) / threads < 148LL * 32 ? (vecs + threads - 1) / threads
                                                                                          : 148LL * 32);
        launch_chained(swiglu_bf16x8_kernel, vec_blocks, threads, 0, stream, (const __nv_bfloat16*)gate_up,
                       (__nv_bfloat16*)out, vecs, inner / 8);
    } else if (act_dtype == kBFloat16)
        launch_chained(swiglu_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (const __nv_bfloat16*)gate_up,
                       (__nv_bfloat16*)out, total, inner);
    else
        CELEG_REQUIRE(false, "swiglu: unknown dtype code %d", act_dtype);
    return check_launch("swiglu");
}
