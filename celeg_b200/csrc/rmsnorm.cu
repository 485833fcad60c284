// Fused residual add + RMSNorm with an optional row gather.
//
//   x = residual[r] (+ delta[r]);  residual[r] = x (if asked);  out[i] = x / sqrt(mean(x^2) + eps) * w
//
// with r = rows[i] when a row list is given (the rows whose logits are wanted), else r = i.
// The sum, the reciprocal root and the product with the weight are float32; the result is
// rounded once to the activation type. Counterparts in celeg: rmsnorm_kernel and
// residual_kernel (src/backend/cuda/kernels/norm.cuh:1-62), which run as two launches and
// round the normalised value to bf16 before the weight multiply.
#include "common.cuh"

namespace celeg_b200 {

template <typename A>
__global__ void add_rmsnorm_kernel(float* residual, const A* delta,
                                   const float* __restrict__ weight, A* out,
                                   const int* rows, int width, float eps, int write_residual) {
    __shared__ float scratch[33];
    chain_release();
    chain_wait();
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float* res = residual + (size_t)r * width;
    const A* del = delta ? delta + (size_t)r * width : nullptr;
    float sum = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float x = res[c];
        if (del) x += to_float(del[c]);
        sum += x * x;
    }
    sum = block_sum(sum, scratch);
    const float inv = 1.0f / sqrtf(sum / (float)width + eps);
    A* dst = out + (size_t)i * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float x = res[c];
        if (del) x += to_float(del[c]);
        if (write_residual && del) res[c] = x;
        dst[c] = from_float<A>(x * inv * weight[c]);
    }
}

// Widths that are a multiple of 4 with 16-byte aligned rows: a thread keeps its elements in registers
// between the two passes (the residual is read once), four at a time.
template <typename A, int kPerThread>
__global__ void add_rmsnorm_vec4_kernel(float* residual, const A* delta, const float* __restrict__ weight, A* out,
                                        const int* rows, int width, float eps, int write_residual) {
    __shared__ float scratch[33];
    chain_release();
    chain_wait();
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float4* res = reinterpret_cast<float4*>(residual + (size_t)r * width);
    const int quads = width >> 2;
    float4 x[kPerThread];
    float sum = 0.0f;
#pragma unroll
    for (int u = 0; u < kPerThread; ++u) {
        const int q = threadIdx.x + u * blockDim.x;
        if (q < quads) {
            float4 v = res[q];
            if (delta) {
                const A* d = delta + (size_t)r * width + 4 * q;
                if (sizeof(A) == 2) {
                    const uint2 raw = *reinterpret_cast<const uint2*>(d);
                    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
                    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
                    v.x += lo.x; v.y += lo.y; v.z += hi.x; v.w += hi.y;
                } else {
                    const float4 dv = *reinterpret_cast<const float4*>(d);
                    v.x += dv.x; v.y += dv.y; v.z += dv.z; v.w += dv.w;
                }
                if (write_residual) res[q] = v;
            }
            x[u] = v;
            sum += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    }
    sum = block_sum(sum, scratch);
    const float inv = 1.0f / sqrtf(sum / (float)width + eps);
#pragma unroll
    for (int u = 0; u < kPerThread; ++u) {
        const int q = threadIdx.x + u * blockDim.x;
        if (q < quads) {
            const float4 w = __ldg(reinterpret_cast<const float4*>(weight) + q);
            const float4 v = x[u];
            A* dst = out + (size_t)i * width + 4 * q;
            if (sizeof(A) == 2) {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * inv * w.x, v.y * inv * w.y);
                const __nv_bfloat162 hi = __floats2bfloat162_rn(v.z * inv * w.z, v.w * inv * w.w);
                uint2 raw;
                raw.x = *reinterpret_cast<const unsigned*>(&lo);
                raw.y = *reinterpret_cast<const unsigned*>(&hi);
                *reinterpret_cast<uint2*>(dst) = raw;
            } else {
                *reinterpret_cast<float4*>(dst) = make_float4(v.x * inv * w.x, v.y * inv * w.y, v.z * inv * w.z,
                                                              v.w * inv * w.w);
            }
        }
    }
}

// Plain RMSNorm over rows of `width` elements of an activation tensor (used for parts that
// normalise something other than the residual stream).
template <typename A>
__global__ void rmsnorm_rows_kernel(const A* in, const float* __restrict__ weight,
                                    A* out, int width, float eps) {
    __shared__ float scratch[33];
    const A* src = in + (size_t)blockIdx.x * width;
    float sum = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float x = to_float(src[c]);
        sum += x * x;
    }
    sum = block_sum(sum, scratch);
    const float inv = 1.0f / sqrtf(sum / (float)width + eps);
    A* dst = out + (size_t)blockIdx.x * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x)
        dst[c] = from_float<A>(to_float(src[c]) * inv * weight[c]);
}

static int norm_threads(int width) { return width >= 2048 ? 512 : width >= 512 ? 256 : 128; }

}  // namespace celeg_b200

using namespace celeg_b200;

CELEG_API int celeg_add_rmsnorm(float* residual, const void* delta, const float* weight, void* out,
                                const int* rows, int n_rows, int width, float eps, int write_residual,
                                int act_dtype, cudaStream_t stream) {
    CELEG_REQUIRE(n_rows >= 0 && width > 0 && eps > 0.0f, "add_rmsnorm: invalid sizes rows=%d width=%d eps=%g",
                  n_rows, width, eps);
    CELEG_REQUIRE(!(rows && write_residual), "add_rmsnorm: a gathered norm does not write the residual back");
    if (n_rows == 0) return 0;
    constexpr int kPerThread = 4;
    const bool aligned = (((size_t)residual | (size_t)delta | (size_t)weight | (size_t)out) & 15) == 0;
    if (width % 4 == 0 && width <= 1024 * 4 * kPerThread && aligned && (act_dtype == kFloat32 || act_dtype == kBFloat16)) {
        const int quads = width / 4;
        int vec_threads = (quads + kPerThread - 1) / kPerThread;
        vec_threads = (vec_threads + 31) / 32 * 32;
        if (vec_threads < 64) vec_threads = 64;
        if (act_dtype == kFloat32)
            launch_chained_class(kChainNorm, add_rmsnorm_vec4_kernel<float, kPerThread>, n_rows, vec_threads, 0, stream,
                                 residual, (const float*)delta, weight, (float*)out, rows, width, eps, write_residual);
        else
            launch_chained_class(kChainNorm, add_rmsnorm_vec4_kernel<__nv_bfloat16, kPerThread>, n_rows, vec_threads, 0,
                                 stream, residual, (const __nv_bfloat16*)delta, weight, (__nv_bfloat16*)out, rows, width,
                                 eps, write_residual);
        return check_launch("add_rmsnorm");
    }
    const int threads = norm_threads(width);
    if (act_dtype == kFloat32)
        launch_chained_class(kChainNorm, add_rmsnorm_kernel<float>, n_rows, threads, 0, stream, residual, (const float*)delta,
                       weight, (float*)out, rows, width, eps, write_residual);
    else if (act_dtype == kBFloat16)
        launch_chained_class(kChainNorm, add_rmsnorm_kernel<__nv_bfloat16>, n_rows, threads, 0, stream, residual,
                       (const __nv_bfloat16*)delta, weight, (__nv_bfloat16*)out, rows, width, eps, write_residual);
    else
        CELEG_REQUIRE(false, "add_rmsnorm: unknown dtype code %d", act_dtype);
    return check_launch("add_rmsnorm");
}

CELEG_API int celeg_rmsnorm_rows(const void* in, const float* weight, void* out, int n_rows, int width,
                                 float eps, int act_dtype, cudaStream_t stream) {
    CELEG_REQUIRE(n_rows >= 0 && width > 0 && eps > 0.0f, "rmsnorm_rows: invalid sizes rows=%d width=%d eps=%g",
                  n_rows, width, eps);
    if (n_rows == 0) return 0;
    const int threads = norm_threads(width);
    if (act_dtype == kFloat32)
        rmsnorm_rows_kernel<float><<<n_rows, threads, 0, stream>>>((const float*)in, weight, (float*)out, width,
                                                                   eps);
    else if (act_dtype == kBFloat16)
        rmsnorm_rows_kernel<__nv_bfloat16><<<n_rows, threads, 0, stream>>>(
            (const __nv_bfloat16*)in, weight, (__nv_bfloat16*)out, width, eps);
    else
        CELEG_REQUIRE(false, "rmsnorm_rows: unknown dtype code %d", act_dtype);
    return check_launch("rmsnorm_rows");
}
