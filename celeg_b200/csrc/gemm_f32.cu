// True 32-bit matrix product Y[M,N] = X[M,K] * W[N,K]^T (both operands row-major with K
// contiguous, as checkpoints store projection weights): float32 operands, FFMA accumulation in
// ascending k, no tensor cores and no reduced-precision operand mode. Every output element is
// produced by one thread with the same order of additions whatever M is, so a row's result
// does not depend on what else is in the batch.
//
// celeg has no 32-bit GPU path (its CUDA backend calls cuBLAS with bf16 operands:
// src/backend/cuda/runtime/gemm_dispatcher.cpp:49-64); this kernel is what makes the float32
// model path independent of any library's math mode.
#include "common.cuh"

namespace celeg_b200 {

constexpr int kTileM = 64, kTileN = 64, kTileK = 16;

// 256 threads; thread (ty, tx) owns a 4x4 patch: rows ty*4.., columns tx*4..
__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                       float* __restrict__ y, int m, int n, int k, int ldx,
                                                       int ldw, int ldy, int accumulate) {
    __shared__ float xs[kTileK][kTileM + 4];
    __shared__ float ws[kTileK][kTileN + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int row0 = blockIdx.y * kTileM, col0 = blockIdx.x * kTileN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < k; k0 += kTileK) {
        // each thread loads 4 elements of each tile: tile row = idx / 16, k = idx % 16
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = threadIdx.x + i * 256;
            const int r = idx >> 4, kk = idx & 15;
            const int gr = row0 + r, gc = col0 + r, gk = k0 + kk;
            xs[kk][r] = (gr < m && gk < k) ? x[(size_t)gr * ldx + gk] : 0.0f;
            ws[kk][r] = (gc < n && gk < k) ? w[(size_t)gc * ldw + gk] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kTileK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gr = row0 + ty * 4 + i;
        if (gr >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gc = col0 + tx * 4 + j;
            if (gc >= n) continue;
            float* dst = y + (size_t)gr * ldy + gc;
            *dst = accumulate ? *dst + acc[i][j] : acc[i][j];
        }
    }
}

}  // namespace celeg_b200

using namespace celeg_b200;

CELEG_API int celeg_gemm_f32(const float* x, const float* w, float* y, int m, int n, int k, int ldx, int ldw,
                             int ldy, int accumulate, cudaStream_t stream) {
    CELEG_REQUIRE(m >= 0 && n > 0 && k > 0 && ldx >= k && ldw >= k && ldy >= n,
                  "gemm_f32: invalid sizes m=%d n=%d k=%d ldx=%d ldw=%d ldy=%d", m, n, k, ldx, ldw, ldy);
    if (m == 0) return 0;
    dim3 grid((n + kTileN - 1) / kTileN, (m + kTileM - 1) / kTileM);
    CELEG_REQUIRE(grid.y <= 65535, "gemm_f32: %d rows exceed one launch", m);
    gemm_f32_kernel<<<grid, 256, 0, stream>>>(x, w, y, m, n, k, ldx, ldw, ldy, accumulate);
    return check_launch("gemm_f32");
}
