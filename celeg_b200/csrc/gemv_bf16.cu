// Small-batch matrix product for decoding: Y[M,N] = X[M,K] * W[N,K]^T with M <= 16 rows of
// activations, bfloat16 operands, float32 accumulation. With so few rows the product is bound by
// reading W once from HBM, so the kernel is organised around that stream:
//
//   * W rows are the M dimension of mma.sync.m16n8k16 ("swap A and B"): a block owns 16 weight rows
//     (32 with the SwiGLU epilogue: 16 gate rows and their 16 up rows), its 8 warps take every
//     8th 32-element slice of K, and the eight partial tiles meet in shared memory.
//   * A thread loads 16 contiguous bytes of a weight row straight from global memory into the
//     registers of two MMAs: because the sum over k may run in any order, the 8 elements a thread
//     holds are declared to be k-slots {2c,2c+1,2c+8,2c+9} of two successive k16 steps, and the
//     activation fragment is loaded with the same permutation (also 16 contiguous bytes). No
//     shared-memory staging and no ldmatrix are needed, and every load is a full 16-byte vector.
//   * Several slices are in flight per warp (unrolled loads) to cover HBM latency.
//
// Epilogues: store (bfloat16 or float32), add into the float32 residual stream, SwiGLU, and the short
// convolution's gate (three weight tiles per block: the B, C and X rows of the same 16 channels of the
// input projection; bx = B*X, taps over the request's carried state, C * conv, state shifted; for steps
// in which every request brings ONE token).
// The number of warps per block (8, 16 or 32, all on the same 16 weight rows) is chosen by the host:
// a narrow matrix has few blocks, and only more warps per block put enough loads in flight to keep
// HBM busy. Any N; K must be a multiple of 8 (16-byte rows); otherwise the caller uses the library
// product.
// Across kernel boundaries: launched with programmatic stream serialization, a block issues its first weight
// loads before it waits for the kernel before it (weights are constant data), and its last blocks ask the
// first megabytes of the next product's weights into the L2 (GemvPrefetch).
//
// Counterpart in celeg: bf16_gemv_kernel for M = 1 (include/celeg/backend/cuda/kernels/gemv_kernels.cuh:12-44,
// one warp per output row, no tensor cores) and cuBLAS for M > 1.
#include "common.cuh"

namespace celeg_b200 {

constexpr int kGemvMaxConvTaps = 16;

enum GemvMode : int { kGemvStoreBf16 = 0, kGemvStoreF32 = 1, kGemvAddResidual = 2, kGemvSwiGlu = 3, kGemvConv = 4 };

struct GemvConvArgs {
    const float* conv_w;         // [channels, taps]
    int taps;
    float* state;                // this layer's state inside slot 0: [taps-1][channels] per slot
    long long slot_stride;
    const int* span_slot;        // state slot of row i (row i is the single token of span i)
};

// The norm between two products, split over them. The product that ends a part adds its result to
// the float32 residual stream; it can also leave behind x' = bf16(residual * w) with w the weight of the
// RMSNorm that follows, and each block's share of every row's sum of squares. The product that begins
// the next part takes x' as its operand and multiplies its sums by 1 / sqrt(mean square + eps) of
// the row (the scale is a factor of the whole row, so it commutes with the product). No kernel of its
// own for residual add + norm, nothing recomputed, no block waits for another.
struct GemvNormArgs {
    // this product's operand still lacks the row scale: [rows][partials_in] sums of squares, or null
    const float* sumsq_in;
    int partials_in;
    int sumsq_in_stride;
    float eps;
    int width;                   // the mean runs over this many elements
    // add-residual mode: also write x' for the norm that follows and this block's sums, or null
    const float* next_w;         // [n]
    __nv_bfloat16* xw_out;       // [m, ldxw]
    int ldxw;
    float* sumsq_out;            // [m][sumsq_out_stride], entry blockIdx.x
    int sumsq_out_stride;
};

__device__ __forceinline__ uint4 ldg_stream(const void* ptr) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(ptr));
    return v;
}

// Activations are written by the kernel before this one: the load is a volatile asm so that the
// compiler cannot move it above the wait for that kernel.
__device__ __forceinline__ uint4 ld_activation(const void* ptr) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(ptr));
    return v;
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                               unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The weights that the next product of the step will stream (a hint; may be empty). Each block asks the L2 for
// its slice of them when its own loads are done: a step of a model is a chain of short kernels, and between
// two of them (the last blocks draining, the launch, the first loads) the memory would otherwise stand idle.
struct GemvPrefetch {
    const char* ptr;
    long long bytes;      // a multiple of 16
};

// MT: 8-row tiles of activations (M <= 8*MT). WT: 16-row tiles of W per block (1, or 2 for SwiGLU).
template <int MT, int WT, int MODE, int kGemvUnroll, int kGemvWarps>
__global__ void __launch_bounds__(kGemvWarps * 32)
gemv_bf16_kernel(const __nv_bfloat16* x, int ldx, const __nv_bfloat16* __restrict__ w, int ldw,
                 void* __restrict__ y, int ldy, int m, int n, int k, int second_tile_offset, GemvConvArgs conv,
                 GemvNormArgs norm, GemvPrefetch ahead) {
    constexpr int kGemvThreads = kGemvWarps * 32;
    extern __shared__ __align__(16) float partial_raw[];
    __shared__ float row_scale[16];
    __shared__ float squares[16][17];
    float (*partial)[WT][MT][32][4] = reinterpret_cast<float (*)[WT][MT][32][4]>(partial_raw);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, c = lane & 3;
    const int row0 = blockIdx.x * 16;

    // weight rows of this thread: tile t covers rows row0 + t*second_tile_offset + {g, g+8}
    const __nv_bfloat16* w_lo[WT];
    const __nv_bfloat16* w_hi[WT];
#pragma unroll
    for (int t = 0; t < WT; ++t) {
        const int base = row0 + t * second_tile_offset;
        const int r_lo = min(base + g, n - 1 + t * second_tile_offset);     // rows past the end repeat the last one
        const int r_hi = min(base + g + 8, n - 1 + t * second_tile_offset);
        w_lo[t] = w + (size_t)r_lo * ldw + c * 8;
        w_hi[t] = w + (size_t)r_hi * ldw + c * 8;
    }
    // activation rows of this thread: tile j covers row j*8 + g (rows past m read row m-1, results unused)
    const __nv_bfloat16* x_row[MT];
#pragma unroll
    for (int j = 0; j < MT; ++j) x_row[j] = x + (size_t)min(j * 8 + g, m - 1) * ldx + c * 8;

    float acc[WT][MT][4];
#pragma unroll
    for (int t = 0; t < WT; ++t)
#pragma unroll
        for (int j = 0; j < MT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[t][j][e] = 0.0f;

    const int slices = k / 32;                       // full 32-element slices; the tail is handled below
    // Convolution epilogue with few taps: the thread that will finish element `threadIdx.x` of the block's tile
    // fetches its request's carried taps and its channel's kernel while the weights stream, instead of
    // after the sums are there (a chain of three dependent loads at the very end of a short kernel).
    constexpr int kEarlyTaps = 4;
    float early_history[kEarlyTaps - 1], early_kernel[kEarlyTaps];
    const bool early = MODE == kGemvConv && conv.taps <= kEarlyTaps && (int)threadIdx.x < MT * 128;
    // The epilogue that adds to the residual stream likewise: the stream's old value and the next norm's weight.
    float early_residual = 0.0f, early_next_w = 0.0f;
    const bool early_add = MODE == kGemvAddResidual && (int)threadIdx.x < MT * 128;
    auto fetch_early = [&]() {
        if (early_add) {
            const int i = threadIdx.x, j = i / 128, ln = (i % 128) / 4, e = i % 4;
            const int out_col = row0 + (ln >> 2) + ((e >> 1) << 3);
            const int out_row = j * 8 + ((ln & 3) << 1) + (e & 1);
            if (out_row < m && out_col < n) {
                early_residual = reinterpret_cast<const float*>(y)[(size_t)out_row * ldy + out_col];
                if (norm.next_w) early_next_w = norm.next_w[out_col];
            }
        }
        if (!early) return;
        const int i = threadIdx.x, j = i / 128, ln = (i % 128) / 4, e = i % 4;
        const int out_col = row0 + (ln >> 2) + ((e >> 1) << 3);
        const int out_row = j * 8 + ((ln & 3) << 1) + (e & 1);
        if (out_row >= m || out_col >= n) return;
        const int keep = conv.taps - 1;
        const float* st = conv.state + (size_t)conv.span_slot[out_row] * conv.slot_stride + out_col;
        const float* cw = conv.conv_w + (size_t)out_col * conv.taps;
#pragma unroll
        for (int tp = 0; tp < kEarlyTaps - 1; ++tp) early_history[tp] = tp < keep ? st[(size_t)tp * n] : 0.0f;
#pragma unroll
        for (int tp = 0; tp < kEarlyTaps; ++tp) early_kernel[tp] = tp < conv.taps ? cw[tp] : 0.0f;
    };
    bool waited = false;
    for (int s0 = warp; s0 < slices; s0 += kGemvWarps * kGemvUnroll) {
        uint4 a_lo[kGemvUnroll][WT], a_hi[kGemvUnroll][WT];
#pragma unroll
        for (int u = 0; u < kGemvUnroll; ++u) {
            const int s = s0 + u * kGemvWarps;
            if (s < slices) {
#pragma unroll
                for (int t = 0; t < WT; ++t) {
                    a_lo[u][t] = ldg_stream(w_lo[t] + s * 32);
                    a_hi[u][t] = ldg_stream(w_hi[t] + s * 32);
                }
            }
        }
        // the first batch of weights (constant data) is already on its way when the kernel starts
        // to wait for the activations of the kernel before it
        const bool first = !waited;
        if (!waited) {
            chain_wait();
            waited = true;
            fetch_early();
        }
        uint4 b[kGemvUnroll][MT];
#pragma unroll
        for (int u = 0; u < kGemvUnroll; ++u) {
            const int s = s0 + u * kGemvWarps;
            if (s < slices) {
#pragma unroll
                for (int j = 0; j < MT; ++j) b[u][j] = ld_activation(x_row[j] + s * 32);
            }
        }
        if (first && norm.sumsq_in) {
            // the rows' scales (needed by the epilogue only), while weights and activations are on their
            // way: a warp per row
            for (int r = warp; r < m; r += kGemvWarps) {
                float total = 0.0f;
                for (int i = lane; i < norm.partials_in; i += 32)
                    total += __ldcg(norm.sumsq_in + (size_t)r * norm.sumsq_in_stride + i);
                total = warp_sum(total);
                if (lane == 0) row_scale[r] = 1.0f / sqrtf(total / (float)norm.width + norm.eps);
            }
        }
#pragma unroll
        for (int u = 0; u < kGemvUnroll; ++u) {
            const int s = s0 + u * kGemvWarps;
            if (s < slices) {
#pragma unroll
                for (int j = 0; j < MT; ++j) {
#pragma unroll
                    for (int t = 0; t < WT; ++t) {
                        mma_bf16_16816(acc[t][j], a_lo[u][t].x, a_hi[u][t].x, a_lo[u][t].y, a_hi[u][t].y, b[u][j].x,
                                       b[u][j].y);
                        mma_bf16_16816(acc[t][j], a_lo[u][t].z, a_hi[u][t].z, a_lo[u][t].w, a_hi[u][t].w, b[u][j].z,
                                       b[u][j].w);
                    }
                }
            }
        }
    }
    if (!waited) {
        chain_wait();
        fetch_early();
        if (norm.sumsq_in) {
            for (int r = warp; r < m; r += kGemvWarps) {
                float total = 0.0f;
                for (int i = lane; i < norm.partials_in; i += 32)
                    total += __ldcg(norm.sumsq_in + (size_t)r * norm.sumsq_in_stride + i);
                total = warp_sum(total);
                if (lane == 0) row_scale[r] = 1.0f / sqrtf(total / (float)norm.width + norm.eps);
            }
        }
    }
    if (ahead.bytes > 0 && threadIdx.x == 0) {
        // the blocks that run last ask for it: what they ask for is on its way while the grid drains
        const int askers = min((int)gridDim.x, 148);
        const int rank = (int)blockIdx.x - ((int)gridDim.x - askers);
        if (rank >= 0) {
            const long long slice = ((ahead.bytes + askers - 1) / askers + 127) & ~127LL;
            const long long begin = (long long)rank * slice;
            if (begin < ahead.bytes) {
                const unsigned size = (unsigned)min(slice, ahead.bytes - begin);
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(ahead.ptr + begin), "r"(size) : "memory");
            }
        }
    }
    // tail of K (k % 32 in {8, 16, 24}): 8-element groups beyond the last full slice, zero-filled
    const int tail = k - slices * 32;
    if (tail > 0 && warp == (slices % kGemvWarps)) {
        const bool have = c * 8 < tail;
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int j = 0; j < MT; ++j) {
            const uint4 b = have ? ld_activation(x_row[j] + slices * 32) : zero;
#pragma unroll
            for (int t = 0; t < WT; ++t) {
                const uint4 lo = have ? ldg_stream(w_lo[t] + slices * 32) : zero;
                const uint4 hi = have ? ldg_stream(w_hi[t] + slices * 32) : zero;
                mma_bf16_16816(acc[t][j], lo.x, hi.x, lo.y, hi.y, b.x, b.y);
                mma_bf16_16816(acc[t][j], lo.z, hi.z, lo.w, hi.w, b.z, b.w);
            }
        }
    }

#pragma unroll
    for (int t = 0; t < WT; ++t)
#pragma unroll
        for (int j = 0; j < MT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) partial[warp][t][j][lane][e] = acc[t][j][e];
    __syncthreads();

    // 16 x (8*MT) outputs per weight tile; thread `i` sums the 8 warps' partials of one element
    for (int i = threadIdx.x; i < MT * 128; i += kGemvThreads) {
        const int j = i / 128, ln = (i % 128) / 4, e = i % 4;
        float sum[WT];
#pragma unroll
        for (int t = 0; t < WT; ++t) {
            float v = 0.0f;
#pragma unroll
            for (int wp = 0; wp < kGemvWarps; ++wp) v += partial[wp][t][j][ln][e];
            sum[t] = v;
        }
        // accumulator element e of lane ln: weight row (ln/4) + 8*(e/2), activation row 2*(ln%4) + (e%2)
        const int out_col = row0 + (ln >> 2) + ((e >> 1) << 3);
        const int out_row = j * 8 + ((ln & 3) << 1) + (e & 1);
        if (MODE == kGemvAddResidual && norm.next_w && out_row < m && out_col >= n)
            squares[out_row][out_col - row0] = 0.0f;
        if (out_row >= m || out_col >= n) continue;
        if (norm.sumsq_in) {
            const float scale = row_scale[out_row];
#pragma unroll
            for (int t = 0; t < WT; ++t) sum[t] *= scale;
        }
        if (MODE == kGemvStoreBf16) {
            reinterpret_cast<__nv_bfloat16*>(y)[(size_t)out_row * ldy + out_col] = __float2bfloat16_rn(sum[0]);
        } else if (MODE == kGemvStoreF32) {
            reinterpret_cast<float*>(y)[(size_t)out_row * ldy + out_col] = sum[0];
        } else if (MODE == kGemvAddResidual) {
            // the product as a plain product would store it (one rounding to bfloat16), added in float32
            float* dst = reinterpret_cast<float*>(y) + (size_t)out_row * ldy + out_col;
            const bool fetched = early_add && i == (int)threadIdx.x;       // (fetched while the weights streamed)
            const float updated = (fetched ? early_residual : *dst) + __bfloat162float(__float2bfloat16_rn(sum[0]));
            *dst = updated;
            if (norm.next_w) {
                const float next_w = fetched ? early_next_w : norm.next_w[out_col];
                norm.xw_out[(size_t)out_row * norm.ldxw + out_col] = __float2bfloat16_rn(updated * next_w);
                squares[out_row][out_col - row0] = updated * updated;
            }
        } else if (MODE == kGemvConv) {
            // B, C, X as a plain product would store them (one rounding each), then the span kernel's
            // arithmetic in the same order, so that both ways give the same bits
            const float bb = __bfloat162float(__float2bfloat16_rn(sum[0]));
            const float cc = __bfloat162float(__float2bfloat16_rn(sum[WT >= 3 ? 1 : 0]));
            const float xx = __bfloat162float(__float2bfloat16_rn(sum[WT - 1]));
            const float bx = bb * xx;
            const int keep = conv.taps - 1;
            float* st = conv.state + (size_t)conv.span_slot[out_row] * conv.slot_stride + out_col;   // [keep][n]
            const float* cw = conv.conv_w + (size_t)out_col * conv.taps;
            float history[kGemvMaxConvTaps];
            float acc_conv = 0.0f;
            if (early && i == (int)threadIdx.x) {
                // (same values, same order of the sum: fetched while the weights streamed)
#pragma unroll
                for (int tp = 0; tp < kGemvMaxConvTaps; ++tp) history[tp] = tp < kEarlyTaps - 1 ? early_history[tp] : 0.0f;
#pragma unroll
                for (int tp = 0; tp < kEarlyTaps - 1; ++tp)
                    if (tp < keep) acc_conv += early_kernel[tp] * early_history[tp];
                float last = 0.0f;
#pragma unroll
                for (int tp = 0; tp < kEarlyTaps; ++tp)
                    if (tp == keep) last = early_kernel[tp];
                acc_conv += last * bx;
            } else {
#pragma unroll
                for (int tp = 0; tp < kGemvMaxConvTaps; ++tp) history[tp] = tp < keep ? st[(size_t)tp * n] : 0.0f;
                for (int tp = 0; tp < keep; ++tp) acc_conv += cw[tp] * history[tp];
                acc_conv += cw[keep] * bx;
            }
            reinterpret_cast<__nv_bfloat16*>(y)[(size_t)out_row * ldy + out_col] = __float2bfloat16_rn(cc * acc_conv);
            for (int tp = 0; tp + 1 < keep; ++tp) st[(size_t)tp * n] = history[tp + 1];
            if (keep > 0) st[(size_t)(keep - 1) * n] = bx;
        } else {
            // the product with the up projection uses the gate as it would be stored: one rounding
            // each, as when the two halves are written by a plain product and read back
            const float gate = __bfloat162float(__float2bfloat16_rn(sum[0]));
            const float up = __bfloat162float(__float2bfloat16_rn(sum[WT - 1]));
            reinterpret_cast<__nv_bfloat16*>(y)[(size_t)out_row * ldy + out_col] =
                __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
        }
    }
    if (MODE == kGemvAddResidual && norm.next_w) {
        // this block's 16 columns of every row, summed in a fixed order
        __syncthreads();
        if (threadIdx.x < m) {
            float total = 0.0f;
#pragma unroll
            for (int col = 0; col < 16; ++col) total += squares[threadIdx.x][col];
            norm.sumsq_out[(size_t)threadIdx.x * norm.sumsq_out_stride + blockIdx.x] = total;
        }
    }
}

static thread_local GemvPrefetch g_gemv_ahead = {nullptr, 0};      // the caller's hint for the next product (taken at its entry)
static thread_local GemvPrefetch g_gemv_launch_ahead = {nullptr, 0};   // the hint of the product being launched

template <int MT, int WT, int MODE, int UNROLL, int WARPS>
static int launch_one(const __nv_bfloat16* x, int ldx, const __nv_bfloat16* w, int ldw, void* y, int ldy, int m,
                      int n, int k, int tile_offset, const GemvConvArgs& conv, const GemvNormArgs& norm,
                      cudaStream_t stream) {
    const size_t smem = (size_t)WARPS * WT * MT * 128 * sizeof(float);
    auto kernel = gemv_bf16_kernel<MT, WT, MODE, UNROLL, WARPS>;
    if (smem > 40 * 1024) {
        const cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) {
            set_error("gemv_bf16: %s", cudaGetErrorString(status));
            return -2;
        }
    }
    const GemvPrefetch ahead = g_gemv_launch_ahead;
    g_gemv_launch_ahead = {nullptr, 0};
    launch_chained_class(kChainGemv, kernel, (n + 15) / 16, WARPS * 32, smem, stream, x, ldx, w, ldw, y, ldy, m, n, k,
                         tile_offset, conv, norm, ahead);
    return check_launch("gemv_bf16");
}

template <int MT, int WARPS, int UNROLL>
static int launch_gemv(int mode, const __nv_bfloat16* x, int ldx, const __nv_bfloat16* w, int ldw, void* y, int ldy,
                       int m, int n, int k, const GemvConvArgs& conv, const GemvNormArgs& norm, cudaStream_t stream) {
    switch (mode) {
        case kGemvStoreBf16:
            return launch_one<MT, 1, kGemvStoreBf16, UNROLL, WARPS>(x, ldx, w, ldw, y, ldy, m, n, k, 0, conv, norm, stream);
        case kGemvStoreF32:
            return launch_one<MT, 1, kGemvStoreF32, UNROLL, WARPS>(x, ldx, w, ldw, y, ldy, m, n, k, 0, conv, norm, stream);
        case kGemvAddResidual:
            return launch_one<MT, 1, kGemvAddResidual, UNROLL, WARPS>(x, ldx, w, ldw, y, ldy, m, n, k, 0, conv, norm, stream);
        case kGemvSwiGlu:
            // n = inner width; rows [0, n) are the gate, rows [n, 2n) the up projection
            // (9 to 16 rows: half the loads in flight per warp, or the registers allow one block per SM only)
            return launch_one<MT, 2, kGemvSwiGlu, (UNROLL > 2 ? 2 : UNROLL) * (WARPS == 8 && MT == 1 ? 2 : 1), WARPS>(
                x, ldx, w, ldw, y, ldy, m, n, k, n, conv, norm, stream);
        case kGemvConv:
            // n = channels; rows [0, n) are B, [n, 2n) C, [2n, 3n) X
            return launch_one<MT, 3, kGemvConv, 2, WARPS>(x, ldx, w, ldw, y, ldy, m, n, k, n, conv, norm, stream);
    }
    set_error("gemv_bf16: unknown mode %d", mode);
    return -1;
}

static int g_gemv_warps = 0;      // 0: chosen from the shape; 8, 16 or 32: forced (for measurements)

}  // namespace celeg_b200

using namespace celeg_b200;

CELEG_API void celeg_gemv_set_warps(int warps) { g_gemv_warps = warps; }

// A hint for the next celeg_gemv_bf16* launch only: `bytes` of device memory at `ptr` (the weights that the
// product after it will read) are asked into the L2 by that launch's blocks. The memory must stay
// allocated as long as the launch, or a CUDA graph that captured it, may run.
CELEG_API int celeg_gemv_prefetch_next(const void* ptr, long long bytes) {
    CELEG_REQUIRE(bytes >= 0 && (((size_t)ptr) & 15) == 0, "gemv_bf16: a prefetch of %lld bytes at an address that is "
                  "not 16-byte aligned", bytes);
    g_gemv_ahead = {(const char*)ptr, ptr ? (bytes & ~15LL) : 0};
    return 0;
}

// mode 0: y bf16 [m, n] = x w^T; 1: y float32; 2: y float32 += x w^T; 3: w is [2n, k] (gate rows then up
// rows), y bf16 [m, n] = silu(x gate^T) * (x up^T); 4: w is [3n, k] (B, C, X rows of the short convolution),
// y bf16 [m, n] = C * conv(B*X) over the carried state, which is shifted (needs the conv arguments; row i
// of x is the only token of request i in this step).
static int gemv_checked(const void* x, int ldx, const void* w, int ldw, void* y, int ldy, int m, int n, int k, int mode,
                        const float* conv_w, int taps, float* state, long long slot_stride, const int* span_slot,
                        const GemvNormArgs& norm, cudaStream_t stream) {
    const GemvPrefetch ahead = g_gemv_ahead;          // a hint never outlives the call it was given for
    g_gemv_ahead = {nullptr, 0};
    g_gemv_launch_ahead = {nullptr, 0};
    CELEG_REQUIRE(m >= 0 && n > 0 && k > 0, "gemv_bf16: invalid sizes m=%d n=%d k=%d", m, n, k);
    CELEG_REQUIRE(m <= 16, "gemv_bf16: %d activation rows exceed 16; use the library product", m);
    CELEG_REQUIRE(k % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0,
                  "gemv_bf16: k=%d, ldx=%d and ldw=%d must be multiples of 8 (16-byte rows)", k, ldx, ldw);
    CELEG_REQUIRE(ldx >= k && ldw >= k && ldy >= n, "gemv_bf16: leading dimensions ldx=%d ldw=%d ldy=%d too small",
                  ldx, ldw, ldy);
    CELEG_REQUIRE((((size_t)x | (size_t)w) & 15) == 0, "gemv_bf16: operands must be 16-byte aligned");
    if (mode == kGemvConv)
        CELEG_REQUIRE(conv_w && state && span_slot && taps >= 1 && taps <= kGemvMaxConvTaps,
                      "gemv_bf16: the convolution epilogue needs kernel, state and slots (taps=%d, at most %d)", taps,
                      kGemvMaxConvTaps);
    if (m == 0) return 0;
    g_gemv_launch_ahead = ahead;
    const __nv_bfloat16* xp = (const __nv_bfloat16*)x;
    const __nv_bfloat16* wp = (const __nv_bfloat16*)w;
    GemvConvArgs conv = {conv_w, taps, state, slot_stride, span_slot};
    // blocks = n/16. A narrow matrix has fewer blocks than SMs; then only more warps per block put
    // enough loads in flight (each warp keeps 4 x 1 KiB of weights in flight, HBM needs some 50 KiB
    // per SM). Measured on B200 at 8 rows: 2048x8192 11.2 us with 8 warps, 8.7 us with 32; 2048x2048
    // 4.2 -> 3.7 us with 16; wider matrices are fastest with 8.
    const int blocks = (n + 15) / 16;
    const int slices = k / 32;
    int warps = g_gemv_warps;
    if (warps == 0) {
        if (blocks <= 148)
            warps = slices >= 128 ? 32 : 16;
        else
            warps = 8;
        if (mode == kGemvConv && warps > 16) warps = 16;
    }
    if (slices <= 16 && warps > 8) warps = 8;
#define CELEG_GEMV_DISPATCH(MT)                                                                                    \
    if (warps == 8) return launch_gemv<MT, 8, 4>(mode, xp, ldx, wp, ldw, y, ldy, m, n, k, conv, norm, stream);           \
    if (warps == 16) return launch_gemv<MT, 16, 4>(mode, xp, ldx, wp, ldw, y, ldy, m, n, k, conv, norm, stream);         \
    return launch_gemv<MT, 32, 2>(mode, xp, ldx, wp, ldw, y, ldy, m, n, k, conv, norm, stream);
    if (m <= 8) {
        CELEG_GEMV_DISPATCH(1)
    }
    CELEG_GEMV_DISPATCH(2)
#undef CELEG_GEMV_DISPATCH
}

CELEG_API int celeg_gemv_bf16(const void* x, int ldx, const void* w, int ldw, void* y, int ldy, int m, int n, int k,
                              int mode, const float* conv_w, int taps, float* state, long long slot_stride,
                              const int* span_slot, cudaStream_t stream) {
    const GemvNormArgs none = {nullptr, 0, 0, 0.0f, 0, nullptr, nullptr, 0, nullptr, 0};
    return gemv_checked(x, ldx, w, ldw, y, ldy, m, n, k, mode, conv_w, taps, state, slot_stride, span_slot, none, stream);
}

// The same product as one half of a split RMSNorm (see GemvNormArgs).
//   sumsq_in != null: x is residual * norm weight, not yet scaled; the sums are multiplied by
//     1 / sqrt(sum of the row's `partials_in` entries / width + eps) (any mode).
//   next_w != null (mode 2 only): beside y += product, xw_out = bf16(y * next_w) and
//     sumsq_out[row][block] = this block's share of sum(y^2) are written; the product has
//     (n + 15) / 16 blocks, so sumsq_out_stride must be at least that.
CELEG_API int celeg_gemv_bf16_split_norm(const void* x, int ldx, const void* w, int ldw, void* y, int ldy, int m, int n,
                                         int k, int mode, const float* conv_w, int taps, float* state,
                                         long long slot_stride, const int* span_slot, const float* sumsq_in,
                                         int partials_in, int sumsq_in_stride, float eps, int width,
                                         const float* next_w, void* xw_out, int ldxw, float* sumsq_out,
                                         int sumsq_out_stride, cudaStream_t stream) {
    CELEG_REQUIRE(!sumsq_in || (partials_in > 0 && sumsq_in_stride >= partials_in && eps > 0.0f && width > 0),
                  "gemv_bf16: the row scale needs partials_in=%d <= stride=%d, eps > 0 and a width", partials_in,
                  sumsq_in_stride);
    CELEG_REQUIRE(!next_w || (mode == kGemvAddResidual && xw_out && sumsq_out && ldxw >= n &&
                              sumsq_out_stride >= (n + 15) / 16),
                  "gemv_bf16: the norm that follows can be prepared in mode 2 only, with outputs of ldxw=%d >= n=%d "
                  "and a stride of at least %d sums", ldxw, n, (n + 15) / 16);
    const GemvNormArgs norm = {sumsq_in, partials_in, sumsq_in_stride, eps, width,
                               next_w, (__nv_bfloat16*)xw_out, ldxw, sumsq_out, sumsq_out_stride};
    return gemv_checked(x, ldx, w, ldw, y, ldy, m, n, k, mode, conv_w, taps, state, slot_stride, span_slot, norm, stream);
}
