// Products of 17 to 64 rows of activations (decode steps of many requests, small prompt portions):
//
//     Y[T, N] = epilogue(X[T, K] * W[N, K]^T)        bfloat16 operands, float32 accumulation
//
// With so few rows the product is bound by reading W once, as the small-batch product is
// (gemv_bf16.cu), but the tensor cores that suit it are the fifth-generation ones:
//
//   * The weights are the M side: a block owns 128 weight rows of each of its 1 to 3 tile sets
//     (1: plain; 2: gate rows and their up rows; 3: the B, C and X rows of the short convolution), the
//     T rows of activations are the N side (padded to a multiple of 32), and the accumulators
//     [128 x T] of the sets lie side by side in tensor memory. TMA brings a [128 x 64] box per set and a
//     [T x 64] box of X per k-tile into a ring of stages (128-byte swizzle); one thread issues
//     tcgen05.mma (M = 128, N = T, K = 16), tcgen05.commit frees the stage.
//   * A matrix of 2,048 rows has only 16 such tiles, far too few blocks to pull the whole HBM
//     bandwidth. The k range is therefore split over the 1, 2, 4 or 8 blocks of a thread-block
//     cluster: each block multiplies its k slice and stores rows [128 r / S, 128 (r+1) / S) of its
//     partial [128 x T] tile into the shared memory of block r of the cluster (st.shared::cluster, one
//     slot per sender, no waiting); after one cluster barrier block r adds up its S slots in a fixed
//     order and runs the epilogue on its rows. No atomics, no second kernel, the same result every run.
//   * Epilogues as in the small-batch product: store (bfloat16 or float32), add to the float32
//     residual stream, SwiGLU, and the short convolution's gate with carried state (one token per
//     request).
//
// Every wait on an mbarrier is bounded (tcgen05.cuh); a block that gives up records an error code and
// still takes part in the cluster barriers, which have no time limit of their own.
//
// Measured on a B200 at 64 rows (weights cold, CUDA-graph chains over rotating copies): 2048 x 8192 19.7 us
// with four splits (the library product 13.3), 2048 x 2048 10.9 us (5.7), gate|up 8192 x 2048 with SwiGLU
// 27.8 us (15.9 with its activation kernel), 65536 x 2048 94 us (56). A block's k loop runs at the speed of
// the stream once it is going, but with 128 weight rows a block a matrix of 2,048 rows is 16 tiles: four
// splits use 64 SMs, eight splits need clusters of eight, of which the GPU does not hold sixteen at once
// (24 us); set-up, the cluster barrier and the epilogue are not overlapped with anything, and wide
// matrices come in three and a half waves. Until tiles of 64 rows and a persistent form with a
// double-buffered accumulator change that, the engine keeps the library product for these row counts and
// runs this kernel only when asked to (CELEG_B200_TC_PRODUCTS=stream).
//
// celeg hands these products to cuBLAS (src/backend/cuda/runtime/gemm_dispatcher.cpp:49-64) and runs
// the activation, the convolution and the residual add as kernels of their own.
#include "tcgen05.cuh"

namespace celeg_b200 {

constexpr int kStreamThreads = 128;
constexpr int kStreamMaxRows = 64;
constexpr int kStreamMaxStages = 6;
constexpr int kStreamMaxConvTaps = 16;
constexpr unsigned kStreamWeightTileBytes = kTileM * kTileK * 2;

enum StreamMode : int { kStreamStoreBf16 = 0, kStreamStoreF32 = 1, kStreamAddResidual = 2, kStreamSwiGlu = 3, kStreamConv = 4 };

struct StreamParams {
    int rows;                 // T
    int t_pad;                // T rounded up to a multiple of 32
    int n;                    // columns of Y = weight rows per tile set
    int k;
    int splits;               // blocks of a cluster, along k
    int k_tiles_per_split;
    int mode;
    void* y;
    int ldy;
    const float* conv_w;      // mode 4: [n, taps]
    int taps;
    float* state;
    long long slot_stride;
    const int* span_slot;
    int* error_flag;
};

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

// The address that `local` (a shared-memory address of this block) has in block `rank` of the cluster.
__device__ __forceinline__ unsigned cluster_address(unsigned local, unsigned rank) {
    unsigned remote;
    asm("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}
__device__ __forceinline__ void store_cluster_shared(unsigned remote, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(remote), "f"(v) : "memory");
}

// MODE is a template parameter: the code of one epilogue is small, and a block runs it once, cold;
// with all five behind run-time branches the loop was bound by instruction fetch (about 800 cycles per
// four outputs of a thread, whatever it loaded or stored).
template <int WT, int MODE>
__device__ __forceinline__ void stream_epilogue(const StreamParams& p, const float (&sum)[WT], const float residual,
                                                const int token, const int column) {
    if (MODE == kStreamStoreBf16) {
        reinterpret_cast<__nv_bfloat16*>(p.y)[(size_t)token * p.ldy + column] = __float2bfloat16_rn(sum[0]);
    } else if (MODE == kStreamStoreF32) {
        reinterpret_cast<float*>(p.y)[(size_t)token * p.ldy + column] = sum[0];
    } else if (MODE == kStreamAddResidual) {
        // the product as a plain product would store it (one rounding to bfloat16), added in float32
        // (`residual` is the value read before, together with those of the thread's other tokens)
        reinterpret_cast<float*>(p.y)[(size_t)token * p.ldy + column] =
            residual + __bfloat162float(__float2bfloat16_rn(sum[0]));
    } else if (MODE == kStreamSwiGlu) {
        const float gate = __bfloat162float(__float2bfloat16_rn(sum[0]));
        const float up = __bfloat162float(__float2bfloat16_rn(sum[WT - 1]));
        reinterpret_cast<__nv_bfloat16*>(p.y)[(size_t)token * p.ldy + column] =
            __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
    } else {
        // B, C, X as a plain product would store them, then the arithmetic of the span kernel
        const float bb = __bfloat162float(__float2bfloat16_rn(sum[0]));
        const float cc = __bfloat162float(__float2bfloat16_rn(sum[WT >= 3 ? 1 : 0]));
        const float xx = __bfloat162float(__float2bfloat16_rn(sum[WT - 1]));
        const float bx = bb * xx;
        const int keep = p.taps - 1;
        float* st = p.state + (size_t)p.span_slot[token] * p.slot_stride + column;      // [keep][n]
        const float* cw = p.conv_w + (size_t)column * p.taps;
        // one pass over the carried taps: each is used and moved one place down
        float acc = 0.0f;
        float older = keep > 0 ? st[0] : 0.0f;
#pragma unroll 1
        for (int tp = 0; tp < keep; ++tp) {
            acc += cw[tp] * older;
            const float newer = tp + 1 < keep ? st[(size_t)(tp + 1) * p.n] : bx;
            st[(size_t)tp * p.n] = newer;
            older = newer;
        }
        acc += cw[keep] * bx;
        reinterpret_cast<__nv_bfloat16*>(p.y)[(size_t)token * p.ldy + column] = __float2bfloat16_rn(cc * acc);
    }
}

// grid = (tiles of 128 weight rows, 1, splits), cluster = (1, 1, splits)
template <int WT, int MODE>
__global__ void __launch_bounds__(kStreamThreads)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const StreamParams p, const int STAGES) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long full_bar[kStreamMaxStages], empty_bar[kStreamMaxStages], accum_bar;
    __shared__ unsigned tmem_base_slot;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int n0 = blockIdx.x * kTileM;
    const int rank = blockIdx.z;                                   // = rank in the cluster (1, 1, splits)
    const int k_tiles = (p.k + kTileK - 1) / kTileK;
    const int kt_begin = rank * p.k_tiles_per_split;
    const int kt_end = min(k_tiles, kt_begin + p.k_tiles_per_split);
    const int my_tiles = max(0, kt_end - kt_begin);
    const unsigned bytes_x = (unsigned)p.t_pad * kTileK * 2;
    const unsigned stage_bytes = WT * kStreamWeightTileBytes + bytes_x;
    unsigned tmem_columns = 32;
    while (tmem_columns < (unsigned)(WT * p.t_pad)) tmem_columns <<= 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        mbar_init(smem_u32(&accum_bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) tmem_alloc(smem_u32(&tmem_base_slot), tmem_columns);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const unsigned tmem_base = tmem_base_slot;
    int error = 0;

    if (warp == 0 && lane == 0) {
        for (int i = 0; i < my_tiles && !error; ++i) {
            const int s = i % STAGES;
            if (i >= STAGES && !mbar_wait(smem_u32(&empty_bar[s]), ((i / STAGES) - 1) & 1)) {
                error = 41;
                break;
            }
            const unsigned bar = smem_u32(&full_bar[s]);
            mbar_expect_tx(bar, stage_bytes);
            const unsigned dst = smem_base + s * stage_bytes;
            const int k0 = (kt_begin + i) * kTileK;
#pragma unroll
            for (int t = 0; t < WT; ++t) tma_load_2d(dst + t * kStreamWeightTileBytes, &map_w, bar, k0, t * p.n + n0);
            tma_load_2d(dst + WT * kStreamWeightTileBytes, &map_x, bar, k0, 0);
        }
    } else if (warp == 1 && lane == 0) {
        const unsigned idesc = instruction_descriptor(kTileM, p.t_pad);
        for (int i = 0; i < my_tiles && !error; ++i) {
            const int s = i % STAGES;
            if (!mbar_wait(smem_u32(&full_bar[s]), (i / STAGES) & 1)) {
                error = 42;
                break;
            }
            tcgen05_fence_after();
            const unsigned w_addr = smem_base + s * stage_bytes;
            const unsigned long long desc_x = smem_descriptor(w_addr + WT * kStreamWeightTileBytes);
#pragma unroll
            for (int kk = 0; kk < kTileK / kUmmaK; ++kk) {
#pragma unroll
                for (int t = 0; t < WT; ++t)
                    umma_bf16(tmem_base + (unsigned)(t * p.t_pad), smem_descriptor(w_addr + t * kStreamWeightTileBytes) + 2 * kk,
                              desc_x + 2 * kk, idesc, (i > 0 || kk > 0) ? 1u : 0u);
            }
            umma_commit(smem_u32(&empty_bar[s]));
        }
        if (!error && my_tiles > 0) umma_commit(smem_u32(&accum_bar));
    }
    if (error) atomicExch(p.error_flag, error);

    // Slots behind the ring, one per sender: [sender][set][token][row of mine] float32. A thread reads its
    // row of the accumulators from tensor memory and stores it into the slot of this block in the block
    // that owns the row; the stores are not waited for.
    __syncwarp();
    bool have = true;
    if (my_tiles > 0) {
        have = mbar_wait(smem_u32(&accum_bar), 0);
        have = __all_sync(0xffffffffu, have);
        if (!have && lane == 0) atomicExch(p.error_flag, 43);
    }
    tcgen05_fence_after();
    const int rows_here = kTileM / p.splits;
    const unsigned slots_addr = smem_base + (unsigned)STAGES * stage_bytes;
    const int row = warp * 32 + lane;
    if (have) {
        const unsigned owner_base = cluster_address(slots_addr, (unsigned)(row / rows_here));
        const int mine = row % rows_here;
#pragma unroll 1
        for (int t = 0; t < WT; ++t) {
#pragma unroll 1
            for (int c0 = 0; c0 < p.t_pad; c0 += 32) {
                float v[32];
                if (my_tiles > 0) {
                    tmem_load_32(tmem_base + ((unsigned)(warp * 32) << 16) + (unsigned)(t * p.t_pad + c0), v);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0.0f;
                }
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    store_cluster_shared(owner_base + (unsigned)(((((rank * WT + t) * p.t_pad) + c0 + i) * rows_here + mine) * 4),
                                         v[i]);
            }
        }
    } else if (warp == 0 && lane == 0) {
        // giving up: copies that were issued must land before the shared memory goes away
        for (int s = 0; s < STAGES && s < my_tiles; ++s) mbar_wait(smem_u32(&full_bar[s]), 0);
    }
    // every block's stores are done and visible when all have passed this barrier; after it a block only
    // reads its own shared memory, so it may leave whenever it is done
    if (p.splits > 1)
        cluster_sync_all();
    else
        __syncthreads();

    // this block's rows: the S slots summed in the order of the ranks, then the epilogue. A thread keeps
    // its row and walks over the tokens, four at a time, the residual's loads in flight together.
    const float* slots = reinterpret_cast<const float*>(smem_raw + (slots_addr - smem_u32(smem_raw)));
    const int local = threadIdx.x % rows_here;
    const int token_step = kStreamThreads / rows_here;
    const int column = n0 + rank * rows_here + local;
    constexpr int kBatch = 4;
    if (column < p.n) {
        for (int first = threadIdx.x / rows_here; first < p.rows; first += kBatch * token_step) {
            float sum[kBatch][WT];
            float residual[kBatch];
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
                const int token = first + b * token_step;
                residual[b] = 0.0f;
#pragma unroll
                for (int t = 0; t < WT; ++t) sum[b][t] = 0.0f;
                if (token < p.rows) {
                    if (MODE == kStreamAddResidual)
                        residual[b] = __ldcg(reinterpret_cast<const float*>(p.y) + (size_t)token * p.ldy + column);
#pragma unroll
                    for (int t = 0; t < WT; ++t) {
                        for (int source = 0; source < p.splits; ++source)
                            sum[b][t] += slots[(size_t)(((source * WT + t) * p.t_pad) + token) * rows_here + local];
                    }
                }
            }
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
                const int token = first + b * token_step;
                if (token < p.rows) stream_epilogue<WT, MODE>(p, sum[b], residual[b], token, column);
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, tmem_columns);
}

template <int WT, int MODE>
static int launch_stream(const CUtensorMap& map_w, const CUtensorMap& map_x, const StreamParams& p, int tiles,
                         cudaStream_t stream) {
    const size_t stage = WT * kStreamWeightTileBytes + (size_t)p.t_pad * kTileK * 2;
    const size_t slots = (size_t)WT * p.t_pad * kTileM * sizeof(float);
    static int smem_limit = 0;
    if (smem_limit == 0) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&smem_limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess)
            smem_limit = 200 * 1024;
    }
    int stages = (int)(((size_t)smem_limit - 2048 - slots) / stage);
    if (stages > kStreamMaxStages) stages = kStreamMaxStages;
    if (stages < 2) {
        set_error("gemm_stream: %d rows of %d tile sets leave no room for two stages beside the partial tiles", p.rows, WT);
        return -1;
    }
    const size_t smem = (size_t)stages * stage + slots + 1024;
    auto kernel = gemm_stream_kernel<WT, MODE>;
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (status != cudaSuccess) {
        set_error("gemm_stream: %s (shared memory %zu bytes)", cudaGetErrorString(status), smem);
        return -2;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(tiles, 1, p.splits);
    config.blockDim = dim3(kStreamThreads);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = 1;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = p.splits;
    config.attrs = attribute;
    config.numAttrs = 1;
    status = cudaLaunchKernelEx(&config, kernel, map_w, map_x, p, stages);
    if (status != cudaSuccess) {
        set_error("gemm_stream: launch failed: %s", cudaGetErrorString(status));
        return -2;
    }
    return check_launch("gemm_stream");
}

static int g_stream_splits = 0;       // 0: chosen from the shape; 1, 2, 4 or 8: forced (for measurements)

}  // namespace celeg_b200

using namespace celeg_b200;

CELEG_API void celeg_gemm_stream_set_splits(int splits) { g_stream_splits = splits; }

// mode 0: y bf16 [rows, n] = x w^T; 1: y float32; 2: y float32 += x w^T (rounded to bf16 first);
// 3: w is [2n, k] (gate rows then up rows), y bf16 = silu(x gate^T) * (x up^T); 4: w is [3n, k] (B, C, X
// rows of the short convolution), y bf16 = C * conv(B*X) over the carried state, which is shifted (row i
// of x is the only token of request i in this step). 1 <= rows <= 64; x must have x_rows >= rows rows
// that may be read; k, ldx and ldw multiples of 8; x and w 16-byte aligned.
CELEG_API int celeg_gemm_stream(const void* x, int ldx, int x_rows, const void* w, int ldw, void* y, int ldy, int rows,
                                int n, int k, int mode, const float* conv_w, int taps, float* state,
                                long long slot_stride, const int* span_slot, int* error_flag, cudaStream_t stream) {
    CELEG_REQUIRE(rows >= 0 && rows <= kStreamMaxRows && n > 0 && k > 0, "gemm_stream: invalid sizes rows=%d n=%d k=%d "
                  "(at most %d rows)", rows, n, k, kStreamMaxRows);
    CELEG_REQUIRE(k % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ldx >= k && ldw >= k && ldy >= n && x_rows >= rows,
                  "gemm_stream: k=%d, ldx=%d, ldw=%d must be multiples of 8 and cover the operands (ldy=%d, x_rows=%d)",
                  k, ldx, ldw, ldy, x_rows);
    CELEG_REQUIRE((((size_t)x | (size_t)w) & 15) == 0 && error_flag, "gemm_stream: operands must be 16-byte aligned");
    CELEG_REQUIRE(mode >= kStreamStoreBf16 && mode <= kStreamConv, "gemm_stream: unknown mode %d", mode);
    if (mode == kStreamConv)
        CELEG_REQUIRE(conv_w && state && span_slot && taps >= 1 && taps <= kStreamMaxConvTaps,
                      "gemm_stream: the convolution epilogue needs kernel, state and slots (taps=%d, at most %d)", taps,
                      kStreamMaxConvTaps);
    if (rows == 0) return 0;
    const int sets = mode == kStreamSwiGlu ? 2 : mode == kStreamConv ? 3 : 1;
    StreamParams p;
    p.rows = rows;
    p.t_pad = (rows + 31) / 32 * 32;
    p.n = n;
    p.k = k;
    p.mode = mode;
    p.y = y;
    p.ldy = ldy;
    p.conv_w = conv_w;
    p.taps = taps;
    p.state = state;
    p.slot_stride = slot_stride;
    p.span_slot = span_slot;
    p.error_flag = error_flag;
    const int tiles = (n + kTileM - 1) / kTileM;
    const int k_tiles = (k + kTileK - 1) / kTileK;
    // enough blocks to pull the whole bandwidth (about one per SM), no more splits than k-tiles
    int splits = g_stream_splits;
    if (splits == 0) {
        splits = 1;
        while (splits < 8 && tiles * splits < 96 && splits * 2 <= k_tiles) splits *= 2;
    }
    CELEG_REQUIRE(splits == 1 || splits == 2 || splits == 4 || splits == 8, "gemm_stream: %d splits", splits);
    while (splits > 1 && splits > k_tiles) splits /= 2;
    p.splits = splits;
    p.k_tiles_per_split = (k_tiles + splits - 1) / splits;
    CUtensorMap map_w, map_x;
    if (!tensor_map_for(w, (long long)sets * n, k, ldw, kTileM, &map_w)) return -2;
    if (!tensor_map_for(x, x_rows, k, ldx, p.t_pad, &map_x)) return -2;
    switch (mode) {
        case kStreamStoreBf16: return launch_stream<1, kStreamStoreBf16>(map_w, map_x, p, tiles, stream);
        case kStreamStoreF32: return launch_stream<1, kStreamStoreF32>(map_w, map_x, p, tiles, stream);
        case kStreamAddResidual: return launch_stream<1, kStreamAddResidual>(map_w, map_x, p, tiles, stream);
        case kStreamSwiGlu: return launch_stream<2, kStreamSwiGlu>(map_w, map_x, p, tiles, stream);
        default: return launch_stream<3, kStreamConv>(map_w, map_x, p, tiles, stream);
    }
}
