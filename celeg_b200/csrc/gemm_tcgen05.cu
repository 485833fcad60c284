// bfloat16 matrix product on Blackwell's fifth-generation tensor cores:
//
//     C[M,N] = A[M,K] * B[N,K]^T      (both operands row-major with K contiguous, float32 accumulation)
//
// One block computes a 128 x BN tile. Operand tiles of 64 k-elements (128 bytes per row) are brought
// into shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle) into a ring of stages guarded by
// mbarriers; one elected thread issues tcgen05.mma (M = 128, N = BN, K = 16) reading both operands
// from shared memory through matrix descriptors, with the accumulator in tensor memory (TMEM);
// tcgen05.commit hands a stage back to the producer when the MMAs that read it have finished. After
// the last k-tile the four warps read the accumulator with tcgen05.ld (each warp its 32 lanes) and run
// the epilogue: store bfloat16 or float32, or SwiGLU (the B tile then holds BN/2 gate rows and their
// BN/2 up rows, the output is silu(gate) * up).
//
// Every wait on an mbarrier is bounded: after kMaxPolls unsuccessful polls the thread records an error
// code, stops taking part, and the block leaves through the common exit (pending copies are awaited
// with the same bound, tensor memory is released). The host reads the flag.
//
// celeg calls cuBLAS / cuBLASLt for these products (src/backend/cuda/runtime/gemm_dispatcher.cpp:49-64,
// 171-190) and runs SwiGLU as a separate kernel (src/backend/cuda/kernels/qkv_rope.cuh:24-39).
#include "tcgen05.cuh"

#include <cstdlib>
#include <mutex>
#include <unordered_map>

namespace celeg_b200 {

constexpr int kGemmThreads = 128;

enum TcEpilogue : int { kTcStoreBf16 = 0, kTcStoreF32 = 1, kTcSwiGlu = 2 };

struct TcGemmParams {
    int m, n, k;           // n: columns of C (for SwiGLU: the inner width, B has 2n rows)
    void* c;
    int ldc;
    int* error_flag;
};

template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(kGemmThreads)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const TcGemmParams p) {
    constexpr unsigned kBytesA = kTileM * kTileK * 2;
    constexpr unsigned kBytesB = BN * kTileK * 2;
    constexpr unsigned kTmemColumns = BN < 32 ? 32 : BN;            // power of two >= 32
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], accum_bar;
    __shared__ unsigned tmem_base_slot;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // shared-memory base rounded up to the 1024 bytes the swizzle pattern needs
    const unsigned smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int m0 = blockIdx.y * kTileM;
    const int n0 = blockIdx.x * (EPI == kTcSwiGlu ? BN / 2 : BN);
    const int k_tiles = (p.k + kTileK - 1) / kTileK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        mbar_init(smem_u32(&accum_bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) tmem_alloc(smem_u32(&tmem_base_slot), kTmemColumns);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const unsigned tmem_base = tmem_base_slot;
    int error = 0;

    if (warp == 0 && lane == 0) {
        // producer: TMA loads of the A and B tiles of every k-tile
        for (int kt = 0; kt < k_tiles && !error; ++kt) {
            const int s = kt % STAGES;
            if (kt >= STAGES && !mbar_wait(smem_u32(&empty_bar[s]), ((kt / STAGES) - 1) & 1)) {
                error = 11;
                break;
            }
            const unsigned bar = smem_u32(&full_bar[s]);
            mbar_expect_tx(bar, kBytesA + kBytesB);
            const unsigned a_dst = smem_base + s * (kBytesA + kBytesB);
            const unsigned b_dst = a_dst + kBytesA;
            tma_load_2d(a_dst, &map_a, bar, kt * kTileK, m0);
            if (EPI == kTcSwiGlu) {
                tma_load_2d(b_dst, &map_b, bar, kt * kTileK, n0);                      // gate rows
                tma_load_2d(b_dst + kBytesB / 2, &map_b, bar, kt * kTileK, p.n + n0);  // their up rows
            } else {
                tma_load_2d(b_dst, &map_b, bar, kt * kTileK, n0);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // MMA issuer
        constexpr unsigned idesc = instruction_descriptor(kTileM, BN);
        for (int kt = 0; kt < k_tiles && !error; ++kt) {
            const int s = kt % STAGES;
            if (!mbar_wait(smem_u32(&full_bar[s]), (kt / STAGES) & 1)) {
                error = 12;
                break;
            }
            tcgen05_fence_after();
            const unsigned a_addr = smem_base + s * (kBytesA + kBytesB);
            const unsigned long long desc_a = smem_descriptor(a_addr);
            const unsigned long long desc_b = smem_descriptor(a_addr + kBytesA);
#pragma unroll
            for (int kk = 0; kk < kTileK / kUmmaK; ++kk) {
                // 16 k-elements further inside the 128-byte swizzle row: 32 bytes, 2 in descriptor units
                umma_bf16(tmem_base, desc_a + 2 * kk, desc_b + 2 * kk, idesc, (kt > 0 || kk > 0) ? 1u : 0u);
            }
            umma_commit(smem_u32(&empty_bar[s]));          // the stage is free when these MMAs are done
        }
        if (!error) umma_commit(smem_u32(&accum_bar));      // the accumulator is complete
    }
    if (error) atomicExch(p.error_flag, error);

    // epilogue: every warp reads its 32 lanes of the accumulator
    __syncwarp();
    bool have_accumulator = mbar_wait(smem_u32(&accum_bar), 0);
    have_accumulator = __all_sync(0xffffffffu, have_accumulator);   // tcgen05.ld needs the whole warp
    if (!have_accumulator && lane == 0) atomicExch(p.error_flag, 13);
    tcgen05_fence_after();
    if (have_accumulator) {
        const int row = m0 + warp * 32 + lane;
        constexpr int kOutColumns = EPI == kTcSwiGlu ? BN / 2 : BN;
#pragma unroll 1
        for (int c0 = 0; c0 < kOutColumns; c0 += 32) {
            float v[32];
            tmem_load_32(tmem_base + ((unsigned)(warp * 32) << 16) + (unsigned)c0, v);
            if (EPI == kTcSwiGlu) {
                float u[32];
                tmem_load_32(tmem_base + ((unsigned)(warp * 32) << 16) + (unsigned)(BN / 2 + c0), u);
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    // gate and up as a plain product would store them (one rounding each)
                    const float g = __bfloat162float(__float2bfloat16_rn(v[i]));
                    const float up = __bfloat162float(__float2bfloat16_rn(u[i]));
                    v[i] = g / (1.0f + expf(-g)) * up;
                }
            }
            if (row < p.m) {
                const int col = n0 + c0;
                if (EPI == kTcStoreF32) {
                    float* dst = reinterpret_cast<float*>(p.c) + (size_t)row * p.ldc + col;
                    if (col + 32 <= p.n && (p.ldc & 3) == 0) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                    } else {
                        for (int i = 0; i < 32; ++i)
                            if (col + i < p.n) dst[i] = v[i];
                    }
                } else {
                    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.c) + (size_t)row * p.ldc + col;
                    if (col + 32 <= p.n && (p.ldc & 7) == 0) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 packed;
                            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
                            h[0] = __floats2bfloat162_rn(v[i], v[i + 1]);
                            h[1] = __floats2bfloat162_rn(v[i + 2], v[i + 3]);
                            h[2] = __floats2bfloat162_rn(v[i + 4], v[i + 5]);
                            h[3] = __floats2bfloat162_rn(v[i + 6], v[i + 7]);
                            *reinterpret_cast<uint4*>(dst + i) = packed;
                        }
                    } else {
                        for (int i = 0; i < 32; ++i)
                            if (col + i < p.n) dst[i] = __float2bfloat16_rn(v[i]);
                    }
                }
            }
        }
    } else if (warp == 0 && lane == 0) {
        // leaving early: copies that were issued must land before the shared memory goes away
        for (int s = 0; s < STAGES; ++s) {
            if (s < k_tiles) mbar_wait(smem_u32(&full_bar[s]), 0);
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, kTmemColumns);
}

// ---------------------------------------------------------------------------------- persistent
// The same product as a persistent kernel: one block per SM walks over output tiles of 128 x 256.
// Six warps: warp 0 feeds the ring with TMA, warp 1 issues the MMAs, warps 2-5 are the epilogue. The
// 512 columns of tensor memory hold TWO accumulators, so the MMAs of the next tile run while the
// epilogue warps drain the previous one (tcgen05.ld -> registers -> global). Tiles that run at the same
// time share their B tile (consecutive tile numbers walk down M), which keeps the weights in L2.
constexpr int kPersistentThreads = 192;
constexpr int kPersistentBN = 256;
constexpr int kPersistentStages = 4;

__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}

template <int EPI>
__global__ void __launch_bounds__(kPersistentThreads)
gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                               const TcGemmParams p) {
    constexpr int BN = kPersistentBN, STAGES = kPersistentStages;
    constexpr unsigned kBytesA = kTileM * kTileK * 2;
    constexpr unsigned kBytesB = BN * kTileK * 2;
    constexpr int kOutColumns = EPI == kTcSwiGlu ? BN / 2 : BN;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], accum_full[2], accum_empty[2];
    __shared__ unsigned tmem_base_slot;
    __shared__ volatile int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int k_tiles = (p.k + kTileK - 1) / kTileK;
    const int m_tiles = (p.m + kTileM - 1) / kTileM;
    const int n_tiles = (p.n + kOutColumns - 1) / kOutColumns;
    const int tiles = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&accum_full[b]), 1);
            mbar_init(smem_u32(&accum_empty[b]), 4);       // one arrival per epilogue warp
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) tmem_alloc(smem_u32(&tmem_base_slot), 512);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const unsigned tmem_base = tmem_base_slot;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;                                     // k-tiles issued so far, over all tiles
            for (int tile = blockIdx.x; tile < tiles && !abort_flag; tile += gridDim.x) {
                const int m0 = (tile % m_tiles) * kTileM;
                const int n0 = (tile / m_tiles) * kOutColumns;
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(smem_u32(&empty_bar[s]), ((it / STAGES) - 1) & 1)) {
                        atomicExch(p.error_flag, 21);
                        abort_flag = 1;
                        break;
                    }
                    const unsigned bar = smem_u32(&full_bar[s]);
                    mbar_expect_tx(bar, kBytesA + kBytesB);
                    const unsigned a_dst = smem_base + s * (kBytesA + kBytesB);
                    const unsigned b_dst = a_dst + kBytesA;
                    tma_load_2d(a_dst, &map_a, bar, kt * kTileK, m0);
                    if (EPI == kTcSwiGlu) {
                        tma_load_2d(b_dst, &map_b, bar, kt * kTileK, n0);
                        tma_load_2d(b_dst + kBytesB / 2, &map_b, bar, kt * kTileK, p.n + n0);
                    } else {
                        tma_load_2d(b_dst, &map_b, bar, kt * kTileK, n0);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr unsigned idesc = instruction_descriptor(kTileM, BN);
            int it = 0, local = 0;
            for (int tile = blockIdx.x; tile < tiles && !abort_flag; tile += gridDim.x, ++local) {
                const int buf = local & 1;
                if (local >= 2 && !mbar_wait(smem_u32(&accum_empty[buf]), ((local >> 1) - 1) & 1)) {
                    atomicExch(p.error_flag, 22);
                    abort_flag = 1;
                    break;
                }
                tcgen05_fence_after();
                const unsigned tmem_d = tmem_base + (unsigned)(buf * BN);
                bool ok = true;
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(smem_u32(&full_bar[s]), (it / STAGES) & 1)) {
                        atomicExch(p.error_flag, 23);
                        abort_flag = 1;
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const unsigned a_addr = smem_base + s * (kBytesA + kBytesB);
                    const unsigned long long desc_a = smem_descriptor(a_addr);
                    const unsigned long long desc_b = smem_descriptor(a_addr + kBytesA);
#pragma unroll
                    for (int kk = 0; kk < kTileK / kUmmaK; ++kk)
                        umma_bf16(tmem_d, desc_a + 2 * kk, desc_b + 2 * kk, idesc, (kt > 0 || kk > 0) ? 1u : 0u);
                    umma_commit(smem_u32(&empty_bar[s]));
                }
                if (!ok) break;
                umma_commit(smem_u32(&accum_full[buf]));
            }
        }
    } else {
        // epilogue warps 2..5; a warp may only touch the 32 TMEM lanes of its position modulo 4
        const int quarter = warp & 3;
        int local = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
            const int buf = local & 1;
            bool ready = abort_flag == 0 && mbar_wait(smem_u32(&accum_full[buf]), (local >> 1) & 1);
            ready = __all_sync(0xffffffffu, ready);
            if (!ready) {
                if (lane == 0 && abort_flag == 0) {
                    atomicExch(p.error_flag, 24);
                    abort_flag = 1;
                }
                break;
            }
            tcgen05_fence_after();
            const int m0 = (tile % m_tiles) * kTileM;
            const int n0 = (tile / m_tiles) * kOutColumns;
            const int row = m0 + quarter * 32 + lane;
            const unsigned lane_base = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(buf * BN);
#pragma unroll 1
            for (int c0 = 0; c0 < kOutColumns; c0 += 32) {
                float v[32];
                tmem_load_32(lane_base + (unsigned)c0, v);
                if (EPI == kTcSwiGlu) {
                    float u[32];
                    tmem_load_32(lane_base + (unsigned)(BN / 2 + c0), u);
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const float g = __bfloat162float(__float2bfloat16_rn(v[i]));
                        const float up = __bfloat162float(__float2bfloat16_rn(u[i]));
                        v[i] = g / (1.0f + expf(-g)) * up;
                    }
                }
                if (row < p.m) {
                    const int col = n0 + c0;
                    if (EPI == kTcStoreF32) {
                        float* dst = reinterpret_cast<float*>(p.c) + (size_t)row * p.ldc + col;
                        if (col + 32 <= p.n && (p.ldc & 3) == 0) {
#pragma unroll
                            for (int i = 0; i < 32; i += 4)
                                *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                        } else {
                            for (int i = 0; i < 32; ++i)
                                if (col + i < p.n) dst[i] = v[i];
                        }
                    } else {
                        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.c) + (size_t)row * p.ldc + col;
                        if (col + 32 <= p.n && (p.ldc & 7) == 0) {
#pragma unroll
                            for (int i = 0; i < 32; i += 8) {
                                uint4 packed;
                                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
                                h[0] = __floats2bfloat162_rn(v[i], v[i + 1]);
                                h[1] = __floats2bfloat162_rn(v[i + 2], v[i + 3]);
                                h[2] = __floats2bfloat162_rn(v[i + 4], v[i + 5]);
                                h[3] = __floats2bfloat162_rn(v[i + 6], v[i + 7]);
                                *reinterpret_cast<uint4*>(dst + i) = packed;
                            }
                        } else {
                            for (int i = 0; i < 32; ++i)
                                if (col + i < p.n) dst[i] = __float2bfloat16_rn(v[i]);
                        }
                    }
                }
            }
            // this warp is done reading the accumulator: the MMA warp may overwrite it
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&accum_empty[buf]));
        }
    }
    if (abort_flag && warp == 0 && lane == 0) {
        // leaving early: copies that were issued must land before the shared memory goes away
        for (int s = 0; s < STAGES; ++s) mbar_wait(smem_u32(&full_bar[s]), 0);
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, 512);
}

// ------------------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

struct MapKey {
    const void* base;
    long long rows, cols, ld;
    int box_rows;
    bool operator==(const MapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = std::hash<const void*>()(k.base);
        h = h * 1000003u ^ std::hash<long long>()(k.rows * 31 + k.cols);
        return h * 1000003u ^ std::hash<long long>()(k.ld * 131 + k.box_rows);
    }
};

// A [rows, cols] bfloat16 matrix with `ld` elements between rows, read in boxes of box_rows x 64.
bool tensor_map_for(const void* base, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out) {
    static std::mutex mutex;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key{base, rows, cols, ld, box_rows};
    std::lock_guard<std::mutex> lock(mutex);
    auto found = cache.find(key);
    if (found != cache.end()) {
        *out = found->second;
        return true;
    }
    EncodeTiledFn encode = encode_tiled();
    if (!encode) {
        set_error("gemm_tcgen05: cuTensorMapEncodeTiled is not available from this driver");
        return false;
    }
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)box_rows};
    const cuuint32_t element_strides[2] = {1, 1};
    const CUresult status = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                                   box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (status != CUDA_SUCCESS) {
        set_error("gemm_tcgen05: cuTensorMapEncodeTiled failed with code %d (rows=%lld cols=%lld ld=%lld)", (int)status,
                  rows, cols, ld);
        return false;
    }
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, map);
    *out = map;
    return true;
}

template <int BN, int STAGES, int EPI>
static int launch_tc(const CUtensorMap& map_a, const CUtensorMap& map_b, const TcGemmParams& p, cudaStream_t stream) {
    constexpr size_t smem = (size_t)STAGES * (kTileM * kTileK * 2 + BN * kTileK * 2) + 1024;
    auto kernel = gemm_tcgen05_kernel<BN, STAGES, EPI>;
    const cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (status != cudaSuccess) {
        set_error("gemm_tcgen05: %s", cudaGetErrorString(status));
        return -2;
    }
    constexpr int out_columns = EPI == kTcSwiGlu ? BN / 2 : BN;
    dim3 grid((p.n + out_columns - 1) / out_columns, (p.m + kTileM - 1) / kTileM);
    kernel<<<grid, kGemmThreads, smem, stream>>>(map_a, map_b, p);
    return check_launch("gemm_tcgen05");
}

template <int EPI>
static int launch_tc_persistent(const CUtensorMap& map_a, const CUtensorMap& map_b, const TcGemmParams& p,
                                cudaStream_t stream) {
    constexpr size_t smem = (size_t)kPersistentStages * (kTileM * kTileK * 2 + kPersistentBN * kTileK * 2) + 1024;
    auto kernel = gemm_tcgen05_persistent_kernel<EPI>;
    const cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (status != cudaSuccess) {
        set_error("gemm_tcgen05: %s", cudaGetErrorString(status));
        return -2;
    }
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (sms <= 0) sms = 148;
    }
    constexpr int out_columns = EPI == kTcSwiGlu ? kPersistentBN / 2 : kPersistentBN;
    const int tiles = ((p.m + kTileM - 1) / kTileM) * ((p.n + out_columns - 1) / out_columns);
    kernel<<<tiles < sms ? tiles : sms, kPersistentThreads, smem, stream>>>(map_a, map_b, p);
    return check_launch("gemm_tcgen05 (persistent)");
}

}  // namespace celeg_b200

using namespace celeg_b200;

// c[m, n] = a[m, k] * b[n, k]^T in bfloat16 with float32 accumulation on tcgen05 tensor cores.
// epilogue 0: c bfloat16; 1: c float32; 2: b holds n gate rows then n up rows, c bfloat16 [m, n] =
// silu(a gate^T) * (a up^T). k, lda and ldb must be multiples of 8 (16-byte rows for TMA); operands
// 16-byte aligned. error_flag (device int) receives a code if a bounded wait inside the kernel ran out.
// forced_variant: -1 = the kernel is chosen from the shape, 0..3 = that one (for measurements).
CELEG_API int celeg_gemm_tcgen05(const void* a, int lda, const void* b, int ldb, void* c, int ldc, int m, int n, int k,
                                 int epilogue, int* error_flag, int forced_variant, cudaStream_t stream) {
    CELEG_REQUIRE(m > 0 && n > 0 && k > 0, "gemm_tcgen05: invalid sizes m=%d n=%d k=%d", m, n, k);
    CELEG_REQUIRE(k % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0 && lda >= k && ldb >= k,
                  "gemm_tcgen05: k=%d, lda=%d and ldb=%d must be multiples of 8 and cover k", k, lda, ldb);
    CELEG_REQUIRE((((size_t)a | (size_t)b) & 15) == 0, "gemm_tcgen05: operands must be 16-byte aligned");
    CELEG_REQUIRE(ldc >= n && error_flag != nullptr, "gemm_tcgen05: ldc=%d is smaller than n=%d, or no error flag", ldc, n);
    CELEG_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm_tcgen05: unknown epilogue %d", epilogue);
    CELEG_REQUIRE((m + kTileM - 1) / kTileM <= 65535, "gemm_tcgen05: %d rows exceed one launch", m);
    // Which kernel: many rows -> the persistent kernel (128 x 256 tiles, epilogue hidden under the next
    // tile); few rows -> 128 x 128 tiles with two blocks per SM, which gives more blocks to spread the
    // weight stream over.
    CELEG_REQUIRE(forced_variant >= -1 && forced_variant <= 3, "gemm_tcgen05: unknown variant %d", forced_variant);
    const int variant = forced_variant >= 0 ? forced_variant : (m >= 512 ? 3 : 1);
    const int bn = variant >= 2 ? 256 : 128;
    CUtensorMap map_a, map_b;
    if (!tensor_map_for(a, m, k, lda, kTileM, &map_a)) return -3;
    const long long b_rows = epilogue == kTcSwiGlu ? 2ll * n : n;
    if (!tensor_map_for(b, b_rows, k, ldb, epilogue == kTcSwiGlu ? bn / 2 : bn, &map_b)) return -3;
    TcGemmParams p{m, n, k, c, ldc, error_flag};
#define CELEG_TC_DISPATCH(BN, STAGES)                                                        \
    switch (epilogue) {                                                                      \
        case kTcStoreBf16:                                                                   \
            return launch_tc<BN, STAGES, kTcStoreBf16>(map_a, map_b, p, stream);             \
        case kTcStoreF32:                                                                    \
            return launch_tc<BN, STAGES, kTcStoreF32>(map_a, map_b, p, stream);              \
        default:                                                                             \
            return launch_tc<BN, STAGES, kTcSwiGlu>(map_a, map_b, p, stream);                \
    }
    if (variant == 3) {                // persistent, two accumulators, epilogue under the next tile's MMAs
        switch (epilogue) {
            case kTcStoreBf16:
                return launch_tc_persistent<kTcStoreBf16>(map_a, map_b, p, stream);
            case kTcStoreF32:
                return launch_tc_persistent<kTcStoreF32>(map_a, map_b, p, stream);
            default:
                return launch_tc_persistent<kTcSwiGlu>(map_a, map_b, p, stream);
        }
    }
    if (variant == 0) {
        CELEG_TC_DISPATCH(128, 6)      // one block per SM, deep ring
    }
    if (variant == 2) {
        CELEG_TC_DISPATCH(256, 4)      // wide tile, one block per SM
    }
    CELEG_TC_DISPATCH(128, 3)          // two blocks per SM: one's epilogue under the other's main loop
#undef CELEG_TC_DISPATCH
}
