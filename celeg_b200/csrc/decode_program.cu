// One persistent kernel that executes a whole decoding step (a "decode program": the list of
// operations in decode_program.cuh) for up to 16 requests of one token each, bfloat16.
//
// Why: a decoding step of few requests reads every weight once and is bound by that stream, but as
// a chain of a hundred small kernels the stream stops at every kernel boundary (drain, launch,
// ramp-up). Here one block per SM stays resident for the whole step:
//
//   * A producer warp streams the weights of the block's tiles into a ring of shared-memory stages
//     with TMA (cp.async.bulk.tensor.2d over a tensor map of each weight matrix, boxes of 16 rows x
//     256 elements = 8 KiB, completion counted by mbarriers). Weights are constants, so the producer
//     runs ahead of the consumers across operation boundaries and the HBM stream continues while the
//     blocks synchronise. (Measured before: untiled bulk copies of one row segment each complete at
//     about 14 copies per microsecond and SM whatever their size up to 2 KiB, and 16-byte cp.async
//     from four warps keeps too little in flight: both reach a third to a half of the stream.)
//   * Eight consumer warps multiply: the 16 weight rows of a tile are the M side of
//     mma.sync.m16n8k16 and the requests its N side (as in gemv_bf16.cu, fragments loaded as
//     16-byte vectors with a permuted k order), each warp takes every eighth 32-wide k slice of a
//     stage, the partial tiles meet in shared memory, and the epilogue (store, residual add,
//     SwiGLU, short convolution with carried state) is applied there.
//   * The RMSNorm in front of a product is its prologue: every block normalises the few rows of
//     the float32 residual stream into shared memory itself.
//   * Between operations the blocks meet at a grid barrier (one counter per operation in global
//     memory; the kernel is launched cooperatively so that all blocks are resident). Activations
//     that another block wrote are read past L1 (ld.cg, TMA), never through it.
//   * q/k norm + rotation + cache write and paged attention run the same device functions as the
//     stand-alone kernels, on groups of four consumer warps.
//
// Every wait (mbarrier, grid barrier, flag) is bounded by a timer; when it runs out the block sets
// the error flag, and from then on no wait of any block blocks: the kernel runs to its end with the
// same control flow (results are garbage, the host raises on the flag).
#include "decode_program.cuh"

#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "attention_decode.cuh"
#include "qk_norm_rope.cuh"

namespace celeg_b200 {

constexpr int kProgramConsumerWarps = 8;
constexpr int kProgramConsumers = kProgramConsumerWarps * 32;
constexpr int kProgramThreads = kProgramConsumers + 32;       // + the producer warp
constexpr int kProgramBoxK = 256;                              // elements of k in a TMA box (the most without swizzle)
constexpr int kProgramBoxRowBytes = kProgramBoxK * 2;
constexpr int kProgramWeightBoxBytes = 16 * kProgramBoxRowBytes;
constexpr int kProgramMaxStages = 8;
constexpr int kProgramRowPad = 64;                             // bytes added to a row of the normalised operand:
                                                               // rows 64 bytes apart modulo 128 make 16-byte
                                                               // fragment loads free of bank conflicts
constexpr int kProgramMaxConvTaps = 16;
constexpr long long kProgramWaitLimitNs = 2000000000ll;        // two seconds
constexpr int kErrProgramStage = 31, kErrProgramSlot = 32, kErrProgramGrid = 33;

struct ProgramControl {
    unsigned long long full[kProgramMaxStages];
    unsigned long long empty[kProgramMaxStages];
    volatile int abort;
    volatile int attention_done;      // attention operations this block has finished
    int pad[2];
    float row_sums[kProgramConsumerWarps][16];   // the norm: each warp's share of a row's sum of squares
};
constexpr int kProgramControlBytes = 1024;
static_assert(sizeof(ProgramControl) <= kProgramControlBytes, "control block too large");

// ------------------------------------------------------------------------------- PTX helpers
__device__ __forceinline__ unsigned smem_address(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(void* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_address(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(void* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_address(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect(void* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_address(bar)), "r"(bytes)
                 : "memory");
}
// Waits in hardware until the phase completes or about `nanoseconds` have passed: no polling
// traffic in the shared-memory pipe, which the multiplying warps need.
__device__ __forceinline__ bool mbar_try_wait_for(void* bar, unsigned parity, unsigned nanoseconds) {
    unsigned done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(smem_address(bar)), "r"(parity), "r"(nanoseconds)
        : "memory");
    return done != 0;
}
// Does not wait at all.
__device__ __forceinline__ bool mbar_test_wait(void* bar, unsigned parity) {
    unsigned done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(smem_address(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
// One box of the tensor map, its corner at element x of row y, into shared memory; the bytes of the
// whole box are counted on the mbarrier (also where the box hangs over the matrix and is filled
// with zeros). x * 2 bytes must be a multiple of 16.
__device__ __forceinline__ void tma_load_box(void* dst, const CUtensorMap* map, void* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(
            smem_address(dst)),
        "l"(map), "r"(smem_address(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ bool mbar_try_wait(void* bar, unsigned parity) {
    unsigned done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(smem_address(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
__device__ __forceinline__ long long global_timer() {
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ int load_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void add_release(int* p, int v) {
    asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int load_volatile(const int* p) {
    int v;
    asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void consumer_sync() { named_barrier(1, kProgramConsumers); }
__device__ __forceinline__ uint4 lds128(const unsigned char* p) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(smem_address(p)));
    return v;
}
__device__ __forceinline__ void mma_16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                          unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// --------------------------------------------------------------------------------- bounded waits
// After a wait has run out (here or in any block) nothing waits any more.
__device__ __forceinline__ bool give_up(ProgramControl* control, int* error_flag, long long started, int code) {
    if (load_volatile(error_flag) != 0) {
        control->abort = 1;
        return true;
    }
    if (global_timer() - started > kProgramWaitLimitNs) {
        atomicCAS(error_flag, 0, code);
        control->abort = 1;
        return true;
    }
    return false;
}

__device__ __forceinline__ void wait_mbarrier(void* bar, unsigned parity, ProgramControl* control, int* error_flag,
                                              int code) {
    if (mbar_test_wait(bar, parity)) return;
    const long long started = global_timer();
    for (;;) {
        if (mbar_try_wait_for(bar, parity, 20000u)) return;       // suspended, not spinning
        if (control->abort) return;
        if (give_up(control, error_flag, started, code)) return;
    }
}

// One thread waits until `counter` has reached `target` (all blocks have finished an operation).
__device__ __forceinline__ void wait_counter(const int* counter, int target, ProgramControl* control, int* error_flag) {
    if (load_acquire(counter) >= target) return;
    const long long started = global_timer();
    for (unsigned spins = 1;; ++spins) {
        if (load_acquire(counter) >= target) return;
        if (control->abort) return;
        if ((spins & 63u) == 0u && give_up(control, error_flag, started, kErrProgramGrid)) return;
    }
}

// All consumer threads of all blocks: what was written before is visible to every block after.
__device__ __forceinline__ void grid_barrier(int* counter, int blocks, ProgramControl* control, int* error_flag,
                                             int tid) {
    __threadfence();
    fence_proxy_async();          // TMA loads (async proxy) of other blocks read what was stored here
    consumer_sync();
    if (tid == 0) {
        add_release(counter, 1);
        wait_counter(counter, blocks, control, error_flag);
    }
    consumer_sync();
}

// ------------------------------------------------------------------------------------- producer
// The stages of a product, in the order in which both sides walk them: for each unit (16 output
// columns per tile set) of this block, for each k chunk. A stage holds wt*16 weight rows of `kc`
// elements and, when the operand comes from global memory, the operand's rows behind them.
struct StageCursor {
    int op, unit, chunk;
    int count;                  // stages before this one, over the whole program
    int attention_before;       // attention operations in front of `op`
    int slot, phase;            // count % stages and (count / stages) & 1, kept without dividing
    int chunks;                 // of the current operation
};

__device__ __forceinline__ void advance_slot(int& slot, int& phase, const int stages) {
    if (++slot == stages) {
        slot = 0;
        phase ^= 1;
    }
}

__device__ __forceinline__ int units_of(const ProgramOp& op) { return (op.n + 15) >> 4; }
__device__ __forceinline__ int chunks_of(const ProgramOp& op) { return (op.k + op.kc - 1) / op.kc; }

// Moves the cursor to the first stage at or after `cursor.op` that this block has. `with_operand`:
// only stages whose operand is copied (products that read a given x); the stages skipped are counted.
__device__ __forceinline__ void seek_stage(StageCursor& cursor, const ProgramOp* ops, int n_ops, bool with_operand,
                                           const int stages) {
    while (cursor.op < n_ops) {
        const ProgramOp& op = ops[cursor.op];
        if (op.kind == kOpGemv && units_of(op) > (int)blockIdx.x) {
            if (!with_operand || op.x_source == kXGlobal) {
                cursor.unit = blockIdx.x;
                cursor.chunk = 0;
                cursor.chunks = chunks_of(op);
                return;
            }
            const int mine = (units_of(op) - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
            cursor.count += mine * chunks_of(op);
            cursor.slot = cursor.count % stages;
            cursor.phase = (cursor.count / stages) & 1;
        }
        if (op.kind == kOpAttention) ++cursor.attention_before;
        ++cursor.op;
    }
}

__device__ __forceinline__ void next_stage(StageCursor& cursor, const ProgramOp* ops, int n_ops, bool with_operand,
                                           const int stages) {
    ++cursor.count;
    advance_slot(cursor.slot, cursor.phase, stages);
    if (++cursor.chunk < cursor.chunks) return;
    cursor.chunk = 0;
    cursor.unit += gridDim.x;
    if (cursor.unit < units_of(ops[cursor.op])) return;
    ++cursor.op;
    seek_stage(cursor, ops, n_ops, with_operand, stages);
}

// The producer warp; lane 0 issues. Weights are issued as soon as a slot is free (also for operations
// that have not begun); the operand's boxes only when every block has finished the operation before
// theirs. maps: two tensor maps per operation, of its weights and of its operand.
__device__ void program_producer(const ProgramOp* ops, const int n_ops, const ProgramLayout& layout,
                                 const CUtensorMap* maps, ProgramControl* control, unsigned char* ring,
                                 const int* barriers, int* error_flag, const int lane) {
    if (lane != 0) return;
    const int stages = layout.stages;
    const int x_box_bytes = layout.row_tiles * 8 * kProgramBoxRowBytes;
    StageCursor w = {0, 0, 0, 0, 0, 0, 0, 1}, x = {0, 0, 0, 0, 0, 0, 0, 1};
    seek_stage(w, ops, n_ops, false, stages);
    seek_stage(x, ops, n_ops, true, stages);
    int finished_ops = 0;              // operations [0, finished_ops) are complete on every block
    int issued = 0;                    // stages whose weights were issued
    long long idle_since = 0;
    unsigned idle_spins = 0;
    while (w.op < n_ops || x.op < n_ops) {
        if (control->abort) break;
        bool progress = false;
        if (w.op < n_ops && control->attention_done >= w.attention_before &&
            mbar_test_wait(&control->empty[w.slot], (unsigned)w.phase ^ 1u)) {
            const ProgramOp& op = ops[w.op];
            const int k0 = w.chunk * op.kc;
            const int boxes = (min(op.kc, op.k - k0) + kProgramBoxK - 1) / kProgramBoxK;
            const int all_boxes = op.kc / kProgramBoxK;
            unsigned char* stage = ring + (size_t)w.slot * layout.stage_bytes;
            void* bar = &control->full[w.slot];
            mbar_arrive_expect(bar, (unsigned)(boxes * (op.wt * kProgramWeightBoxBytes +
                                                        (op.x_source == kXGlobal ? x_box_bytes : 0))));
            for (int set = 0; set < op.wt; ++set)
                for (int b = 0; b < boxes; ++b)
                    tma_load_box(stage + (size_t)(set * all_boxes + b) * kProgramWeightBoxBytes, maps + 2 * w.op, bar,
                                 k0 + b * kProgramBoxK, (int)(set * op.tile_offset) + w.unit * 16);
            ++issued;
            next_stage(w, ops, n_ops, false, stages);
            progress = true;
        }
        if (x.op < n_ops && x.count < issued) {
            if (finished_ops < x.op && load_acquire(barriers + x.op - 1) >= (int)gridDim.x) {
                finished_ops = x.op;
                fence_proxy_async();
            }
            if (finished_ops >= x.op) {
                const ProgramOp& op = ops[x.op];
                const int k0 = x.chunk * op.kc;
                const int boxes = (min(op.kc, op.k - k0) + kProgramBoxK - 1) / kProgramBoxK;
                const int all_boxes = op.kc / kProgramBoxK;
                unsigned char* stage = ring + (size_t)x.slot * layout.stage_bytes +
                                       (size_t)op.wt * all_boxes * kProgramWeightBoxBytes;
                for (int b = 0; b < boxes; ++b)
                    tma_load_box(stage + (size_t)b * x_box_bytes, maps + 2 * x.op + 1, &control->full[x.slot],
                                 k0 + b * kProgramBoxK, 0);
                next_stage(x, ops, n_ops, true, stages);
                progress = true;
            }
        }
        if (progress) {
            idle_since = 0;
            idle_spins = 0;
        } else {
            __nanosleep(100);          // polling faster only crowds the shared-memory pipe of the consumers
            if (idle_since == 0) idle_since = global_timer();
            if ((++idle_spins & 63u) == 0u && give_up(control, error_flag, idle_since, kErrProgramSlot)) break;
        }
    }
    // Leave only when no copy of this block is still in flight (matters after a wait has run out;
    // otherwise the consumers have waited for every stage already). The last `stages` stages may be
    // pending, and each completes by itself unless its operand was never issued.
    if (control->abort) {
        const long long started = global_timer();
        for (int back = 0; back < stages && back < issued; ++back) {
            const int n = issued - 1 - back;
            const int slot = n % stages;
            const unsigned parity = (unsigned)((n / stages) & 1);
            while (!mbar_try_wait(&control->full[slot], parity)) {
                if (global_timer() - started > kProgramWaitLimitNs) break;
            }
        }
    }
}

// ------------------------------------------------------------------------------------ consumers
// RMSNorm of the operand rows into shared memory: row i = residual[gather ? gather[i] : i] scaled
// by the reciprocal root of its mean square and by the weight; sum, root and products in float32,
// one rounding to bfloat16. The columns are dealt to the warps in groups of 128 (32 vectors of four
// floats, one per lane), eight rows at a time: a lane's loads of all rows (16 vectors for a width of
// 2,048) and of its two weight vectors are in flight together, the warps' sums of squares meet in
// shared memory, and a row of that width is read once. (A warp per row, written first, needed the
// weights 16 vectors deep and paid their latency again and again between the stores.)
__device__ void norm_prologue(const ProgramOp& op, ProgramControl* control, unsigned char* x_s, const int tid) {
    constexpr int kHeld = 2;                       // vectors per lane and row kept in registers
    const int warp = tid >> 5, lane = tid & 31;
    const int k = op.k;
    const int vectors = k >> 2;
    const int stride = k * 2 + kProgramRowPad;
    const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int row_base = 0; row_base < op.rows; row_base += 8) {
        const int rows = min(8, op.rows - row_base);
        const float* source[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const int row = row_base + min(r, rows - 1);
            source[r] = op.residual + (size_t)(op.gather ? op.gather[row] : row) * op.ld_residual;
        }
        float4 held[8][kHeld], weight[kHeld];
#pragma unroll
        for (int u = 0; u < kHeld; ++u) {
            const int v = (u * kProgramConsumerWarps + warp) * 32 + lane;
#pragma unroll
            for (int r = 0; r < 8; ++r)
                held[r][u] = (r < rows && v < vectors) ? __ldcg(reinterpret_cast<const float4*>(source[r]) + v) : zero;
            weight[u] = v < vectors ? __ldg(reinterpret_cast<const float4*>(op.norm_weight) + v) : zero;
        }
        float sums[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            sums[r] = 0.0f;
#pragma unroll
            for (int u = 0; u < kHeld; ++u)
                sums[r] += held[r][u].x * held[r][u].x + held[r][u].y * held[r][u].y + held[r][u].z * held[r][u].z +
                           held[r][u].w * held[r][u].w;
        }
        // widths beyond 2,048: the further vectors are read here and again below
        for (int v = (kHeld * kProgramConsumerWarps + warp) * 32 + lane; v < vectors; v += kProgramConsumers) {
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                if (r < rows) {
                    const float4 a = __ldcg(reinterpret_cast<const float4*>(source[r]) + v);
                    sums[r] += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 8; ++r) sums[r] = warp_sum(sums[r]);
        if (row_base > 0) consumer_sync();         // the sums of the eight rows before have been read
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < 8; ++r) control->row_sums[warp][r] = sums[r];
        }
        consumer_sync();
        float inv[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            float total = 0.0f;
#pragma unroll
            for (int w = 0; w < kProgramConsumerWarps; ++w) total += control->row_sums[w][r];
            inv[r] = 1.0f / sqrtf(total / (float)k + op.eps);
        }
#pragma unroll
        for (int u = 0; u < kHeld; ++u) {
            const int v = (u * kProgramConsumerWarps + warp) * 32 + lane;
            if (v < vectors) {
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    if (r < rows) {
                        const float4 a = held[r][u];
                        __nv_bfloat162 packed[2];
                        packed[0] = __floats2bfloat162_rn(a.x * inv[r] * weight[u].x, a.y * inv[r] * weight[u].y);
                        packed[1] = __floats2bfloat162_rn(a.z * inv[r] * weight[u].z, a.w * inv[r] * weight[u].w);
                        *reinterpret_cast<uint2*>(x_s + (size_t)(row_base + r) * stride + (size_t)v * 8) =
                            *reinterpret_cast<const uint2*>(packed);
                    }
                }
            }
        }
        for (int v = (kHeld * kProgramConsumerWarps + warp) * 32 + lane; v < vectors; v += kProgramConsumers) {
            const float4 w = __ldg(reinterpret_cast<const float4*>(op.norm_weight) + v);
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                if (r < rows) {
                    const float4 a = __ldcg(reinterpret_cast<const float4*>(source[r]) + v);
                    __nv_bfloat162 packed[2];
                    packed[0] = __floats2bfloat162_rn(a.x * inv[r] * w.x, a.y * inv[r] * w.y);
                    packed[1] = __floats2bfloat162_rn(a.z * inv[r] * w.z, a.w * inv[r] * w.w);
                    *reinterpret_cast<uint2*>(x_s + (size_t)(row_base + r) * stride + (size_t)v * 8) =
                        *reinterpret_cast<const uint2*>(packed);
                }
            }
        }
    }
    consumer_sync();
}

// The epilogue of one unit: element (activation row, output column) with the sums of the tile sets.
template <int WT>
__device__ __forceinline__ void apply_epilogue(const ProgramOp& op, const float (&sum)[WT], const int out_row,
                                               const int out_col) {
    const int n = op.n;
    if (op.epilogue == kEpiStoreBf16) {
        reinterpret_cast<__nv_bfloat16*>(op.y)[(size_t)out_row * op.ldy + out_col] = __float2bfloat16_rn(sum[0]);
    } else if (op.epilogue == kEpiStoreF32) {
        reinterpret_cast<float*>(op.y)[(size_t)out_row * op.ldy + out_col] = sum[0] * op.out_scale;
    } else if (op.epilogue == kEpiAddResidual) {
        // the product as the stand-alone path stores it (one rounding to bfloat16), added in float32
        float* dst = reinterpret_cast<float*>(op.y) + (size_t)out_row * op.ldy + out_col;
        __stcg(dst, __ldcg(dst) + __bfloat162float(__float2bfloat16_rn(sum[0])));
    } else if (op.epilogue == kEpiConv) {
        const float bb = __bfloat162float(__float2bfloat16_rn(sum[0]));
        const float cc = __bfloat162float(__float2bfloat16_rn(sum[WT >= 3 ? 1 : 0]));
        const float xx = __bfloat162float(__float2bfloat16_rn(sum[WT - 1]));
        const float bx = bb * xx;
        const int keep = op.taps - 1;
        float* st = op.state + (size_t)op.span_slot[out_row] * op.slot_stride + out_col;      // [keep][n]
        const float* cw = op.conv_w + (size_t)out_col * op.taps;
        float history[kProgramMaxConvTaps];
#pragma unroll
        for (int tp = 0; tp < kProgramMaxConvTaps; ++tp) history[tp] = tp < keep ? st[(size_t)tp * n] : 0.0f;
        float acc_conv = 0.0f;
        for (int tp = 0; tp < keep; ++tp) acc_conv += cw[tp] * history[tp];
        acc_conv += cw[keep] * bx;
        reinterpret_cast<__nv_bfloat16*>(op.y)[(size_t)out_row * op.ldy + out_col] = __float2bfloat16_rn(cc * acc_conv);
        for (int tp = 0; tp + 1 < keep; ++tp) st[(size_t)tp * n] = history[tp + 1];
        if (keep > 0) st[(size_t)(keep - 1) * n] = bx;
    } else {
        const float gate = __bfloat162float(__float2bfloat16_rn(sum[0]));
        const float up = __bfloat162float(__float2bfloat16_rn(sum[WT - 1]));
        reinterpret_cast<__nv_bfloat16*>(op.y)[(size_t)out_row * op.ldy + out_col] =
            __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
    }
}

// All consumer warps: the units of this block of one product.
template <int MT, int WT>
__device__ void gemv_consume(const ProgramOp& op, const ProgramLayout& layout, ProgramControl* control,
                             unsigned char* ring, const unsigned char* x_s, float* partial, int& slot, int& phase,
                             int* error_flag, const int tid) {
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, c = lane & 3;
    const int units = units_of(op), chunks = chunks_of(op);
    const int kc = op.kc, k = op.k;
    const int all_boxes = kc / kProgramBoxK;
    const bool from_norm = op.x_source == kXNorm;
    // a stage: for each tile set its boxes of [16 rows][256], then the operand's boxes of [8 MT rows][256]
    const int x_box_bytes = MT * 8 * kProgramBoxRowBytes;
    const int x_stride = from_norm ? k * 2 + kProgramRowPad : kProgramBoxRowBytes;
    const int stages = layout.stages;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    // byte offsets of this lane's fragments inside a stage and inside the operand
    const int w_lane = g * kProgramBoxRowBytes + c * 16;
    const int x_lane = g * x_stride + c * 16;
    for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
        if (op.epilogue == kEpiConv && tid < MT * 128) {
            // the carried state of this thread's element will be wanted in the epilogue: bring it to L2 now
            const int ln = (tid % 128) / 4, e = tid % 4;
            const int out_col = unit * 16 + (ln >> 2) + ((e >> 1) << 3);
            const int out_row = (tid / 128) * 8 + ((ln & 3) << 1) + (e & 1);
            if (out_row < op.rows && out_col < op.n) {
                const float* st = op.state + (size_t)op.span_slot[out_row] * op.slot_stride + out_col;
                for (int tp = 0; tp + 1 < op.taps; ++tp)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(st + (size_t)tp * op.n));
            }
        }
        // two sets of accumulators, for the even and the odd of a warp's slices: half as long a chain
        // of dependent MMAs
        float acc[2][WT][MT][4];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int t = 0; t < WT; ++t)
#pragma unroll
                for (int j = 0; j < MT; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[h][t][j][e] = 0.0f;
        for (int chunk = 0; chunk < chunks; ++chunk) {
            const unsigned parity = (unsigned)phase;
            wait_mbarrier(&control->full[slot], parity, control, error_flag, kErrProgramStage);
            const unsigned char* stage = ring + (size_t)slot * layout.stage_bytes;
            const int k0 = chunk * kc;
            const int len = min(kc, k - k0);
            const unsigned char* w_base = stage + w_lane;
            const unsigned char* x_base =
                (from_norm ? x_s + (size_t)k0 * 2 : stage + (size_t)WT * all_boxes * kProgramWeightBoxBytes) + x_lane;
            const int slices = (len + 31) >> 5;
            for (int s0 = warp; s0 < slices; s0 += 2 * kProgramConsumerWarps) {
                uint4 lo[2][WT], hi[2][WT], b[2][MT];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    // always load (from slice 0 when there is nothing to load: a valid place), then
                    // clear: a load under a condition costs a branch each
                    const int s = s0 + h * kProgramConsumerWarps;
                    const bool inside = s < slices && s * 32 + c * 8 < len;
                    const int s_safe = inside ? s : 0;
                    // slice s lies in box s / 8 at byte (s % 8) * 64 of the box's rows
                    const int w_offset = (s_safe >> 3) * kProgramWeightBoxBytes + (s_safe & 7) * 64;
                    const int x_offset = from_norm ? s_safe * 64 : (s_safe >> 3) * x_box_bytes + (s_safe & 7) * 64;
#pragma unroll
                    for (int t = 0; t < WT; ++t) {
                        const unsigned char* set_base = w_base + t * all_boxes * kProgramWeightBoxBytes + w_offset;
                        lo[h][t] = lds128(set_base);
                        hi[h][t] = lds128(set_base + 8 * kProgramBoxRowBytes);
                        if (!inside) lo[h][t] = hi[h][t] = zero;
                    }
#pragma unroll
                    for (int j = 0; j < MT; ++j) {
                        b[h][j] = lds128(x_base + j * 8 * x_stride + x_offset);
                        if (!inside) b[h][j] = zero;
                    }
                }
#pragma unroll
                for (int j = 0; j < MT; ++j) {
#pragma unroll
                    for (int t = 0; t < WT; ++t) {
#pragma unroll
                        for (int h = 0; h < 2; ++h)
                            mma_16816(acc[h][t][j], lo[h][t].x, hi[h][t].x, lo[h][t].y, hi[h][t].y, b[h][j].x, b[h][j].y);
#pragma unroll
                        for (int h = 0; h < 2; ++h)
                            mma_16816(acc[h][t][j], lo[h][t].z, hi[h][t].z, lo[h][t].w, hi[h][t].w, b[h][j].z, b[h][j].w);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&control->empty[slot]);
            advance_slot(slot, phase, stages);
        }
        consumer_sync();                 // the epilogue of the unit before has read its partial tiles
#pragma unroll
        for (int t = 0; t < WT; ++t)
#pragma unroll
            for (int j = 0; j < MT; ++j)
                *reinterpret_cast<float4*>(partial + ((((size_t)warp * WT + t) * MT + j) * 32 + lane) * 4) =
                    make_float4(acc[0][t][j][0] + acc[1][t][j][0], acc[0][t][j][1] + acc[1][t][j][1],
                                acc[0][t][j][2] + acc[1][t][j][2], acc[0][t][j][3] + acc[1][t][j][3]);
        consumer_sync();
        for (int i = tid; i < MT * 128; i += kProgramConsumers) {
            const int j = i / 128, ln = (i % 128) / 4, e = i % 4;
            float sum[WT];
#pragma unroll
            for (int t = 0; t < WT; ++t) {
                float v = 0.0f;
#pragma unroll
                for (int wp = 0; wp < kProgramConsumerWarps; ++wp)
                    v += partial[((((size_t)wp * WT + t) * MT + j) * 32 + ln) * 4 + e];
                sum[t] = v;
            }
            // accumulator element e of lane ln: weight row (ln/4) + 8*(e/2), activation row 2*(ln%4) + (e%2)
            const int out_col = unit * 16 + (ln >> 2) + ((e >> 1) << 3);
            const int out_row = j * 8 + ((ln & 3) << 1) + (e & 1);
            if (out_row < op.rows && out_col < op.n) apply_epilogue<WT>(op, sum, out_row, out_col);
        }
    }
}

__device__ void embed_consume(const ProgramOp& op, const int tid) {
    // eight elements per thread; n (the width) is a multiple of 8
    const int vectors = op.n >> 3;
    const __nv_bfloat16* table = reinterpret_cast<const __nv_bfloat16*>(op.w);
    float* out = reinterpret_cast<float*>(op.y);
    for (long long i = (long long)blockIdx.x * kProgramConsumers + tid; i < (long long)op.rows * vectors;
         i += (long long)gridDim.x * kProgramConsumers) {
        const int row = (int)(i / vectors), col = (int)(i % vectors) * 8;
        const int token = op.token_ids[row];
        float values[8];
        if (token < 0 || token >= op.vocab) {            // the host refuses such ids before launch
#pragma unroll
            for (int e = 0; e < 8; ++e) values[e] = 0.0f;
        } else {
            const uint4 raw = __ldg(reinterpret_cast<const uint4*>(table + (size_t)token * op.ldw + col));
            bf16x8_to_float(raw, values);
#pragma unroll
            for (int e = 0; e < 8; ++e) values[e] *= op.multiplier;
        }
        float* dst = out + (size_t)row * op.ldy + col;
        __stcg(reinterpret_cast<float4*>(dst), make_float4(values[0], values[1], values[2], values[3]));
        __stcg(reinterpret_cast<float4*>(dst + 4), make_float4(values[4], values[5], values[6], values[7]));
    }
}

__device__ void qk_consume(const ProgramOp& op, int* error_flag, const int tid) {
    const QkNormRopeArgs args = {op.q_weight, op.k_weight, op.inv_freq, op.positions, op.token_span, op.block_table,
                                 op.table_stride, op.page_stride, op.rows, op.q_heads, op.kv_heads, op.head_dim,
                                 op.rotary_dim, op.page_tokens, op.eps, op.store_kv, error_flag};
    const long long units = (long long)op.rows * (op.q_heads + 2 * op.kv_heads);
    __nv_bfloat16* qkv = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(op.x));
    for (long long unit = (long long)blockIdx.x * kProgramConsumerWarps + (tid >> 5); unit < units;
         unit += (long long)gridDim.x * kProgramConsumerWarps)
        qk_norm_rope_unit<__nv_bfloat16>(qkv, reinterpret_cast<__nv_bfloat16*>(op.k_cache),
                                         reinterpret_cast<__nv_bfloat16*>(op.v_cache), args, unit, tid & 31);
}

struct GroupSync {
    int id;
    __device__ __forceinline__ void operator()() const { named_barrier(id, kDecodeThreads); }
};

template <int D_PAD, int BN>
__device__ void attention_consume(const ProgramOp& op, const ProgramLayout& layout, unsigned char* arena,
                                  int* error_flag, const int tid) {
    const int group = tid / kDecodeThreads;                 // four warps serve one item at a time
    if (group >= layout.attention_groups) return;
    DecodeParams p;
    p.q = reinterpret_cast<const __nv_bfloat16*>(op.x);
    p.q_row_stride = op.q_row_stride;
    p.out = reinterpret_cast<__nv_bfloat16*>(op.y);
    p.k_cache = reinterpret_cast<const __nv_bfloat16*>(op.k_cache);
    p.v_cache = reinterpret_cast<const __nv_bfloat16*>(op.v_cache);
    p.page_stride = op.page_stride;
    p.positions = op.positions;
    p.token_span = op.token_span;
    p.block_table = op.block_table;
    p.table_stride = op.table_stride;
    p.q_heads = op.q_heads;
    p.kv_heads = op.kv_heads;
    p.head_dim = op.head_dim;
    p.page_tokens = op.page_tokens;
    p.window = op.window;
    p.chunk = op.chunk;
    p.max_splits = op.max_splits;
    p.scale = op.scale;
    p.partial_o = op.partial_o;
    p.partial_ml = op.partial_ml;
    p.counters = op.counters;
    p.error_flag = error_flag;
    p.fuse_qk = 0;                 // the program has an operation of its own for the q/k post-processing
    p.q_norm_w = p.k_norm_w = p.inv_freq = nullptr;
    p.rotary_dim = 0;
    p.norm_eps = 0.0f;
    p.k_cache_w = p.v_cache_w = nullptr;
    const GroupSync sync = {2 + group};
    unsigned char* mine = arena + (size_t)group * layout.attention_item_bytes;
    const long long items = (long long)op.rows * op.kv_heads * op.max_splits;
    for (long long item = (long long)blockIdx.x * layout.attention_groups + group; item < items;
         item += (long long)gridDim.x * layout.attention_groups) {
        const int split = (int)(item % op.max_splits);
        const int kvh = (int)((item / op.max_splits) % op.kv_heads);
        const int t = (int)(item / ((long long)op.max_splits * op.kv_heads));
        sync();                          // the item before is done with the shared memory
        attention_decode_item<D_PAD, BN>(p, split, kvh, t, mine, tid % kDecodeThreads, sync);
    }
}

// --------------------------------------------------------------------------------------- kernel
// barriers: [n_ops + 1] ints, zero before the first launch; entry i counts the blocks that have
// finished operation i, the last entry the blocks that have finished the program. The block that
// finishes last clears them all, so that every launch leaves them zero.
template <int MT>
__global__ void __launch_bounds__(kProgramThreads, 1)
decode_program_kernel(const ProgramOp* __restrict__ ops, const int n_ops, const ProgramLayout layout,
                      const CUtensorMap* __restrict__ maps, int* barriers, int* error_flag, long long* timeline) {
    extern __shared__ __align__(128) unsigned char smem[];
    ProgramControl* control = reinterpret_cast<ProgramControl*>(smem);
    unsigned char* arena = smem + kProgramControlBytes;
    unsigned char* x_s = arena;
    float* partial = reinterpret_cast<float*>(arena + layout.x_bytes);
    unsigned char* ring = arena + layout.x_bytes + layout.partial_bytes;
    const int tid = threadIdx.x;
    if (tid == 0) {
        for (int s = 0; s < kProgramMaxStages; ++s) {
            mbar_init(&control->full[s], 1);
            mbar_init(&control->empty[s], kProgramConsumerWarps);
        }
        control->abort = 0;
        control->attention_done = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (tid >= kProgramConsumers) {
        program_producer(ops, n_ops, layout, maps, control, ring, barriers, error_flag, tid & 31);
        return;
    }

    int slot = 0, phase = 0;
    int attention_done = 0;
    if (timeline && blockIdx.x == 0 && tid == 0) timeline[0] = global_timer();
    for (int i = 0; i < n_ops; ++i) {
        const ProgramOp& op = ops[i];
        if (op.kind == kOpEmbed) {
            embed_consume(op, tid);
        } else if (op.kind == kOpGemv) {
            if (units_of(op) > (int)blockIdx.x) {
                if (op.x_source == kXNorm) norm_prologue(op, control, x_s, tid);
                if (op.wt == 1)
                    gemv_consume<MT, 1>(op, layout, control, ring, x_s, partial, slot, phase, error_flag, tid);
                else if (op.wt == 2)
                    gemv_consume<MT, 2>(op, layout, control, ring, x_s, partial, slot, phase, error_flag, tid);
                else
                    gemv_consume<MT, 3>(op, layout, control, ring, x_s, partial, slot, phase, error_flag, tid);
            }
        } else if (op.kind == kOpQkNormRope) {
            qk_consume(op, error_flag, tid);
        } else {
            // the shared memory of the items overlays everything behind the control block: nothing of a
            // product is live now, and the producer holds back the weights of later products
            if (op.head_dim <= 64)
                attention_consume<64, 64>(op, layout, arena, error_flag, tid);
            else if (op.head_dim <= 128)
                attention_consume<128, 64>(op, layout, arena, error_flag, tid);
            else
                attention_consume<256, 32>(op, layout, arena, error_flag, tid);
            fence_proxy_async();         // TMA will overwrite what ordinary stores wrote here
            consumer_sync();
            if (tid == 0) control->attention_done = ++attention_done;
        }
        // diagnostics: when block 0 finished its share of operation i, and when every block had
        if (timeline && blockIdx.x == 0 && tid == 0) timeline[1 + 2 * i] = global_timer();
        if (i + 1 < n_ops) grid_barrier(barriers + i, gridDim.x, control, error_flag, tid);
        if (timeline && blockIdx.x == 0 && tid == 0) timeline[2 + 2 * i] = global_timer();
    }
    consumer_sync();
    if (tid == 0) {
        __threadfence();
        const int finished = atomicAdd(barriers + n_ops, 1);
        if (finished == (int)gridDim.x - 1) {
            for (int i = 0; i <= n_ops; ++i) barriers[i] = 0;
            __threadfence();
        }
    }
}

static int g_program_sms = 0;
static int g_program_smem = 0;

static int program_device_limits() {
    if (g_program_sms > 0) return 0;
    int device = 0;
    cudaError_t status = cudaGetDevice(&device);
    if (status == cudaSuccess) status = cudaDeviceGetAttribute(&g_program_sms, cudaDevAttrMultiProcessorCount, device);
    if (status == cudaSuccess)
        status = cudaDeviceGetAttribute(&g_program_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    if (status != cudaSuccess) {
        set_error("decode_program: cannot read the device's limits: %s", cudaGetErrorString(status));
        g_program_sms = 0;
        return -2;
    }
    return 0;
}

static size_t attention_item_bytes_for(int head_dim) {
    if (head_dim <= 64) return decode_item_bytes<64, 64>();
    if (head_dim <= 128) return decode_item_bytes<128, 64>();
    return decode_item_bytes<256, 32>();
}

}  // namespace celeg_b200

using namespace celeg_b200;

CELEG_API int celeg_decode_program_op_bytes() { return (int)sizeof(ProgramOp); }
CELEG_API int celeg_decode_program_layout_bytes() { return (int)sizeof(ProgramLayout); }

// Checks the operations (host copies), chooses the k chunk of every product (written into the
// operations) and the shared-memory layout. `sms` and `smem_limit` may be 0 (= ask the current
// device); tests without a device pass them. Returns 0, or -1 with the reason in celeg_last_error()
// when the program cannot run as one kernel (the caller then runs the operations as separate kernels).
CELEG_API int celeg_decode_program_prepare(void* ops_raw, int n_ops, void* layout_raw, int sms, int smem_limit) {
    ProgramOp* ops = reinterpret_cast<ProgramOp*>(ops_raw);
    ProgramLayout* layout = reinterpret_cast<ProgramLayout*>(layout_raw);
    CELEG_REQUIRE(ops && layout && n_ops > 0, "decode_program: no operations");
    if (sms <= 0 || smem_limit <= 0) {
        if (program_device_limits() != 0) return -2;
        sms = g_program_sms;
        smem_limit = g_program_smem;
    }
    int rows = 0, x_bytes = 0, max_wt = 1;
    size_t attention_bytes = 0;
    for (int i = 0; i < n_ops; ++i) {
        const ProgramOp& op = ops[i];
        CELEG_REQUIRE(op.rows > 0 && op.rows <= 16, "decode_program: operation %d has %d rows (1 to 16)", i, op.rows);
        rows = op.rows > rows ? op.rows : rows;
    }
    const int mt = rows <= 8 ? 1 : 2;
    for (int i = 0; i < n_ops; ++i) {
        const ProgramOp& op = ops[i];
        if (op.kind == kOpEmbed) {
            CELEG_REQUIRE(op.w && op.y && op.token_ids && op.n > 0 && op.n % 8 == 0 && op.ldw % 8 == 0 && op.ldy % 4 == 0 &&
                              op.vocab > 0 && (((size_t)op.w | (size_t)op.y) & 15) == 0,
                          "decode_program: embedding %d needs a width that is a multiple of 8 and aligned tables", i);
        } else if (op.kind == kOpGemv) {
            CELEG_REQUIRE(op.w && op.y && op.n > 0 && op.k > 0 && op.k % 8 == 0 && op.ldw % 8 == 0 && op.ldw >= op.k &&
                              ((size_t)op.w & 15) == 0,
                          "decode_program: product %d needs k=%d and ldw=%d to be multiples of 8 and aligned weights",
                          i, op.k, op.ldw);
            CELEG_REQUIRE(op.wt >= 1 && op.wt <= 3 && op.epilogue >= kEpiStoreBf16 && op.epilogue <= kEpiConv,
                          "decode_program: product %d has an unknown shape (wt=%d epilogue=%d)", i, op.wt, op.epilogue);
            CELEG_REQUIRE((op.epilogue == kEpiSwiGlu) == (op.wt == 2) && (op.epilogue == kEpiConv) == (op.wt == 3),
                          "decode_program: product %d: %d tile sets do not fit epilogue %d", i, op.wt, op.epilogue);
            CELEG_REQUIRE(op.ldy >= op.n, "decode_program: product %d: ldy=%d is less than n=%d", i, op.ldy, op.n);
            if (op.x_source == kXNorm) {
                CELEG_REQUIRE(op.residual && op.norm_weight && op.eps > 0.0f && op.ld_residual % 4 == 0 &&
                                  op.ld_residual >= op.k &&
                                  (((size_t)op.residual | (size_t)op.norm_weight) & 15) == 0,
                              "decode_program: product %d: the norm in front needs aligned float32 rows", i);
                const int bytes = mt * 8 * (op.k * 2 + kProgramRowPad);
                x_bytes = bytes > x_bytes ? bytes : x_bytes;
            } else {
                CELEG_REQUIRE(op.x_source == kXGlobal && op.x && op.ldx % 8 == 0 && op.ldx >= op.k &&
                                  ((size_t)op.x & 15) == 0 && op.x_rows >= op.rows,
                              "decode_program: product %d: the operand needs ldx=%d to be a multiple of 8 and "
                              "aligned rows", i, op.ldx);
            }
            if (op.epilogue == kEpiConv)
                CELEG_REQUIRE(op.conv_w && op.state && op.span_slot && op.taps >= 1 && op.taps <= kProgramMaxConvTaps,
                              "decode_program: product %d: the convolution needs kernel, state and slots (taps=%d, "
                              "at most %d)", i, op.taps, kProgramMaxConvTaps);
            max_wt = op.wt > max_wt ? op.wt : max_wt;
        } else if (op.kind == kOpQkNormRope) {
            CELEG_REQUIRE(op.x && op.positions && op.token_span && op.q_heads > 0 && op.kv_heads >= 0 &&
                              op.head_dim > 0 && op.head_dim <= kMaxHeadDim && op.page_tokens > 0 &&
                              op.rotary_dim >= 0 && op.rotary_dim <= op.head_dim && op.rotary_dim % 2 == 0,
                          "decode_program: q/k operation %d has invalid sizes", i);
            CELEG_REQUIRE(!op.store_kv || (op.block_table && op.k_cache && op.v_cache),
                          "decode_program: q/k operation %d stores without a cache", i);
        } else if (op.kind == kOpAttention) {
            CELEG_REQUIRE(op.x && op.y && op.k_cache && op.v_cache && op.positions && op.token_span && op.block_table &&
                              op.partial_o && op.partial_ml && op.counters,
                          "decode_program: attention %d lacks a buffer", i);
            CELEG_REQUIRE(op.q_heads > 0 && op.kv_heads > 0 && op.q_heads % op.kv_heads == 0 &&
                              op.q_heads / op.kv_heads <= kMaxGroup && op.head_dim % 8 == 0 && op.head_dim > 0 &&
                              op.head_dim <= kMaxDecodeHeadDim && op.q_row_stride % 8 == 0 && op.chunk > 0 &&
                              op.max_splits > 0 && op.page_tokens > 0,
                          "decode_program: attention %d has sizes the decode kernel does not take", i);
            const size_t bytes = attention_item_bytes_for(op.head_dim);
            attention_bytes = bytes > attention_bytes ? bytes : attention_bytes;
        } else {
            CELEG_REQUIRE(false, "decode_program: operation %d has unknown kind %d", i, op.kind);
        }
    }
    const int partial_bytes = kProgramConsumerWarps * max_wt * mt * 128 * (int)sizeof(float);
    const int arena = smem_limit - kProgramControlBytes;
    x_bytes = (x_bytes + 127) / 128 * 128;
    const int ring_bytes = (arena - x_bytes - partial_bytes) / 128 * 128;
    // A stage holds, per 256 elements of k, a box of 16 rows for each tile set and one of the operand's
    // rows when it is copied. Stages of 36 KiB keep five of them in flight beside the operand of a
    // model 2,048 wide; fewer, smaller ones when the operand is wide.
    int stage_bytes = 36 * 1024;
    int stages = ring_bytes / stage_bytes;
    if (stages < 3) {
        stages = 3;
        stage_bytes = ring_bytes / 3 / 1024 * 1024;
    }
    if (stages > kProgramMaxStages) stages = kProgramMaxStages;
    CELEG_REQUIRE(ring_bytes > 0 && stage_bytes >= 8 * 1024,
                  "decode_program: %d bytes of shared memory leave no room for weight stages beside a %d-byte "
                  "operand", smem_limit, x_bytes);
    for (int i = 0; i < n_ops; ++i) {
        ProgramOp& op = ops[i];
        if (op.kind != kOpGemv) continue;
        const int per_box = op.wt * kProgramWeightBoxBytes + (op.x_source == kXGlobal ? mt * 8 * kProgramBoxRowBytes : 0);
        int boxes = stage_bytes / per_box;
        const int k_boxes = (op.k + kProgramBoxK - 1) / kProgramBoxK;
        boxes = boxes < k_boxes ? boxes : k_boxes;
        CELEG_REQUIRE(boxes >= 1, "decode_program: product %d does not fit a stage of %d bytes", i, stage_bytes);
        const int chunks = (k_boxes + boxes - 1) / boxes;
        boxes = (k_boxes + chunks - 1) / chunks;                     // chunks of even length
        op.kc = boxes * kProgramBoxK;
    }
    int groups = 0;
    if (attention_bytes > 0) {
        groups = (int)((size_t)arena / attention_bytes);
        groups = groups > 2 ? 2 : groups;
        CELEG_REQUIRE(groups >= 1, "decode_program: attention needs %zu bytes of shared memory, %d are there",
                      attention_bytes, arena);
    }
    layout->row_tiles = mt;
    layout->stages = stages;
    layout->stage_bytes = stage_bytes;
    layout->x_bytes = x_bytes;
    layout->partial_bytes = partial_bytes;
    layout->attention_groups = groups;
    layout->attention_item_bytes = (int)((attention_bytes + 127) / 128 * 128);
    layout->smem_bytes = kProgramControlBytes + x_bytes + partial_bytes + stages * stage_bytes;
    const int attention_total = kProgramControlBytes + groups * layout->attention_item_bytes;
    if (attention_total > layout->smem_bytes) layout->smem_bytes = attention_total;
    CELEG_REQUIRE(layout->smem_bytes <= smem_limit, "decode_program: layout of %d bytes exceeds %d", layout->smem_bytes,
                  smem_limit);
    layout->grid = sms;
    layout->reserved[0] = layout->reserved[1] = layout->reserved[2] = 0;
    return 0;
}

// Writes the tensor maps of a prepared program into `maps_raw` (host memory, 2 * n_ops maps of 128
// bytes: for operation i its weights at 2 i and its copied operand at 2 i + 1; the others stay zero).
// Needs the driver (a device), unlike celeg_decode_program_prepare. The caller copies them to the device.
CELEG_API int celeg_decode_program_encode_maps(const void* ops_raw, int n_ops, const void* layout_raw, void* maps_raw) {
    const ProgramOp* ops = reinterpret_cast<const ProgramOp*>(ops_raw);
    const ProgramLayout& layout = *reinterpret_cast<const ProgramLayout*>(layout_raw);
    CUtensorMap* maps = reinterpret_cast<CUtensorMap*>(maps_raw);
    static_assert(sizeof(CUtensorMap) == 128, "a tensor map has 128 bytes");
    CELEG_REQUIRE(ops && maps && n_ops > 0, "decode_program: missing arguments");
    typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                      const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                      CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeTiledFn encode = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess)
            encode = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    CELEG_REQUIRE(encode != nullptr, "decode_program: cuTensorMapEncodeTiled is not available from this driver");
    memset(maps, 0, sizeof(CUtensorMap) * 2 * (size_t)n_ops);
    for (int i = 0; i < n_ops; ++i) {
        const ProgramOp& op = ops[i];
        if (op.kind != kOpGemv) continue;
        for (int which = 0; which < 2; ++which) {
            if (which == 1 && op.x_source != kXGlobal) continue;
            // [rows, k] bfloat16, `ld` elements between rows, read in boxes of box_rows x 256, not swizzled;
            // what hangs over the matrix reads as zero
            const void* base = which == 0 ? op.w : op.x;
            const long long rows = which == 0 ? (long long)(op.wt - 1) * op.tile_offset + op.n : op.x_rows;
            const long long ld = which == 0 ? op.ldw : op.ldx;
            const int box_rows = which == 0 ? 16 : layout.row_tiles * 8;
            const cuuint64_t dims[2] = {(cuuint64_t)op.k, (cuuint64_t)rows};
            const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
            const cuuint32_t box[2] = {(cuuint32_t)kProgramBoxK, (cuuint32_t)box_rows};
            const cuuint32_t element_strides[2] = {1, 1};
            const CUresult status =
                encode(&maps[2 * i + which], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                       box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            CELEG_REQUIRE(status == CUDA_SUCCESS,
                          "decode_program: cuTensorMapEncodeTiled failed with code %d for operation %d (rows=%lld "
                          "k=%d ld=%lld)", (int)status, i, rows, op.k, ld);
        }
    }
    return 0;
}

// ops: device copy of the prepared operations; maps: device copy of their tensor maps. barriers:
// [n_ops + 1] ints, zero before the first launch (each launch leaves them zero; clear them after an
// error). timeline: null, or [1 + 2 n_ops] device words that receive nanosecond time stamps of block 0
// (start; for each operation: its own share done, all blocks done), for measurements. One cooperative launch.
CELEG_API int celeg_decode_program_run(const void* ops, int n_ops, const void* layout_raw, const void* maps,
                                       int* barriers, int* error_flag, long long* timeline, cudaStream_t stream) {
    const ProgramLayout layout = *reinterpret_cast<const ProgramLayout*>(layout_raw);
    CELEG_REQUIRE(ops && maps && barriers && error_flag && n_ops > 0, "decode_program: missing arguments");
    CELEG_REQUIRE(((size_t)maps & 63) == 0, "decode_program: tensor maps must be 64-byte aligned");
    CELEG_REQUIRE(layout.stages >= 2 && layout.stages <= kProgramMaxStages && layout.grid > 0 &&
                      (layout.row_tiles == 1 || layout.row_tiles == 2),
                  "decode_program: the layout was not prepared");
    auto kernel = layout.row_tiles == 1 ? decode_program_kernel<1> : decode_program_kernel<2>;
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, layout.smem_bytes);
    if (status != cudaSuccess) {
        set_error("decode_program: %s", cudaGetErrorString(status));
        return -2;
    }
    int resident = 0;
    status = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kernel, kProgramThreads, layout.smem_bytes);
    if (status != cudaSuccess || resident < 1) {
        set_error("decode_program: the kernel does not fit an SM (%s)",
                  status == cudaSuccess ? "no resident block" : cudaGetErrorString(status));
        return -2;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(layout.grid);
    config.blockDim = dim3(kProgramThreads);
    config.dynamicSmemBytes = layout.smem_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeCooperative;      // all blocks resident at once, or the launch fails
    attribute[0].val.cooperative = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    const ProgramOp* ops_typed = reinterpret_cast<const ProgramOp*>(ops);
    const CUtensorMap* maps_typed = reinterpret_cast<const CUtensorMap*>(maps);
    status = cudaLaunchKernelEx(&config, kernel, ops_typed, n_ops, layout, maps_typed, barriers, error_flag, timeline);
    if (status != cudaSuccess) {
        set_error("decode_program: launch failed: %s", cudaGetErrorString(status));
        return -2;
    }
    return check_launch("decode_program");
}
