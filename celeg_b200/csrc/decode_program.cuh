// The description of a decode program: the operations of one decoding step of a model, in run
// order, as plain data. The host fills one ProgramOp per operation (the parts of a model emit
// them; no operation knows which model it belongs to), celeg_decode_program_prepare() checks them
// and chooses the tiling, and one persistent kernel executes the list (decode_program.cu).
//
// celeg launches one kernel per operation and layer (src/backend/cuda/packed/layer_executor.cu:101-216);
// a program has no counterpart there.
#pragma once
#include "common.cuh"

namespace celeg_b200 {

enum ProgramOpKind : int {
    kOpEmbed = 0,         // residual[r, :] = multiplier * table[token_ids[r], :]
    kOpGemv = 1,          // y = epilogue(x W^T), x either given or the RMSNorm of the residual stream
    kOpQkNormRope = 2,    // per-head norm + rotation of q and k, k and v written to the paged cache
    kOpAttention = 3,     // paged attention of one query token per request
};

enum ProgramXSource : int { kXGlobal = 0, kXNorm = 1 };

// The epilogues of the small-batch product (same codes as celeg_gemv_bf16's modes).
enum ProgramEpilogue : int { kEpiStoreBf16 = 0, kEpiStoreF32 = 1, kEpiAddResidual = 2, kEpiSwiGlu = 3, kEpiConv = 4 };

// Every field is plain data; pointers are device pointers that stay valid while the program is
// used. The Python side mirrors this struct field by field (celeg_decode_program_op_bytes() guards
// the layout).
struct ProgramOp {
    // --- product
    const void* w;              // [wt tile sets of n rows, k] bfloat16 (embed: the table [vocab, n])
    const void* x;              // kXGlobal: [rows, k] bfloat16; q/k op and attention: the q|k|v projection
    void* y;                    // output [rows, n] (embed: the float32 residual stream)
    const float* residual;      // kXNorm: float32 [*, k], normalised row by row into the operand
    const float* norm_weight;   // kXNorm: [k]
    const int* gather;          // kXNorm: optional list of residual rows (row i of the operand = residual[gather[i]])
    const float* conv_w;        // kEpiConv: [n, taps]
    float* state;               // kEpiConv: carried taps of this layer inside slot 0
    const int* span_slot;       // kEpiConv: state slot of row i
    const int* token_ids;       // embed
    // --- q/k post-processing and attention
    const float* q_weight;
    const float* k_weight;
    const float* inv_freq;
    const int* positions;
    const int* token_span;
    const int* block_table;
    void* k_cache;
    void* v_cache;
    float* partial_o;
    float* partial_ml;
    int* counters;
    long long slot_stride;
    long long page_stride;
    long long tile_offset;      // rows between the tile sets of w (swiglu: n, conv: n)
    int kind, rows, n, k;
    int wt;                     // tile sets per unit: 1, 2 (gate, up) or 3 (B, C, X)
    int epilogue, x_source;
    int kc;                     // k elements per pipeline stage, a multiple of 256 (chosen by prepare)
    int ldw, ldx, ldy, ld_residual, taps;
    int table_stride, q_heads, kv_heads, head_dim, rotary_dim, page_tokens, window, chunk, max_splits;
    int store_kv, q_row_stride, vocab;
    int x_rows;                 // rows the copied operand's buffer has (at least `rows`)
    float eps, out_scale, scale, multiplier;
};

// Chosen by celeg_decode_program_prepare() and passed to the launch unchanged.
struct ProgramLayout {
    int row_tiles;        // MT: 1 for up to 8 rows, 2 for up to 16
    int stages;           // pipeline slots for weights
    int stage_bytes;
    int x_bytes;          // the normalised operand
    int partial_bytes;    // the warps' partial tiles
    int attention_groups; // groups of four warps that serve attention items at the same time (1 or 2)
    int attention_item_bytes;
    int smem_bytes;       // everything
    int grid;             // blocks: one per SM
    int reserved[3];
};

}  // namespace celeg_b200
