"""Decode programs: a decoding step written down as a list of operations that one persistent
kernel executes (csrc/decode_program.cu), instead of a launch per operation.

A part that can take part has a method

    emit_decode(builder, x, step)      mixers and feed-forwards; x is a NormedRows (the rows of the
                                       residual stream after the part's norm) -- the part appends its
                                       operations and ends with builder.product(..., add_to_residual=True)
    emit_decode(builder, step)         arrangements
    as_prologue()                      norms: (weight, eps) when the norm is a plain RMSNorm that a product
                                       can apply to its operand itself, else None

A part without the method (or one that raises ProgramUnsupported) makes the model run the step as
separate kernels, as for every step that is not a pure decoding step of few requests. The builder
knows nothing about models: it is handed tensors and sizes.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional

import torch

from .. import kernels
from ..kernels import ProgramOp, ProgramUnsupported

MAX_ROWS = 16

STORE, STORE_F32, ADD_RESIDUAL, SWIGLU, CONV = 0, 1, 2, 3, 4     # epilogues, the codes of the small-batch product


def enabled() -> bool:
    """CELEG_B200_DECODE_PROGRAM=1 runs pure decoding steps of up to 16 requests as one persistent kernel.
    Off by default: measured on a B200 at LFM2-1.2B sizes the program takes 1.1 ms a step at 8 requests
    against 0.77 ms for the same step as a CUDA graph of separate kernels (its fixed cost per operation,
    norm prologue + grid barrier + pipeline ramp, is about twice that of a kernel boundary in a graph)."""
    return os.environ.get("CELEG_B200_DECODE_PROGRAM", "0") == "1"


@dataclass
class NormedRows:
    """The operand of a product that is the RMSNorm of rows of the float32 residual stream."""
    weight: torch.Tensor                 # float32 [width]
    eps: float
    gather: Optional[torch.Tensor] = None   # int32 row list; None = rows 0..rows-1


class ProgramBuilder:
    """Collects the operations of one decoding step of ``rows`` requests (one token each)."""

    def __init__(self, rt, rows: int, residual: torch.Tensor, error_flag: torch.Tensor):
        if rt.act_dtype != torch.bfloat16:
            raise ProgramUnsupported("decode programs are bfloat16 only")
        if not 0 < rows <= MAX_ROWS:
            raise ProgramUnsupported(f"a decode program takes 1 to {MAX_ROWS} rows, not {rows}")
        self.rt = rt
        self.rows = rows
        self.residual = residual
        self.error_flag = error_flag
        self.ops: List[ProgramOp] = []
        self.keep: List[torch.Tensor] = []       # every tensor an operation points into

    # ---------------------------------------------------------------------------------- helpers
    def _ptr(self, tensor: Optional[torch.Tensor], dtype: Optional[torch.dtype] = None, what: str = "tensor") -> Optional[int]:
        if tensor is None:
            return None
        if not tensor.is_cuda or (dtype is not None and tensor.dtype != dtype):
            raise ProgramUnsupported(f"{what} must be a CUDA tensor of {dtype}, got {tensor.dtype} on {tensor.device}")
        self.keep.append(tensor)
        return tensor.data_ptr()

    @staticmethod
    def _row_stride(tensor: torch.Tensor, what: str) -> int:
        if tensor.dim() != 2 or tensor.stride(1) != 1:
            raise ProgramUnsupported(f"{what} must be a matrix with contiguous rows")
        return tensor.stride(0)

    # ------------------------------------------------------------------------------- operations
    def embed(self, table: torch.Tensor, token_ids: torch.Tensor, multiplier: float) -> None:
        """residual[r] = multiplier * table[token_ids[r]]"""
        op = ProgramOp()
        op.kind = kernels.OP_EMBED
        op.rows = self.rows
        op.w = self._ptr(table, torch.bfloat16, "the embedding table")
        op.ldw = self._row_stride(table, "the embedding table")
        op.vocab, op.n = table.shape
        op.y = self._ptr(self.residual, torch.float32, "the residual stream")
        op.ldy = self._row_stride(self.residual, "the residual stream")
        op.token_ids = self._ptr(token_ids, torch.int32, "token ids")
        op.multiplier = multiplier
        self.ops.append(op)

    def product(self, x, weight: torch.Tensor, out: Optional[torch.Tensor] = None, epilogue: int = STORE,
                add_to_residual: bool = False, rows: Optional[int] = None, out_scale: float = 1.0,
                conv_kernel: Optional[torch.Tensor] = None, taps: int = 0, state: Optional[torch.Tensor] = None,
                slot_stride: int = 0, span_slot: Optional[torch.Tensor] = None) -> None:
        """out = epilogue(x weight^T). x: a bfloat16 matrix, or NormedRows. SWIGLU: weight holds the gate
        rows then the up rows; CONV: the B, C and X rows of the short convolution, with the kernel
        [channels, taps], the layer's carried state and the slots of the rows. add_to_residual: the
        product, rounded to bfloat16 as a stored product would be, is added to the float32 residual."""
        op = ProgramOp()
        op.kind = kernels.OP_GEMV
        op.rows = self.rows if rows is None else rows
        sets = {SWIGLU: 2, CONV: 3}.get(epilogue, 1)
        total, k = weight.shape
        if total % sets:
            raise ProgramUnsupported(f"a weight of {total} rows does not hold {sets} equal parts")
        op.wt = sets
        op.n = total // sets
        op.k = k
        op.tile_offset = op.n
        op.w = self._ptr(weight, torch.bfloat16, "a projection weight")
        op.ldw = self._row_stride(weight, "a projection weight")
        if isinstance(x, NormedRows):
            op.x_source = kernels.X_NORM
            op.residual = self._ptr(self.residual, torch.float32, "the residual stream")
            op.ld_residual = self._row_stride(self.residual, "the residual stream")
            op.norm_weight = self._ptr(x.weight, torch.float32, "a norm weight")
            if x.weight.numel() != k:
                raise ProgramUnsupported(f"a norm of width {x.weight.numel()} in front of a product over {k}")
            op.eps = x.eps
            op.gather = self._ptr(x.gather, torch.int32, "the row list")
        else:
            op.x_source = kernels.X_GLOBAL
            op.x = self._ptr(x, torch.bfloat16, "an operand")
            op.ldx = self._row_stride(x, "an operand")
            op.x_rows = x.shape[0]
            if x.shape[1] < k:
                raise ProgramUnsupported(f"an operand of width {x.shape[1]} for a product over {k}")
        if add_to_residual:
            if epilogue != STORE or op.n != self.residual.shape[1]:
                raise ProgramUnsupported("only a plain product of the stream's width can be added to it")
            op.epilogue = ADD_RESIDUAL
            op.y = self._ptr(self.residual, torch.float32, "the residual stream")
            op.ldy = self._row_stride(self.residual, "the residual stream")
        else:
            op.epilogue = epilogue
            wanted = torch.float32 if epilogue == STORE_F32 else torch.bfloat16
            op.y = self._ptr(out, wanted, "the output of a product")
            op.ldy = self._row_stride(out, "the output of a product")
        op.out_scale = out_scale
        if epilogue == CONV:
            op.conv_w = self._ptr(conv_kernel, torch.float32, "the convolution kernel")
            op.taps = taps
            op.state = self._ptr(state, torch.float32, "the convolution state")
            op.slot_stride = slot_stride
            op.span_slot = self._ptr(span_slot, torch.int32, "the state slots")
        self.ops.append(op)

    def qk_norm_rope(self, qkv: torch.Tensor, q_norm, k_norm, inv_freq, rotary_dim: int, positions, token_span,
                     table: torch.Tensor, k_cache, v_cache, heads: int, stored_kv_heads: int, head_dim: int,
                     page_tokens: int, eps: float, store: bool) -> None:
        """Per-head norm and rotation of q (in place) and k, k and v written to their cache pages."""
        if qkv.stride(0) != (heads + 2 * stored_kv_heads) * head_dim:
            raise ProgramUnsupported("the q|k|v projection must be packed")
        op = ProgramOp()
        op.kind = kernels.OP_QK_NORM_ROPE
        op.rows = self.rows
        op.x = self._ptr(qkv, torch.bfloat16, "the q|k|v projection")
        op.q_weight = self._ptr(q_norm, torch.float32, "the q norm")
        op.k_weight = self._ptr(k_norm, torch.float32, "the k norm")
        op.inv_freq = self._ptr(inv_freq, torch.float32, "the rotation frequencies")
        op.rotary_dim = rotary_dim if inv_freq is not None else head_dim & ~1
        op.positions = self._ptr(positions, torch.int32, "positions")
        op.token_span = self._ptr(token_span, torch.int32, "token spans")
        op.block_table = self._ptr(table, torch.int32, "the block table")
        op.table_stride = table.stride(0)
        op.k_cache = self._ptr(k_cache, torch.bfloat16, "the key cache")
        op.v_cache = self._ptr(v_cache, torch.bfloat16, "the value cache")
        op.page_stride = k_cache.stride(0)
        op.q_heads, op.kv_heads, op.head_dim, op.page_tokens = heads, stored_kv_heads, head_dim, page_tokens
        op.eps = eps
        op.store_kv = 1 if store else 0
        self.ops.append(op)

    def attention(self, q: torch.Tensor, out: torch.Tensor, k_cache, v_cache, positions, token_span, table,
                  heads: int, kv_heads: int, head_dim: int, page_tokens: int, window: int, scale: float, chunk: int,
                  max_splits: int, partial_o, partial_ml, counters) -> None:
        """Paged attention of each row's one query token over its request's keys."""
        op = ProgramOp()
        op.kind = kernels.OP_ATTENTION
        op.rows = self.rows
        op.x = self._ptr(q, torch.bfloat16, "the queries")
        op.q_row_stride = self._row_stride(q, "the queries")
        op.y = self._ptr(out, torch.bfloat16, "the attention output")
        if out.stride(0) != heads * head_dim:
            raise ProgramUnsupported("the attention output must be packed")
        op.k_cache = self._ptr(k_cache, torch.bfloat16, "the key cache")
        op.v_cache = self._ptr(v_cache, torch.bfloat16, "the value cache")
        op.page_stride = k_cache.stride(0)
        op.positions = self._ptr(positions, torch.int32, "positions")
        op.token_span = self._ptr(token_span, torch.int32, "token spans")
        op.block_table = self._ptr(table, torch.int32, "the block table")
        op.table_stride = table.stride(0)
        op.q_heads, op.kv_heads, op.head_dim, op.page_tokens = heads, kv_heads, head_dim, page_tokens
        op.window = window or 0
        op.scale = scale
        op.chunk, op.max_splits = chunk, max_splits
        op.partial_o = self._ptr(partial_o, torch.float32, "attention scratch")
        op.partial_ml = self._ptr(partial_ml, torch.float32, "attention scratch")
        op.counters = self._ptr(counters, torch.int32, "attention counters")
        self.ops.append(op)

    # ---------------------------------------------------------------------------------- finish
    def build(self) -> "DecodeProgram":
        packed, layout = kernels.decode_program_prepare(self.ops)
        device = self.rt.device
        maps = kernels.decode_program_maps(packed, len(self.ops), layout)
        ops_device = torch.frombuffer(bytearray(packed), dtype=torch.uint8).to(device)
        maps_device = torch.frombuffer(bytearray(maps), dtype=torch.uint8).to(device)
        barriers = torch.zeros(len(self.ops) + 1, dtype=torch.int32, device=device)
        return DecodeProgram(ops_device, len(self.ops), layout, maps_device, barriers, self.error_flag, self.keep)


class DecodeProgram:
    """Prepared operations on the device; ``run()`` is one kernel launch."""

    def __init__(self, ops_device, n_ops, layout, maps_device, barriers, error_flag, keep):
        self.ops_device = ops_device
        self.n_ops = n_ops
        self.layout = layout
        self.maps_device = maps_device
        self.barriers = barriers
        self.error_flag = error_flag
        self.keep = keep

    def run(self, timeline: Optional[torch.Tensor] = None) -> None:
        kernels.decode_program_run(self.ops_device, self.n_ops, self.layout, self.maps_device, self.barriers,
                                   self.error_flag, timeline)

    def reset(self) -> None:
        """After a device error the barrier counters may be left mid-count."""
        self.barriers.zero_()
