"""What parts share at run time: the device, the precision of the path, scratch buffers, the
matrix product, and the description of the step being run."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from .. import kernels
from .options import KernelOptions


LIBRARY_ROW_STEP = 64        # row counts of library products are rounded up to a multiple of this (of 8 up to it)


class _Sink:
    """Where a part is about to leave its output, and the norm that will read the stream next."""
    __slots__ = ("buffer", "norm", "weight", "split", "used")

    def __init__(self, buffer, norm, weight, split):
        self.buffer, self.norm, self.weight, self.split, self.used = buffer, norm, weight, split, False


class ResidualStream:
    """The float32 residual stream of one step, with what is still owed to it: a part writes its
    output to a buffer, the buffer becomes ``pending``, and it is added inside the next norm kernel
    (residual add and norm are one launch).

    Steps of few rows on the bfloat16 path skip that launch: when the part that reads the stream next
    takes a split norm (``takes_split_norm``), the product that ends a part adds to the stream itself
    and prepares the norm that follows (``expect`` tells the runtime where that product will write),
    and ``normed`` hands the next part a :class:`kernels.SplitNorm` instead of normalised rows."""

    def __init__(self, rt: "Runtime", hidden: int):
        self.rt = rt
        self.hidden = hidden
        self.residual = rt.scratch("stream.residual", hidden, torch.float32)
        self.pending: Optional[torch.Tensor] = None
        self.prepared = None                    # (norm, SplitNorm) left by the last product
        self.after_layer = None                 # the norm after the layer being run, if its reader takes a split norm
        self.pieces = (hidden + 15) // 16
        if rt.act_dtype == torch.bfloat16:
            self.xw = rt.scratch("stream.split_norm", hidden, torch.bfloat16)
            self.sumsq = torch.zeros((kernels.GEMV_MAX_ROWS, self.pieces), dtype=torch.float32, device=rt.device)

    def begin(self) -> None:
        self.pending = None
        self.prepared = None
        self.after_layer = None
        self.rt.sink = None

    def split(self, norm, pieces: int):
        """(weight, SplitNorm) for a norm that can be split, else None."""
        halves = norm.as_prologue() if hasattr(norm, "as_prologue") else None
        if halves is None or self.rt.act_dtype != torch.bfloat16 or norm.width != self.hidden:
            return None
        weight, eps = halves
        return weight, kernels.SplitNorm(self.xw, self.sumsq, pieces, eps, self.hidden)

    def normed(self, norm, out: torch.Tensor, rows: int, gather: Optional[torch.Tensor] = None):
        """out = norm(stream + pending) for the first ``rows`` rows (or the gathered ones). Without
        ``gather`` what was pending is added for good. Returns ``out``, or the split norm that the
        last product prepared for exactly this norm."""
        if self.prepared is not None:
            prepared_norm, split = self.prepared
            self.prepared = None
            if prepared_norm is norm and gather is None:
                return split
            raise RuntimeError("a norm was prepared for another reader than the one that asks")
        norm.add_norm(self.residual, self.pending, out, rows, rows=gather)
        if gather is None:
            self.pending = None
        return out

    def expect(self, buffer: torch.Tensor, upcoming, rows: int) -> None:
        """A part is about to write its output to ``buffer``; ``upcoming`` is the norm that reads the
        stream after it (None when its reader wants normalised rows)."""
        self.rt.sink = None
        if upcoming is None or not self.rt.small_batch(rows):
            return
        halves = self.split(upcoming, self.pieces)
        if halves is not None:
            self.rt.sink = _Sink(buffer, upcoming, halves[0], halves[1])
            self.rt.sink_residual = self.residual

    def add_later(self, delta: torch.Tensor) -> None:
        assert self.pending is None
        sink, self.rt.sink = self.rt.sink, None
        if sink is not None and sink.used:
            self.prepared = (sink.norm, sink.split)          # the product has added to the stream already
            return
        self.pending = delta


class Runtime:
    """One per model instance. ``act_dtype`` is float32 (everything in true 32-bit) or bfloat16
    (the serving path: bfloat16 matrices and activations; residual stream, norms, softmax,
    rotation angles and conv state in float32)."""

    def __init__(self, device: torch.device, act_dtype: torch.dtype, max_tokens: int, max_requests: int = 8,
                 max_context: int = 4096, options: Optional[KernelOptions] = None):
        options = options or KernelOptions()
        if act_dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"dtype must be float32 or bfloat16, got {act_dtype}")
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise kernels.KernelLibraryError("celeg_b200 runs on a CUDA device only; there is no CPU path")
        self.act_dtype = act_dtype
        self.max_tokens = max_tokens
        self.max_requests = max_requests
        self.max_context = max_context
        options.validate()
        self.options = options
        self.fuse_small_batches = options.fuse_small_batches
        self.tensor_core_products = options.tensor_core_products
        self.tensor_core_min_rows = options.tensor_core_min_rows
        self.tensor_core_min_width = options.tensor_core_min_width
        self.tensor_core_variant = options.tensor_core_variant
        self.split_norms = options.split_norms
        self.fuse_decode_qk = options.fuse_decode_qk
        self.tcgen05_attention = options.tcgen05_attention
        # Decode steps are a chain of short weight-streaming kernels, the same chain every step. Each of them
        # asks the first megabytes of its successor's weights into the L2, so that memory works across the
        # kernel boundary; the successor of a weight is learnt from the order of the calls (the first step of
        # a shape runs outside graph capture).
        self.prefetch_bytes = int(options.prefetch_mb * (1 << 20))
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.sink: Optional[_Sink] = None         # set by the residual stream around a part's forward
        self.sink_residual: Optional[torch.Tensor] = None
        self._weight_after: Dict[int, Tuple[int, int]] = {}
        self._streamed_last: Optional[int] = None
        self._flat: Dict[Tuple[str, int, torch.dtype], torch.Tensor] = {}
        self._placed: Dict[tuple, Tuple[torch.Tensor, torch.Tensor]] = {}
        self._scratch: Dict[Tuple[str, int, torch.dtype], torch.Tensor] = {}
        self.weight_bytes = 0                   # what matrix() and vector() have put on the device
        kernels.library()                       # fail now, not at the first step, if it is missing

    def scratch(self, tag: str, columns: int, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """A persistent [max_tokens, columns] buffer. Parts that ask with the same tag, width and
        type share it, which is safe because layers run one after another."""
        dtype = dtype or self.act_dtype
        key = (tag, columns, dtype)
        if key not in self._scratch:
            self._scratch[key] = torch.empty((self.max_tokens, columns), dtype=dtype, device=self.device)
        return self._scratch[key]

    def flat_scratch(self, tag: str, elements: int, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """A persistent 1-D buffer shared by parts that ask with the same tag, size and type."""
        key = (tag, elements, dtype)
        if key not in self._flat:
            make = torch.zeros if zero else torch.empty
            self._flat[key] = make(elements, dtype=dtype, device=self.device)
        return self._flat[key]

    def matrix(self, weight: torch.Tensor) -> torch.Tensor:
        """A projection weight on the device in the path's matrix precision. A tensor that two parts name (a
        head tied to the embedding table) is placed once: both get the same device tensor."""
        key = (weight.data_ptr(), tuple(weight.shape), tuple(weight.stride()), weight.dtype)
        held = self._placed.get(key)
        if held is not None and held[0] is weight:
            return held[1]
        placed = weight.to(device=self.device, dtype=self.act_dtype).contiguous()
        self.weight_bytes += placed.numel() * placed.element_size()
        self._placed[key] = (weight, placed)
        return placed

    def release_sources(self) -> None:
        """Forget the host tensors that :meth:`matrix` has placed (call when the model is built)."""
        self._placed = {}

    def vector(self, weight: torch.Tensor) -> torch.Tensor:
        """A small weight (norm scale, conv kernel) on the device in float32 (exact widening)."""
        placed = weight.to(device=self.device, dtype=torch.float32).contiguous()
        self.weight_bytes += placed.numel() * 4
        return placed

    def takes_split_norm(self, rows: int, weight: torch.Tensor) -> bool:
        """Whether a product of ``rows`` rows with ``weight`` can take an operand that still lacks its
        row scale (a :class:`kernels.SplitNorm`): only the small-batch kernel applies one."""
        return (self.split_norms and self.small_batch(rows) and weight.dtype == torch.bfloat16
                and weight.shape[1] % 8 == 0 and weight.stride(0) % 8 == 0)

    def small_batch(self, rows: int) -> bool:
        """Whether a step of ``rows`` tokens takes the fused small-batch products."""
        return (self.fuse_small_batches and self.act_dtype == torch.bfloat16 and
                0 < rows <= kernels.GEMV_MAX_ROWS)

    def _ahead(self, weight: torch.Tensor) -> Optional[Tuple[int, int]]:
        """Notes that ``weight`` (a matrix of this runtime's model, alive as long as the runtime) is streamed
        now, after the one noted before; returns (address, bytes) of what followed it last time, if known."""
        if self.prefetch_bytes <= 0:
            return None
        here = weight.data_ptr()
        if self._streamed_last is not None and self._streamed_last != here:
            self._weight_after[self._streamed_last] = (here, min(weight.numel() * weight.element_size(),
                                                                 self.prefetch_bytes))
        self._streamed_last = here
        return self._weight_after.get(here)

    def linear(self, x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, rows: int) -> None:
        """out[:rows] = x[:rows] @ weight.T. float32 path: this package's FFMA kernel. bfloat16 path: at
        most 16 rows go to this package's weight-streaming kernel, more rows to the library product
        (cuBLAS through torch), as celeg uses cuBLAS for these
        (src/backend/cuda/runtime/gemm_dispatcher.cpp:49-64); float32 accumulation everywhere."""
        if rows == 0:
            return
        split = isinstance(x, kernels.SplitNorm)
        operand = x.xw if split else x
        if self.act_dtype == torch.float32:
            kernels.gemm_f32(x, weight, out, rows)
        elif kernels.gemv_supported(rows, operand, weight):
            sink = self.sink
            if sink is not None and out is sink.buffer and weight.shape[0] == self.sink_residual.shape[1]:
                # the product that ends a part: added to the stream here, and the next norm prepared
                kernels.gemv_bf16(x, weight, self.sink_residual, rows, kernels.GEMV_ADD_RESIDUAL,
                                  prepare=sink.split, next_weight=sink.weight, ahead=self._ahead(weight))
                sink.used = True
                return
            kernels.gemv_bf16(x, weight, out, rows,
                              kernels.GEMV_STORE_F32 if out.dtype == torch.float32 else kernels.GEMV_STORE,
                              ahead=self._ahead(weight))
        elif split:
            raise kernels.KernelLibraryError("an operand without its row scale reached a product that cannot apply it")
        elif self.tensor_core_products == "all" and kernels.gemm_tcgen05_supported(x, weight):
            kernels.gemm_tcgen05(x, weight, out, rows,
                                 kernels.TC_STORE_F32 if out.dtype == torch.float32 else kernels.TC_STORE,
                                 self.error_flag, self.tensor_core_variant)
        else:
            # The library chooses its kernel per shape and looks every new shape up (tens of microseconds on
            # the host): steps whose number of rows changes every time (decoded tokens beside portions) would pay
            # that for every product. The product therefore runs on a row count from a coarse grid; the rows
            # past ``rows`` hold what an earlier step left there, each row of a product depends on its own
            # row of the operand only, and nobody reads their results.
            step = 8 if rows <= LIBRARY_ROW_STEP else LIBRARY_ROW_STEP      # (few rows: the library has faster kernels)
            padded = min(-(-rows // step) * step, x.shape[0], out.shape[0])
            if out.dtype == torch.float32:
                torch.mm(x[:padded], weight.t(), out_dtype=torch.float32, out=out[:padded])
            else:
                torch.mm(x[:padded], weight.t(), out=out[:padded])

    def linear_swiglu(self, x: torch.Tensor, gate_up_weight: torch.Tensor, scratch: torch.Tensor,
                      out: torch.Tensor, rows: int, inner: int) -> None:
        """out[:rows] = silu(x gate^T) * (x up^T) with gate_up_weight = [gate rows; up rows]. Few
        bfloat16 rows: one weight-streaming kernel; very many bfloat16 rows: one tcgen05 kernel; otherwise the
        product into ``scratch`` and the activation kernel."""
        if rows == 0:
            return
        operand = x.xw if isinstance(x, kernels.SplitNorm) else x
        if self.act_dtype == torch.bfloat16 and kernels.gemv_supported(rows, operand, gate_up_weight):
            kernels.gemv_bf16(x, gate_up_weight, out, rows, kernels.GEMV_SWIGLU, ahead=self._ahead(gate_up_weight))
            return
        if (self.act_dtype == torch.bfloat16 and kernels.gemm_tcgen05_supported(x, gate_up_weight)
                and (self.tensor_core_products == "all"
                     or (self.tensor_core_products == "swiglu" and rows >= self.tensor_core_min_rows
                         and gate_up_weight.shape[1] >= self.tensor_core_min_width))):
            kernels.gemm_tcgen05(x, gate_up_weight, out, rows, kernels.TC_SWIGLU, self.error_flag,
                                 self.tensor_core_variant)
            return
        self.linear(x, gate_up_weight, scratch, rows)
        kernels.swiglu(scratch, out, rows, inner)

    def linear_short_conv(self, x: torch.Tensor, in_weight: torch.Tensor, conv_kernel: torch.Tensor, taps: int,
                          binding, out: torch.Tensor, step: "StepContext") -> bool:
        """The short convolution's input projection with its gate fused in, for steps in which every
        request brings one token and there are few of them. Returns False when that does not apply
        and the caller has to run projection and convolution separately."""
        rows = step.tokens
        hidden = conv_kernel.shape[0]
        operand = x.xw if isinstance(x, kernels.SplitNorm) else x
        if not (self.small_batch(rows) and step.max_span == 1 and step.spans == rows and taps <= 16
                and kernels.gemv_supported(rows, operand, in_weight)):
            return False
        kernels.gemv_bf16(x, in_weight, out, rows, kernels.GEMV_CONV, conv_w=conv_kernel, taps=taps,
                          state=binding.state, slot_stride=binding.slot_stride, span_slot=step.span_slot,
                          ahead=self._ahead(in_weight))
        return True


@dataclass
class StepContext:
    """Device-side description of one step, the same for every layer. All index tensors are
    int32 and persistent (their addresses do not change between steps)."""
    tokens: int                       # T: tokens in this step
    spans: int                        # R: requests in this step
    token_ids: torch.Tensor           # [T]
    positions: torch.Tensor           # [T] absolute position of each token in its request
    token_span: torch.Tensor          # [T] index of the span a token belongs to
    span_begin: torch.Tensor          # [R+1] first token of each span (prefix sums)
    span_slot: torch.Tensor           # [R] state slot of each span's request
    block_tables: List[torch.Tensor]  # per paged group: [R, max_pages] page ids, -1 = none
    error_flag: torch.Tensor          # [1] set by a kernel that met an impossible index
    max_span: int = 1                 # longest span (host knowledge, for kernel choice)
    max_context: int = 0              # largest position + 1 in the step
    context_bucket: int = 0           # max_context rounded up to a power of two (launch shapes use this)
    logits_of_all_rows: bool = False  # the wanted rows are exactly rows 0..tokens-1 in order
    host_positions: Optional[list] = None
    host_span_lengths: Optional[list] = None
    leading_single_tokens: int = 0    # how many spans at the start of the step bring exactly one token
    # an upper bound of the prompt attention's query tiles that does not depend on the spans' lengths (steps
    # padded to a launch shape that a graph is replayed for); None: count the tiles from the lengths
    prompt_tile_bound: Optional[int] = None
    extras: Dict[str, object] = field(default_factory=dict)
