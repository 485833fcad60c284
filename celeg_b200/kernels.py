"""Python face of the CUDA kernel library: loads (building it first if needed) the shared
object made from ``celeg_b200/csrc`` and wraps each entry point for torch tensors.

There is no fallback: if the library cannot be built or loaded, :func:`library` raises
:class:`KernelLibraryError`, and every wrapper raises it when a kernel reports an error.
Kernels run on torch's current CUDA stream.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional, Tuple

import torch

from .csrc import build as _build

FLOAT32 = 0
BFLOAT16 = 1


class KernelLibraryError(RuntimeError):
    pass


_LIB: Optional[ctypes.CDLL] = None


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return FLOAT32
    if dtype == torch.bfloat16:
        return BFLOAT16
    raise KernelLibraryError(f"the kernels handle float32 and bfloat16, not {dtype}")


_SIGNATURES = {
    "celeg_embedding": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
    "celeg_add_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int,
                          c_void_p],
    "celeg_rmsnorm_rows": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
    "celeg_short_conv": [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                         c_int, c_int, c_int, c_int, c_int, c_void_p],
    "celeg_qk_norm_rope_store": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                 c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                 c_int, c_void_p, c_int, c_void_p],
    "celeg_attention_generic": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p,
                                c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_int,
                                c_void_p],
    "celeg_attention_decode": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p,
                               c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "celeg_attention_decode_fused": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p,
                                     c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float,
                                     c_void_p],
    "celeg_attention_decode_solo_items": [c_longlong],
    "celeg_attention_decode_resident_blocks": [c_int],
    "celeg_attention_prefill": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p,
                                c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                c_void_p, c_void_p],
    "celeg_attention_prefill_tcgen05": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                        c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                        c_float, c_void_p, c_void_p],
    "celeg_gemv_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                        c_void_p, c_longlong, c_void_p, c_void_p],
    "celeg_gemv_prefetch_next": [c_void_p, c_longlong],
    "celeg_gemv_bf16_split_norm": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                   c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_float, c_int,
                                   c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p],
    "celeg_embedding_split_norm": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p,
                                   c_void_p, c_int, c_void_p],
    "celeg_gemm_tcgen05": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                           c_int, c_void_p],
    "celeg_swiglu": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "celeg_gemm_f32": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "celeg_sample": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                     c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "celeg_sample_scratch_elements": [],
    "celeg_sample_greedy": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_void_p],
    "celeg_mark_seen": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
}


def library() -> ctypes.CDLL:
    """The loaded kernel library; built at the first call in a fresh checkout."""
    global _LIB
    if _LIB is None:
        try:
            path = _build.ensure_built()
            lib = ctypes.CDLL(path)
        except (_build.BuildError, OSError) as exc:
            raise KernelLibraryError(f"the CUDA kernel library of celeg_b200 is not available: {exc}") from exc
        lib.celeg_last_error.restype = ctypes.c_char_p
        lib.celeg_last_error.argtypes = []
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        _LIB = lib
    return _LIB


def library_path() -> str:
    library()
    return _LIB._name  # type: ignore[union-attr]


LAUNCHES = 0        # entry-point calls made so far (each is one kernel launch unless it returned early)


def _check(code: int) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if code != 0:
        raise KernelLibraryError(library().celeg_last_error().decode("utf-8", "replace"))


def _ptr(tensor: Optional[torch.Tensor]) -> Optional[int]:
    if tensor is None:
        return None
    return tensor.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need(tensor: torch.Tensor, dtype: torch.dtype, name: str) -> None:
    if tensor.dtype != dtype or not tensor.is_cuda or not tensor.is_contiguous():
        raise KernelLibraryError(f"{name} must be a contiguous CUDA tensor of {dtype}, got {tensor.dtype} "
                                 f"on {tensor.device}, contiguous={tensor.is_contiguous()}")


# ------------------------------------------------------------------------------ wrappers
class SplitNorm:
    """An RMSNorm split over the two products around it (csrc/gemv_bf16.cu, GemvNormArgs): ``xw`` holds
    bfloat16 rows of residual * weight, ``sumsq[row, :partials]`` the pieces of each row's sum of squares;
    the product that takes ``xw`` as its operand multiplies its sums by 1 / sqrt(sum / width + eps)."""
    __slots__ = ("xw", "sumsq", "partials", "eps", "width")

    def __init__(self, xw: torch.Tensor, sumsq: torch.Tensor, partials: int, eps: float, width: int):
        self.xw, self.sumsq, self.partials, self.eps, self.width = xw, sumsq, partials, eps, width


def embedding(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, multiplier: float = 1.0,
              prepare: Optional[SplitNorm] = None, next_weight: Optional[torch.Tensor] = None) -> None:
    """out[t] = multiplier * table[tokens[t]]. With ``prepare``: also the first half of the norm whose
    weight is ``next_weight`` (``prepare.xw`` and one sum of squares per row are written)."""
    rows = tokens.shape[0]
    _need(tokens, torch.int32, "tokens")
    _need(out, torch.float32, "out")
    vocab, hidden = table.shape
    assert out.shape[0] >= rows and out.shape[1] == hidden
    if prepare is None:
        _check(library().celeg_embedding(_ptr(table), dtype_code(table.dtype), _ptr(tokens), _ptr(out), rows, hidden,
                                         vocab, multiplier, _stream()))
        return
    _need(next_weight, torch.float32, "next_weight")
    assert prepare.xw.dtype == torch.bfloat16 and prepare.xw.stride(0) == hidden and prepare.partials == 1
    _check(library().celeg_embedding_split_norm(
        _ptr(table), dtype_code(table.dtype), _ptr(tokens), _ptr(out), rows, hidden, vocab, multiplier,
        _ptr(next_weight), _ptr(prepare.xw), _ptr(prepare.sumsq), prepare.sumsq.stride(0), _stream()))


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor,
                eps: float, rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None,
                write_residual: bool = True) -> None:
    """out[i] = rmsnorm(residual[r] + delta[r]) * weight; residual[r] updated when not gathering."""
    _need(residual, torch.float32, "residual")
    _need(weight, torch.float32, "weight")
    width = residual.shape[-1]
    if n_rows is None:
        n_rows = rows.shape[0] if rows is not None else residual.shape[0]
    if delta is not None:
        assert delta.dtype == out.dtype and delta.shape[-1] == width
    _check(library().celeg_add_rmsnorm(_ptr(residual), _ptr(delta), _ptr(weight), _ptr(out), _ptr(rows), n_rows,
                                       width, eps, int(write_residual and rows is None), dtype_code(out.dtype),
                                       _stream()))


def rmsnorm_rows(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float, n_rows: int) -> None:
    _need(weight, torch.float32, "weight")
    _check(library().celeg_rmsnorm_rows(_ptr(x), _ptr(weight), _ptr(out), n_rows, x.shape[-1], eps,
                                        dtype_code(x.dtype), _stream()))


def short_conv(proj: torch.Tensor, kernel: torch.Tensor, state: torch.Tensor, slot_stride: int, out: torch.Tensor,
               token_span: torch.Tensor, span_begin: torch.Tensor, span_slot: torch.Tensor, tokens: int, spans: int,
               hidden: int, taps: int, max_span: Optional[int] = None) -> None:
    """``state`` points at this layer's state inside slot 0; ``slot_stride`` floats separate slots.
    ``max_span``: the longest span of the step if the caller knows it (saves a launch when no span is
    longer than the kernel); default: as long as the batch."""
    _need(kernel, torch.float32, "conv kernel")
    assert state.dtype == torch.float32
    _check(library().celeg_short_conv(_ptr(proj), _ptr(kernel), _ptr(state), slot_stride, _ptr(out),
                                      _ptr(token_span), _ptr(span_begin), _ptr(span_slot), tokens, spans, hidden,
                                      taps, tokens if max_span is None else max_span, dtype_code(proj.dtype),
                                      _stream()))


def qk_norm_rope_store(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                       inv_freq: Optional[torch.Tensor], positions: torch.Tensor, token_span: torch.Tensor,
                       block_table: torch.Tensor, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                       tokens: int, q_heads: int, kv_heads: int, head_dim: int, rotary_dim: int, page_tokens: int,
                       eps: float, store_kv, error_flag: torch.Tensor) -> None:
    """k_cache / v_cache: one layer's pages, [pages, kv_heads, page_tokens, head_dim]. ``store_kv``: False/0 = q
    heads only; True/1 = k (normalised, rotated) and v are written to the cache; 2 = k heads are normalised and
    rotated in place like the q heads, v heads and the cache are left alone."""
    page_stride = k_cache.stride(0) if k_cache is not None else 0
    _check(library().celeg_qk_norm_rope_store(
        _ptr(qkv), _ptr(q_weight), _ptr(k_weight), _ptr(inv_freq), _ptr(positions), _ptr(token_span),
        _ptr(block_table), block_table.stride(0), _ptr(k_cache), _ptr(v_cache), page_stride, tokens, q_heads,
        kv_heads, head_dim, rotary_dim, page_tokens, eps, int(store_kv), _ptr(error_flag), dtype_code(qkv.dtype),
        _stream()))


def attention_generic(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, k_cache: torch.Tensor,
                      v_cache: torch.Tensor, positions: torch.Tensor, token_span: torch.Tensor,
                      block_table: torch.Tensor, tokens: int, q_heads: int, kv_heads: int, head_dim: int,
                      page_tokens: int, window: Optional[int], scale: float, error_flag: torch.Tensor) -> None:
    _check(library().celeg_attention_generic(
        _ptr(q), q_row_stride, _ptr(out), _ptr(k_cache), _ptr(v_cache), k_cache.stride(0), _ptr(positions),
        _ptr(token_span), _ptr(block_table), block_table.stride(0), tokens, q_heads, kv_heads, head_dim,
        page_tokens, int(window or 0), scale, _ptr(error_flag), dtype_code(q.dtype), _stream()))


def attention_decode_supported(q_heads: int, kv_heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Shapes the split-key decode kernel takes; everything else goes to the general kernel."""
    return (dtype == torch.bfloat16 and q_heads % kv_heads == 0 and q_heads // kv_heads <= 16
            and head_dim % 8 == 0 and head_dim <= 256)


def attention_decode_resident_blocks(head_dim: int) -> int:
    """Blocks of the decode attention (its one-stage form) that the current device holds at a time; 0 if unknown."""
    return max(0, int(library().celeg_attention_decode_resident_blocks(int(head_dim))))


def attention_decode(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, k_cache: torch.Tensor,
                     v_cache: torch.Tensor, positions: torch.Tensor, token_span: torch.Tensor,
                     block_table: torch.Tensor, tokens: int, q_heads: int, kv_heads: int, head_dim: int,
                     page_tokens: int, window: Optional[int], scale: float, chunk: int, max_splits: int,
                     partial_o: torch.Tensor, partial_ml: torch.Tensor, counters: torch.Tensor,
                     error_flag: torch.Tensor) -> None:
    """One query token per row, keys split into chunks of ``chunk``; scratch: partial_o float32
    [tokens*q_heads*max_splits*head_dim], partial_ml float32 [tokens*q_heads*max_splits*2],
    counters int32 [tokens*kv_heads] (zero before the first call, left zero by every call)."""
    assert partial_o.numel() >= tokens * q_heads * max_splits * head_dim
    assert partial_ml.numel() >= tokens * q_heads * max_splits * 2
    assert counters.numel() >= tokens * kv_heads
    _check(library().celeg_attention_decode(
        _ptr(q), q_row_stride, _ptr(out), _ptr(k_cache), _ptr(v_cache), k_cache.stride(0), _ptr(positions),
        _ptr(token_span), _ptr(block_table), block_table.stride(0), tokens, q_heads, kv_heads, head_dim,
        page_tokens, int(window or 0), scale, chunk, max_splits, _ptr(partial_o), _ptr(partial_ml),
        _ptr(counters), _ptr(error_flag), _stream()))


def attention_decode_fused(qkv: torch.Tensor, q_row_stride: int, out: torch.Tensor, k_cache: torch.Tensor,
                           v_cache: torch.Tensor, positions: torch.Tensor, token_span: torch.Tensor,
                           block_table: torch.Tensor, tokens: int, q_heads: int, kv_heads: int, head_dim: int,
                           page_tokens: int, window: Optional[int], scale: float, chunk: int, max_splits: int,
                           partial_o: torch.Tensor, partial_ml: torch.Tensor, counters: torch.Tensor,
                           error_flag: torch.Tensor, q_weight: Optional[torch.Tensor],
                           k_weight: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], rotary_dim: int,
                           eps: float) -> None:
    """Decode attention over the raw q|k|v projection: per-head norm and rotation of q and of the token's own
    key, the cache write of that key and its value, and the attention, in one launch."""
    _check(library().celeg_attention_decode_fused(
        _ptr(qkv), q_row_stride, _ptr(out), _ptr(k_cache), _ptr(v_cache), k_cache.stride(0), _ptr(positions),
        _ptr(token_span), _ptr(block_table), block_table.stride(0), tokens, q_heads, kv_heads, head_dim, page_tokens,
        int(window or 0), scale, chunk, max_splits, _ptr(partial_o), _ptr(partial_ml), _ptr(counters),
        _ptr(error_flag), _ptr(q_weight), _ptr(k_weight), _ptr(inv_freq), rotary_dim, eps, _stream()))


def attention_prefill_supported(q_heads: int, kv_heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Shapes the tensor-core kernel for prompt portions takes; the rest goes to the general kernel."""
    return dtype == torch.bfloat16 and q_heads % kv_heads == 0 and head_dim % 8 == 0 and head_dim <= 256


def attention_prefill(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, k_cache: torch.Tensor,
                      v_cache: torch.Tensor, positions: torch.Tensor, span_begin: torch.Tensor,
                      block_table: torch.Tensor, tokens: int, spans: int, q_heads: int, kv_heads: int,
                      head_dim: int, page_tokens: int, window: Optional[int], scale: float,
                      error_flag: torch.Tensor) -> None:
    _check(library().celeg_attention_prefill(
        _ptr(q), q_row_stride, _ptr(out), _ptr(k_cache), _ptr(v_cache), k_cache.stride(0), _ptr(positions),
        _ptr(span_begin), _ptr(block_table), block_table.stride(0), tokens, spans, q_heads, kv_heads, head_dim,
        page_tokens, int(window or 0), scale, _ptr(error_flag), _stream()))


def attention_prefill_tcgen05_supported(q_heads: int, kv_heads: int, head_dim: int, page_tokens: int,
                                        dtype: torch.dtype) -> bool:
    """Shapes the tcgen05 kernel for prompt portions takes: head size 64, pages of 8, 16, 32 or 64 tokens."""
    return (dtype == torch.bfloat16 and head_dim == 64 and kv_heads > 0 and q_heads % kv_heads == 0
            and page_tokens >= 8 and page_tokens % 8 == 0 and 64 % page_tokens == 0)


def attention_prefill_tcgen05(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, k_cache: torch.Tensor,
                              v_cache: torch.Tensor, positions: torch.Tensor, span_begin: torch.Tensor,
                              block_table: torch.Tensor, tokens: int, spans: int, tile_count: int, q_heads: int,
                              kv_heads: int, head_dim: int, page_tokens: int, window: Optional[int], scale: float,
                              error_flag: torch.Tensor) -> None:
    """Prompt-portion attention on tcgen05 (S and O' in tensor memory, Q/K/V by TMA).
    ``tile_count`` = sum over the spans of ceil(length / 128)."""
    if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise KernelLibraryError("attention_prefill_tcgen05 needs contiguous cache layers")
    _check(library().celeg_attention_prefill_tcgen05(
        _ptr(q), q_row_stride, q.shape[0], _ptr(out), _ptr(k_cache), _ptr(v_cache), k_cache.shape[0], _ptr(positions),
        _ptr(span_begin), _ptr(block_table), block_table.stride(0), tokens, spans, tile_count, q_heads, kv_heads,
        head_dim, page_tokens, int(window or 0), scale, _ptr(error_flag), _stream()))


GEMV_MAX_ROWS = 16
GEMV_STORE, GEMV_STORE_F32, GEMV_ADD_RESIDUAL, GEMV_SWIGLU, GEMV_CONV = 0, 1, 2, 3, 4


def gemv_supported(rows: int, x: torch.Tensor, w: torch.Tensor) -> bool:
    return (0 < rows <= GEMV_MAX_ROWS and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and w.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0)


def gemv_bf16(x, w: torch.Tensor, y: torch.Tensor, rows: int, mode: int = GEMV_STORE, *,
              conv_w: Optional[torch.Tensor] = None, taps: int = 0, state: Optional[torch.Tensor] = None,
              slot_stride: int = 0, span_slot: Optional[torch.Tensor] = None,
              prepare: Optional[SplitNorm] = None, next_weight: Optional[torch.Tensor] = None,
              ahead: Optional[Tuple[int, int]] = None) -> None:
    """y[:rows] = x[:rows] @ w.T for at most 16 rows, streaming w once. mode GEMV_STORE: y bfloat16;
    GEMV_STORE_F32: y float32; GEMV_ADD_RESIDUAL: y float32, accumulated; GEMV_SWIGLU: w is
    [2*inner, k] (gate rows, then up rows) and y bfloat16 [rows, inner] = silu(gate) * up; GEMV_CONV: w is
    [3*channels, k] (B, C, X rows of the short convolution's input projection), y bfloat16
    [rows, channels] = C * conv(B*X) over each request's carried state, which is shifted; row i is the
    single token of request i, whose state slot is span_slot[i].
    ``x`` may be a :class:`SplitNorm` (the operand still lacks its row scale; applied to the sums here).
    With ``prepare`` (GEMV_ADD_RESIDUAL only): the first half of the norm that follows, weight
    ``next_weight``, is written too: ``prepare.xw`` and this product's pieces of the sums of squares.
    ``ahead`` = (device address, bytes) of the weights that the step's next product will read: this launch
    asks them into the L2 (the memory must outlive every graph that captures the launch)."""
    if ahead is not None and ahead[1] > 0:
        if library().celeg_gemv_prefetch_next(ctypes.c_void_p(ahead[0]), ahead[1]) != 0:      # (no launch)
            raise KernelLibraryError(library().celeg_last_error().decode("utf-8", "replace"))
    blocks = {GEMV_SWIGLU: 2, GEMV_CONV: 3}.get(mode, 1)
    n = w.shape[0] // blocks
    k = w.shape[1]
    scaled = x if isinstance(x, SplitNorm) else None
    operand = scaled.xw if scaled is not None else x
    assert operand.shape[-1] == k and y.shape[-1] >= n
    want = torch.float32 if mode in (GEMV_STORE_F32, GEMV_ADD_RESIDUAL) else torch.bfloat16
    if y.dtype != want:
        raise KernelLibraryError(f"gemv_bf16 mode {mode} writes {want}, got {y.dtype}")
    if scaled is None and prepare is None:
        _check(library().celeg_gemv_bf16(_ptr(operand), operand.stride(0), _ptr(w), w.stride(0), _ptr(y), y.stride(0),
                                         rows, n, k, mode, _ptr(conv_w), taps, _ptr(state), slot_stride,
                                         _ptr(span_slot), _stream()))
        return
    if prepare is not None:
        _need(next_weight, torch.float32, "next_weight")
        if prepare.partials != (n + 15) // 16 or prepare.sumsq.stride(0) < prepare.partials:
            raise KernelLibraryError(f"a product of {n} columns writes {(n + 15) // 16} pieces of the sums, "
                                     f"not {prepare.partials}")
    _check(library().celeg_gemv_bf16_split_norm(
        _ptr(operand), operand.stride(0), _ptr(w), w.stride(0), _ptr(y), y.stride(0), rows, n, k, mode,
        _ptr(conv_w), taps, _ptr(state), slot_stride, _ptr(span_slot),
        _ptr(scaled.sumsq) if scaled else None, scaled.partials if scaled else 0,
        scaled.sumsq.stride(0) if scaled else 0, scaled.eps if scaled else 0.0, scaled.width if scaled else 0,
        _ptr(next_weight) if prepare else None, _ptr(prepare.xw) if prepare else None,
        prepare.xw.stride(0) if prepare else 0, _ptr(prepare.sumsq) if prepare else None,
        prepare.sumsq.stride(0) if prepare else 0, _stream()))


TC_STORE, TC_STORE_F32, TC_SWIGLU = 0, 1, 2


def gemm_tcgen05_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, rows: int, epilogue: int,
                 error_flag: torch.Tensor, variant: int = -1) -> None:
    """y[:rows] = x[:rows] @ w.T on tcgen05 tensor cores (TMA-fed, accumulator in tensor memory).
    TC_STORE: y bfloat16; TC_STORE_F32: y float32; TC_SWIGLU: w is [2*inner, k] (gate rows, then up rows),
    y bfloat16 [rows, inner] = silu(gate) * up. ``variant``: -1 lets the library choose the tile shape,
    0..3 force one (128x128 with 6 or 3 stages, 128x256, persistent with two accumulators)."""
    n = w.shape[0] // 2 if epilogue == TC_SWIGLU else w.shape[0]
    k = w.shape[1]
    want = torch.float32 if epilogue == TC_STORE_F32 else torch.bfloat16
    if y.dtype != want:
        raise KernelLibraryError(f"gemm_tcgen05 epilogue {epilogue} writes {want}, got {y.dtype}")
    assert x.shape[-1] == k and y.shape[-1] >= n
    _check(library().celeg_gemm_tcgen05(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(y), y.stride(0), rows, n, k,
                                        epilogue, _ptr(error_flag), int(variant), _stream()))


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, tokens: int, inner: int) -> None:
    _check(library().celeg_swiglu(_ptr(gate_up), _ptr(out), tokens, inner, dtype_code(gate_up.dtype), _stream()))


def gemm_f32(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, m: int, accumulate: bool = False) -> None:
    """y[:m] (+)= x[:m] @ w.T with float32 operands and FFMA accumulation."""
    _need(w, torch.float32, "w")
    assert x.dtype == torch.float32 and y.dtype == torch.float32
    n, k = w.shape
    assert x.stride(-1) == 1 and y.stride(-1) == 1 and x.shape[-1] == k and y.shape[-1] == n
    _check(library().celeg_gemm_f32(_ptr(x), _ptr(w), _ptr(y), m, n, k, x.stride(0), w.stride(0), y.stride(0),
                                    int(accumulate), _stream()))


def sample_scratch(device) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Scratch that lets :func:`sample` cut the rows of a small batch into pieces (one block each): candidate
    scores, candidate tokens and their counts."""
    elements = int(library().celeg_sample_scratch_elements())
    return (torch.zeros(elements, dtype=torch.float32, device=device),
            torch.zeros(elements, dtype=torch.int32, device=device),
            torch.zeros(elements // 128, dtype=torch.int32, device=device))


def sample(logits: torch.Tensor, rows: int, row_slot: Optional[torch.Tensor], seen: Optional[torch.Tensor],
           rng: Optional[torch.Tensor], temperature: Optional[torch.Tensor], top_k: Optional[torch.Tensor],
           top_p: Optional[torch.Tensor], penalty: Optional[torch.Tensor], out: torch.Tensor,
           scratch: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None) -> None:
    """One token per row with celeg's rules. ``scratch`` (:func:`sample_scratch`): with it, a batch of at most
    32 rows over a large vocabulary runs as 16 blocks per row and a merge; without it, one block per row."""
    _need(logits, torch.float32, "logits")
    _need(out, torch.int32, "out")
    parts = scratch or (None, None, None)
    _check(library().celeg_sample(_ptr(logits), logits.stride(0), logits.shape[1], rows, _ptr(row_slot), _ptr(seen),
                                  _ptr(rng), _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(penalty), _ptr(out),
                                  _ptr(parts[0]), _ptr(parts[1]), _ptr(parts[2]), _stream()))


def sample_greedy(logits: torch.Tensor, rows: int, row_slot: Optional[torch.Tensor], seen: Optional[torch.Tensor],
                  penalty: Optional[torch.Tensor], out: torch.Tensor, partial_score: torch.Tensor,
                  partial_token: torch.Tensor) -> None:
    """Arg-max (first maximum) of every row after the repetition penalty; scratch: rows*64 each."""
    _need(logits, torch.float32, "logits")
    _need(out, torch.int32, "out")
    assert partial_score.numel() >= rows * 64 and partial_token.numel() >= rows * 64
    _check(library().celeg_sample_greedy(_ptr(logits), logits.stride(0), logits.shape[1], rows, _ptr(row_slot),
                                         _ptr(seen), _ptr(penalty), _ptr(out), _ptr(partial_score),
                                         _ptr(partial_token), _stream()))
    global LAUNCHES
    LAUNCHES += 1                                     # two kernels


def mark_seen(seen: torch.Tensor, tokens: torch.Tensor, token_span: torch.Tensor, span_slot: torch.Tensor,
              count: int) -> None:
    _check(library().celeg_mark_seen(_ptr(seen), seen.shape[1], _ptr(tokens), _ptr(token_span), _ptr(span_slot),
                                     count, _stream()))
