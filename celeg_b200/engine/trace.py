"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: every step goes through
the StepFunction that generation uses. celeg has no such tool; its closest pieces are
``--dump-logits`` after prefill (src/app/cuda/main.cpp:554-558) and forced-token evaluation
(src/backend/cpu/model.cpp:162-178).

Input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, ``<out>/<step>.f32`` holds the logits at the wanted
places, little-endian float32 [wanted, vocab]. After every step a line ``done <step>`` is
printed and flushed. ``<out>/model.json`` names the model that made the files (its fingerprint).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import IO, Optional

PAGE_ROUNDING = 64      # --max-tokens counts every live request rounded up to a multiple of this
MAX_STEP_TOKENS = 8192  # tokens one pass holds; a larger step is run as several passes


def replay(model_dir: str, dtype: str, out_dir: str, max_tokens: int, lines: IO[str], done: IO[str],
           device: str = "cuda:0", page_tokens: Optional[int] = None, max_requests: int = 8,
           max_batched_tokens: Optional[int] = None) -> int:
    import torch

    from .loading import DEFAULT_PAGE_TOKENS, load_model
    from .step import StepEntry

    os.makedirs(out_dir, exist_ok=True)
    page_tokens = page_tokens or DEFAULT_PAGE_TOKENS
    if PAGE_ROUNDING % page_tokens and page_tokens % PAGE_ROUNDING:
        raise ValueError(f"page size {page_tokens} neither divides nor is a multiple of {PAGE_ROUNDING}")
    batch_limit = max_batched_tokens or min(max(max_tokens, PAGE_ROUNDING), MAX_STEP_TOKENS)
    loaded = load_model(model_dir, dtype=dtype, device=device, cache_tokens=max_tokens, page_tokens=page_tokens,
                        max_requests=max_requests, max_batched_tokens=batch_limit)
    step_fn = loaded.step
    with open(os.path.join(out_dir, "model.json"), "w", encoding="utf-8") as handle:
        json.dump({"model_fingerprint": loaded.fingerprint, "dtype": str(dtype),
                   "vocab_size": loaded.model.vocab_size}, handle)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        number = record["step"]
        entries = [StepEntry(request_id=item["id"], tokens=item["tokens"], want=item.get("want", []))
                   for item in record.get("entries", []) if len(item["tokens"]) > 0]      # (no tokens: left out)
        if entries:
            pieces = []
            for part in _within_limit(entries, batch_limit, StepEntry):
                logits = step_fn.run(part, auto_begin=True)
                if logits.shape[0] > 0:
                    pieces.append(logits.to("cpu", copy=True).contiguous().numpy().astype("<f4", copy=False))
            if pieces:
                with open(os.path.join(out_dir, f"{number}.f32"), "wb") as handle:
                    for piece in pieces:
                        handle.write(piece.tobytes())
            else:
                torch.cuda.current_stream().synchronize()
            step_fn.raise_on_device_error()
        for request_id in record.get("end", []):
            if loaded.manager.find(request_id) is not None:      # (a request that never brought a token holds nothing)
                step_fn.end(request_id)
        done.write(f"done {number}\n")
        done.flush()
    return 0


def _within_limit(entries, limit: int, entry_type):
    """A step that brings more tokens than the step function's buffers hold is run as several steps, cut
    in order (which changes no logits): yields lists of entries of at most ``limit`` tokens, every
    wanted place kept with the portion that holds it, so the logits come out in the order asked for."""
    total = sum(len(entry.tokens) for entry in entries)
    if total <= limit:
        yield entries
        return
    batch, room = [], limit
    for entry in entries:
        at = 0
        while at < len(entry.tokens):
            take = min(room, len(entry.tokens) - at)
            want = [w - at for w in entry.want if at <= w < at + take]
            batch.append(entry_type(entry.request_id, entry.tokens[at:at + take], want))
            at += take
            room -= take
            if room == 0:
                yield batch
                batch, room = [], limit
    if batch:
        yield batch


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time, each rounded up to 64")
    parser.add_argument("--device", default="cuda:0")
    parser.add_argument("--page-tokens", type=int, default=None)
    args = parser.parse_args(argv)
    try:
        return replay(args.model, args.dtype, args.out, args.max_tokens, sys.stdin, sys.stdout,
                      device=args.device, page_tokens=args.page_tokens)
    except Exception as exc:  # one line for the user, non-zero exit
        print(f"error: {type(exc).__name__}: {exc}", file=sys.stderr, flush=True)
        return 1
