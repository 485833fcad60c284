"""``celeg-run`` for this engine: celeg's option names and meanings where it has them
(src/app/cuda/main.cpp:38-95 defaults, :97-274 parsing, :523-598 output lines), token ids in
place of text because tokenizers are outside this engine.

Kept from celeg: --model, --max-new-tokens (128), --context (4096), --temperature (0.1),
--top-k (1), --top-p (1.0), --repetition-penalty (1.05), --seed (1), --dump-logits FILE,
--print-top N, --tokens-only, --runtime-tokens, --print-config, --benchmark-decode N,
--benchmark-warmup N (8), --benchmark-prefill-tokens N, --runtime-metrics, --memory-report,
--no-cuda-graph, --prefill-chunk (256), --kv-cache bf16, --weight-mode auto|bf16.
Added: --prompt-ids, --prompt-ids-file, --random-weights SEED with --config FILE, --dtype,
--kv-pages, --page-tokens, --max-batched-tokens, --max-active-requests.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time
from typing import List, Optional


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="celeg-run", description="Generate tokens with the celeg_b200 engine.")
    p.add_argument("model_positional", nargs="?", default=None, help="model folder (same as --model)")
    p.add_argument("--model", default=None, help="folder with config.json and model.safetensors")
    p.add_argument("--prompt", default=None, help="not supported: this engine takes token ids (--prompt-ids)")
    p.add_argument("--prompt-ids", default=None, help="comma-separated token ids of the prompt")
    p.add_argument("--prompt-ids-file", default=None, help="file with token ids separated by commas or whitespace")
    p.add_argument("--max-new-tokens", type=int, default=128)
    p.add_argument("--context", type=int, default=4096)
    p.add_argument("--temperature", type=float, default=0.1)
    p.add_argument("--top-k", type=int, default=1)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--repetition-penalty", type=float, default=1.05)
    p.add_argument("--seed", type=int, default=1)
    p.add_argument("--dump-logits", default=None, metavar="FILE.f32",
                   help="write the float32 logits of the last prompt token")
    p.add_argument("--print-top", type=int, default=0, metavar="N")
    p.add_argument("--tokens-only", action="store_true", help="print the prompt's token ids and exit")
    p.add_argument("--runtime-tokens", action="store_true", help="print CELEG_GENERATED_TOKEN_IDS=[...]")
    p.add_argument("--print-config", action="store_true")
    p.add_argument("--benchmark-decode", type=int, default=0, metavar="N")
    p.add_argument("--benchmark-warmup", type=int, default=8, metavar="N")
    p.add_argument("--benchmark-prefill-tokens", type=int, default=0, metavar="N",
                   help="pad or cut the prompt to N tokens by repeating its last id")
    p.add_argument("--runtime-metrics", action="store_true")
    p.add_argument("--memory-report", action="store_true")
    p.add_argument("--no-cuda-graph", action="store_true")
    p.add_argument("--prefill-chunk", type=int, default=256)
    p.add_argument("--kv-cache", default="bf16", help="bf16 only (quantised caches are not part of this engine)")
    p.add_argument("--weight-mode", default="auto", help="auto or bf16 only")
    p.add_argument("--dtype", default="bf16", choices=["bf16", "bfloat16", "fp32", "float32"])
    p.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                   help="write a random model from --config into --model (or a temporary folder) first")
    p.add_argument("--config", default=None, help="config.json for --random-weights")
    p.add_argument("--kv-pages", type=int, default=0)
    p.add_argument("--page-tokens", type=int, default=16)
    p.add_argument("--max-batched-tokens", type=int, default=512)
    p.add_argument("--max-active-requests", type=int, default=8)
    p.add_argument("--device", default="cuda:0")
    return p


def _prompt_ids(args) -> Optional[List[int]]:
    text = None
    if args.prompt_ids is not None:
        text = args.prompt_ids
    elif args.prompt_ids_file is not None:
        with open(args.prompt_ids_file, "r", encoding="utf-8") as handle:
            text = handle.read()
    if text is None:
        return None
    parts = [part for part in text.replace(",", " ").split() if part]
    try:
        return [int(part) for part in parts]
    except ValueError:
        raise ValueError("--prompt-ids must hold integers separated by commas") from None


def run(argv=None) -> int:
    args = build_parser().parse_args(argv)
    model_dir = args.model or args.model_positional
    if args.prompt is not None:
        raise ValueError("--prompt takes text, and tokenizers are outside this engine: give --prompt-ids")
    if args.kv_cache != "bf16":
        raise ValueError("--kv-cache must be bf16 (quantised caches are not part of this engine)")
    if args.weight_mode not in ("auto", "bf16"):
        raise ValueError("--weight-mode must be auto or bf16 (quantised weights are not part of this engine)")

    if args.random_weights is not None:
        if not args.config:
            raise ValueError("--random-weights needs --config FILE")
        from .weights import write_random_model
        with open(args.config, "r", encoding="utf-8") as handle:
            raw = json.load(handle)
        model_dir = model_dir or tempfile.mkdtemp(prefix="celeg_b200_random_")
        write_random_model(model_dir, raw, args.random_weights)
        print(f"random model written to {model_dir}", file=sys.stderr)
    if not model_dir:
        raise ValueError("--model is required")

    from .config import architecture_of, read_config_json
    raw = read_config_json(model_dir)
    architecture = architecture_of(raw)
    if args.print_config:
        from .engine.loading import fingerprint_of
        from .weights import TensorRepository
        repository = TensorRepository(model_dir)
        try:
            config = architecture.resolve_config(architecture.parse_config(raw), repository.shapes())
            fingerprint = fingerprint_of(config, raw, repository)
        finally:
            repository.close()
        print(json.dumps(config.to_dict(), indent=1))
        print(f"model_fingerprint={fingerprint}")
        if _prompt_ids(args) is None:
            return 0

    prompt = _prompt_ids(args)
    if prompt is None:
        raise ValueError("--prompt-ids is required unless --print-config is used")
    if not prompt:
        raise ValueError("the prompt is empty")
    if args.benchmark_prefill_tokens > 0:          # main.cpp:368-376: repeat the last id or cut
        n = args.benchmark_prefill_tokens
        prompt = (prompt + [prompt[-1]] * max(0, n - len(prompt)))[:n]
    if args.tokens_only:
        print(",".join(str(t) for t in prompt))
        return 0

    import torch
    from .engine.engine import Engine
    from .engine.scheduler import EngineOptions, RequestOptions
    from .sampling import SamplingParams
    from .engine.step import StepEntry

    options = EngineOptions(max_active_requests=args.max_active_requests,
                            max_batched_tokens=max(args.max_batched_tokens, 1),
                            prefill_chunk_tokens=args.prefill_chunk, page_tokens=args.page_tokens,
                            logical_kv_pages=args.kv_pages)
    engine = Engine(model_dir, max_context=args.context, dtype=args.dtype, device=args.device, options=options,
                    use_cuda_graph=not args.no_cuda_graph)
    if args.memory_report:
        weights = sum(t.numel() * t.element_size() for t in _model_tensors(engine))
        print(f"memory.weights_bytes={weights}", file=sys.stderr)
        print(f"memory.cache_bytes={engine.loaded.storage.bytes()}", file=sys.stderr)
        print(f"memory.device_allocated_bytes={torch.cuda.memory_allocated(engine.device)}", file=sys.stderr)

    if args.dump_logits or args.print_top > 0:
        # logits of the last prompt token, through the raw step in portions of --prefill-chunk
        logits = None
        for at in range(0, len(prompt), args.prefill_chunk):
            part = prompt[at:at + args.prefill_chunk]
            last = at + len(part) == len(prompt)
            logits = engine.forward([StepEntry("dump", part, [len(part) - 1] if last else [])])
        host = logits[0].to("cpu").numpy().astype("<f4")
        engine.end("dump")
        if args.dump_logits:
            host.tofile(args.dump_logits)
        if args.print_top > 0:
            for token in host.argsort()[::-1][:args.print_top]:
                print(f"top token={int(token)} logit={float(host[token]):.6f}", file=sys.stderr)

    generation = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                                repetition_penalty=args.repetition_penalty, seed=args.seed)
    if args.benchmark_decode > 0:
        return _benchmark(engine, prompt, args, generation)

    request = RequestOptions(max_new_tokens=args.max_new_tokens, generation=generation)
    started = time.perf_counter()
    request_id = engine.submit(prompt, request)
    generated: List[int] = []
    first_token_at = None
    while True:
        engine.step()
        result = engine.poll(request_id)
        if result.tokens and first_token_at is None:
            first_token_at = time.perf_counter()
        for token in result.tokens:
            print(token, end=" ", flush=True)
        generated.extend(result.tokens)
        if result.finished:
            if result.error:
                raise RuntimeError(result.error)
            break
    finished = time.perf_counter()
    print()
    if args.runtime_tokens:
        print("CELEG_GENERATED_TOKEN_IDS=[" + ",".join(str(t) for t in generated) + "]")
    if args.runtime_metrics:
        prefill_s = (first_token_at or finished) - started
        decode_s = finished - (first_token_at or finished)
        decoded = max(len(generated) - 1, 0)
        print(f"runtime.prefill_tokens={len(prompt)}", file=sys.stderr)
        print(f"runtime.prefill_ms={prefill_s * 1e3:.3f}", file=sys.stderr)
        print(f"runtime.prefill_tokens_per_second={len(prompt) / max(prefill_s, 1e-9):.3f}", file=sys.stderr)
        print(f"runtime.decode_tokens={decoded}", file=sys.stderr)
        print(f"runtime.decode_ms={decode_s * 1e3:.3f}", file=sys.stderr)
        print(f"runtime.decode_tokens_per_second={decoded / max(decode_s, 1e-9):.3f}", file=sys.stderr)
        # the engine's own counters (celeg: include/celeg/runtime/concurrency/metrics.hpp:8-58)
        metrics = engine.metrics()
        steps = max(metrics.steps, 1)
        print(f"runtime.scheduler_steps={metrics.steps}", file=sys.stderr)
        print(f"runtime.pages_high_water={metrics.pages_high_water}", file=sys.stderr)
        print(f"runtime.pages_total={metrics.pages_total}", file=sys.stderr)
        print(f"runtime.host_ms_per_step={1e3 * (metrics.host_plan_seconds + metrics.host_launch_seconds + metrics.host_commit_seconds) / steps:.4f}", file=sys.stderr)
        print(f"runtime.gpu_ms_per_step={1e3 * metrics.gpu_seconds / steps:.4f}", file=sys.stderr)
        print(f"runtime.model_fingerprint={engine.loaded.fingerprint}", file=sys.stderr)
    return 0


def _model_tensors(engine):
    return engine.loaded.model.weight_tensors()


def _benchmark(engine, prompt, args, generation) -> int:
    """--benchmark-decode N: time the prefill of the prompt, then N decode steps after
    --benchmark-warmup untimed ones (main.cpp:522-538)."""
    import torch
    from .engine.scheduler import RequestOptions
    total = args.benchmark_warmup + args.benchmark_decode
    request = RequestOptions(max_new_tokens=total + 1, eos_tokens=(), generation=generation)
    request_id = engine.submit(prompt, request)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    produced = 0
    while produced == 0:
        engine.step()
        produced += len(engine.poll(request_id).tokens)
    torch.cuda.synchronize()
    prefill_ms = (time.perf_counter() - t0) * 1e3
    print(f"benchmark.prefill_tokens={len(prompt)}", file=sys.stderr)
    print(f"benchmark.prefill_ms={prefill_ms:.3f}", file=sys.stderr)
    print(f"benchmark.prefill_tokens_per_second={len(prompt) / prefill_ms * 1e3:.3f}", file=sys.stderr)
    for _ in range(args.benchmark_warmup):
        engine.step()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    for _ in range(args.benchmark_decode):
        engine.step()
    torch.cuda.synchronize()
    decode_ms = (time.perf_counter() - t1) * 1e3
    print(f"benchmark.decode_warmup={args.benchmark_warmup}", file=sys.stderr)
    print(f"benchmark.decode_tokens={args.benchmark_decode}", file=sys.stderr)
    print(f"benchmark.decode_ms={decode_ms:.3f}", file=sys.stderr)
    print(f"benchmark.decode_ms_per_token={decode_ms / args.benchmark_decode:.3f}", file=sys.stderr)
    print(f"benchmark.decode_tokens_per_second={args.benchmark_decode / decode_ms * 1e3:.3f}", file=sys.stderr)
    return 0


def main(argv=None) -> int:
    try:
        return run(argv)
    except SystemExit:
        raise
    except Exception as exc:                # main.cpp:601-604: "error: ..." and exit code 1
        print(f"error: {exc}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
