"""Trace replay: feeds given token ids through a model step by step and writes
logits.  It samples nothing and has no forward pass, cache or loader of its
own: it drives the engine's model, step function, cache manager and kernels.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come on standard input, one JSON object a line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: per request its next tokens and the places among them whose logits
are wanted.  All entries of a step run as one batch.  ``end``: requests that
are finished after the step; their pages go back to the pool.  For a step that
wants something ``<out>/<step>.f32`` is written: little-endian fp32
``[wanted, vocab]`` in the order of the entries and of ``want``.  After each
step ``done <step>`` is printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path
from typing import Optional, Sequence


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder the logits files are written to")
    parser.add_argument("--max-tokens", type=int, required=True, help="tokens the cache pool is made for")
    parser.add_argument("--page-size", type=int, default=16)
    parser.add_argument("--max-requests", type=int, default=16, help="live requests at a time")
    parser.add_argument("--decode-mode", choices=["eager", "cuda_graph"], default=None)
    parser.add_argument("--device", default="cuda")
    return parser


def main(argv: Optional[Sequence[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    import torch

    from kairyu_b200.cache.manager import CacheLayout, CacheManager
    from kairyu_b200.cache.storage import CacheStorage
    from kairyu_b200.engine.engine import load_model
    from kairyu_b200.engine.runner import ModelRunner, StepEntry

    if args.max_tokens < 1:
        print("trace_run: --max-tokens must be positive", file=sys.stderr)
        return 2
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    if args.device.startswith("cuda") and not torch.cuda.is_available():
        print("trace_run: no CUDA device is available; this engine has no CPU path", file=sys.stderr)
        return 3
    if args.dtype == "float32":
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
    model, model_config = load_model(args.model, dtype=args.dtype, device=args.device)
    layout = CacheLayout.from_slot_specs(model.cache_slot_specs())
    num_pages = -(-args.max_tokens // args.page_size) + 1  # + the reserved padding page
    cache = CacheManager(layout, num_pages=num_pages, page_size=args.page_size, max_requests=args.max_requests)
    storage = CacheStorage(
        layout,
        num_pages=num_pages,
        page_size=args.page_size,
        max_requests=args.max_requests,
        dtype=model.dtype,
        device=args.device,
    )
    decode_mode = args.decode_mode or ("cuda_graph" if args.device.startswith("cuda") else "eager")
    runner = ModelRunner(
        model,
        cache,
        storage,
        max_model_len=model.spec.max_position_embeddings,
        decode_mode=decode_mode,
        max_graph_batch=args.max_requests,
    )
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = [
            StepEntry(entry["id"], [int(t) for t in entry["tokens"]], tuple(int(w) for w in entry.get("want", ())))
            for entry in record.get("entries", ())
        ]
        if entries:
            logits = runner.step(entries)
            if logits is not None:
                array = logits.to(torch.float32).cpu().numpy().astype("<f4", copy=False)
                array.tofile(out_dir / f"{step}.f32")
            runner.check_errors()
        for request_id in record.get("end", ()):
            if request_id in cache:
                cache.release(request_id)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
