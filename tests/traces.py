"""Builds replay traces (the JSON steps ``bin/trace_run`` reads) that cut the
same requests in different ways, runs them in process or through the program,
and collects the logits by (request, position)."""

from __future__ import annotations

import json
import random
import subprocess
import sys
from pathlib import Path
from typing import Callable, Mapping, Sequence

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent


def make_requests(vocab: int, lengths: Sequence[int], seed: int) -> dict[str, list[int]]:
    generator = torch.Generator().manual_seed(seed)
    return {
        f"r{index}": torch.randint(0, vocab, (length,), generator=generator).tolist()
        for index, length in enumerate(lengths)
    }


def trace_whole(requests: Mapping[str, list[int]]) -> list[dict]:
    """Each request alone and whole, logits at every position."""
    steps = []
    for name, tokens in requests.items():
        steps.append(
            {"step": len(steps), "entries": [{"id": name, "tokens": tokens, "want": list(range(len(tokens)))}], "end": [name]}
        )
    return steps


def trace_decode_tail(requests: Mapping[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for name, tokens in requests.items():
        head = max(len(tokens) - tail, 1)
        steps.append({"step": len(steps), "entries": [{"id": name, "tokens": tokens[:head], "want": list(range(head))}], "end": []})
        for index in range(head, len(tokens)):
            last = index == len(tokens) - 1
            steps.append(
                {"step": len(steps), "entries": [{"id": name, "tokens": [tokens[index]], "want": [0]}], "end": [name] if last else []}
            )
    return steps


def trace_chunks(requests: Mapping[str, list[int]], sizes: Sequence[int] = (24, 7, 2, 13, 3, 64, 2, 5)) -> list[dict]:
    """Portions of changing size, down to two tokens."""
    steps = []
    for name, tokens in requests.items():
        start = 0
        turn = 0
        while start < len(tokens):
            size = min(sizes[turn % len(sizes)], len(tokens) - start)
            turn += 1
            portion = tokens[start : start + size]
            done = start + size == len(tokens)
            steps.append(
                {"step": len(steps), "entries": [{"id": name, "tokens": portion, "want": list(range(size))}], "end": [name] if done else []}
            )
            start += size
    return steps


def trace_mixed(requests: Mapping[str, list[int]], seed: int, max_live: int = 4, skip_chance: float = 0.2) -> list[dict]:
    """Up to ``max_live`` requests at a time: portions of some beside single
    tokens of others, some left out of a step now and then; a request that ends
    frees its pages for the next one to start."""
    rng = random.Random(seed)
    pending = list(requests.items())
    live: dict[str, int] = {}
    steps: list[dict] = []
    while pending or live:
        while pending and len(live) < max_live:
            name, _ = pending.pop(0)
            live[name] = 0
        entries = []
        ended = []
        for name in list(live):
            if len(live) > 1 and rng.random() < skip_chance:
                continue
            tokens = requests[name]
            start = live[name]
            left = len(tokens) - start
            # late in a request behave like decoding: one token at a time
            if left <= 8 or rng.random() < 0.3:
                size = 1
            else:
                size = min(left, rng.choice([2, 3, 5, 9, 16, 17, 31, 40]))
            portion = tokens[start : start + size]
            entries.append({"id": name, "tokens": portion, "want": list(range(size))})
            live[name] = start + size
            if live[name] == len(tokens):
                ended.append(name)
        if not entries:
            continue
        for name in ended:
            del live[name]
        steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def peak_tokens(steps: Sequence[dict], round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held: dict[str, int] = {}
    peak = 0
    for step in steps:
        for entry in step["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        peak = max(peak, sum(-(-count // round_to) * round_to for count in held.values()))
        for name in step["end"]:
            held.pop(name, None)
    return peak


def collect(steps: Sequence[dict], logits_of_step: Callable[[int], np.ndarray | None]) -> dict[tuple[str, int], np.ndarray]:
    """(request, position) -> logits row, from per-step arrays."""
    offset: dict[str, int] = {}
    result: dict[tuple[str, int], np.ndarray] = {}
    for step in steps:
        wanted = sum(len(entry["want"]) for entry in step["entries"])
        array = logits_of_step(step["step"]) if wanted else None
        row = 0
        for entry in step["entries"]:
            start = offset.get(entry["id"], 0)
            for place in entry["want"]:
                result[(entry["id"], start + place)] = array[row]
                row += 1
            offset[entry["id"]] = start + len(entry["tokens"])
        if wanted:
            assert row == array.shape[0]
    return result


def run_in_process(runner, steps: Sequence[dict]) -> dict[tuple[str, int], np.ndarray]:
    """Drive a ModelRunner the way ``bin/trace_run`` does."""
    from kairyu_b200.engine.runner import StepEntry

    arrays: dict[int, np.ndarray] = {}
    for step in steps:
        entries = [StepEntry(e["id"], e["tokens"], tuple(e["want"])) for e in step["entries"]]
        logits = runner.step(entries)
        if logits is not None:
            arrays[step["step"]] = logits.float().cpu().numpy().copy()
        runner.check_errors()
        for name in step["end"]:
            runner.cache.release(name)
        runner.cache.check()
    return collect(steps, lambda index: arrays.get(index))


def run_program(model_dir: Path, out_dir: Path, steps: Sequence[dict], *, dtype: str, max_tokens: int, vocab: int, extra: Sequence[str] = ()) -> dict[tuple[str, int], np.ndarray]:
    """Run ``bin/trace_run`` as a subprocess, one step at a time."""
    command = [
        sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
        "--out", str(out_dir), "--max-tokens", str(max_tokens), *extra,
    ]
    process = subprocess.Popen(command, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for step in steps:
            process.stdin.write(json.dumps(step) + "\n")
            process.stdin.flush()
            line = process.stdout.readline().strip()
            assert line == f"done {step['step']}", f"expected 'done {step['step']}', got {line!r}"
        process.stdin.close()
        assert process.wait(timeout=120) == 0
    finally:
        if process.poll() is None:
            process.kill()

    def load(index: int) -> np.ndarray:
        return np.fromfile(out_dir / f"{index}.f32", dtype="<f4").reshape(-1, vocab)

    return collect(steps, load)
