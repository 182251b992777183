"""Helpers shared by the replay tests: traces with many live rows, traces whose wants are thinned
to chosen positions, the plain model run in bfloat16 arithmetic (what rounding alone costs), and
comparisons that name the rows that are off."""

from __future__ import annotations

from typing import Mapping, Sequence

import numpy as np
import torch

import plain_model


def keep_positions(length: int, spread: int = 9, tail: int = 12) -> list[int]:
    """The first three positions, ``spread`` positions over the middle and the last ``tail``."""
    chosen = set(range(min(3, length))) | set(range(max(0, length - tail), length))
    chosen |= {int(round(i * (length - 1) / (spread + 1))) for i in range(1, spread + 1)}
    return sorted(chosen)


def thin_wants(steps: Sequence[dict], keep: Mapping[str, Sequence[int]]) -> list[dict]:
    """The same steps, asking only for the positions in ``keep`` (absolute, per request)."""
    offset: dict[str, int] = {}
    thinned = []
    for step in steps:
        entries = []
        for entry in step["entries"]:
            start = offset.get(entry["id"], 0)
            wanted = set(keep[entry["id"]])
            entries.append(dict(entry, want=[place for place in entry["want"] if start + place in wanted]))
            offset[entry["id"]] = start + len(entry["tokens"])
        thinned.append(dict(step, entries=entries))
    return thinned


def trace_many_rows(requests: Mapping[str, list[int]], tail: int, per_prefill_step: int = 6) -> list[dict]:
    """All requests live at once: their heads in steps of ``per_prefill_step`` requests each, then
    ``tail`` steps in which every request brings one token (its logits wanted), then the end."""
    names = list(requests)
    steps: list[dict] = []
    for start in range(0, len(names), per_prefill_step):
        group = names[start : start + per_prefill_step]
        steps.append({
            "step": len(steps),
            "entries": [{"id": n, "tokens": requests[n][: len(requests[n]) - tail], "want": [len(requests[n]) - tail - 1]} for n in group],
            "end": [],
        })
    for index in range(tail):
        last = index == tail - 1
        steps.append({
            "step": len(steps),
            "entries": [{"id": n, "tokens": [requests[n][len(requests[n]) - tail + index]], "want": [0]} for n in names],
            "end": names if last else [],
        })
    return steps


def in_bf16(weights: Mapping[str, torch.Tensor], keep_norms_in_fp32: bool) -> dict[str, torch.Tensor]:
    held = {}
    for name, tensor in weights.items():
        keep = keep_norms_in_fp32 and tensor.ndim == 1 and name.endswith("norm.weight")
        held[name] = tensor if keep else tensor.to(torch.bfloat16)
    return held


def plain_rows(config, weights, requests, keep=None) -> dict[tuple[str, int], np.ndarray]:
    """(request, position) -> logits row of the plain model, whole sequences, on the weights' device."""
    rows = {}
    for name, tokens in requests.items():
        logits = plain_model.forward_logits(config, weights, tokens).float()
        positions = range(len(tokens)) if keep is None else keep[name]
        picked = logits[list(positions)].cpu().numpy()
        for index, position in enumerate(positions):
            rows[(name, position)] = picked[index]
    return rows


def worst_error(result: Mapping, expected: Mapping) -> float:
    return max(float(np.abs(row - expected[key]).max()) for key, row in result.items())


def rows_beyond(result: Mapping, expected: Mapping, bound: float, limit: int = 12) -> list:
    """For a failure's message: (request, position, error) of the rows beyond the bound."""
    errors = [(key[0], key[1], float(np.abs(row - expected[key]).max())) for key, row in result.items()]
    return [entry for entry in errors if not entry[2] < bound][:limit]


def assert_same_bits(first: Mapping, second: Mapping, what: str) -> None:
    assert first.keys() == second.keys(), what
    different = [key for key in first if not np.array_equal(first[key], second[key])]
    assert not different, (what, different[:12])
