"""Chooses the next token of each row from its logits, on the device.

Order of operations (kairyu/engine/core/sampler.py:1-27): min-tokens mask,
penalties, then argmax when temperature is 0, else temperature, min-p, top-k,
top-p and a seeded Gumbel-max draw.  One kernel launch edits logits (only when
some row needs it) and one selects tokens for all rows.

Rows whose parameters ask for ``logprobs`` get a report from the *raw* logits
(before any edit or temperature, sampler.py:5-6): the log-softmax value of the
chosen token and the k largest with their ids.  It stays on the device until
the caller fetches it (``take_report``), so that it can ride the same
device-to-host read as the sampled ids.
"""

from __future__ import annotations

from collections import Counter
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from kairyu_b200 import kernels
from kairyu_b200.sampling.params import SamplingParams
from kairyu_b200.sampling.rng import as_signed64, mix_seed, stable_request_seed


@dataclass
class SamplingRow:
    """What the sampler needs to know about one row of logits."""

    request_id: str
    params: SamplingParams
    position: int  # index of the output token being chosen
    prompt_token_ids: Sequence[int] = ()
    output_token_ids: Sequence[int] = ()
    eos_token_ids: Sequence[int] = ()

    def base_seed(self) -> int:
        if self.params.seed is not None:
            return self.params.seed & ((1 << 64) - 1)
        return stable_request_seed(self.request_id)


@dataclass
class LogprobReport:
    """Device tensors of one step's report.  ``values[r, 0]``: the chosen token's log-probability of
    report r; ``values[r, 1 + i]`` / ``indices[r, i]``: the i-th largest and its token id."""

    rows: list[int]  # which rows of the step the reports are for
    k: list[int]  # how many of the largest each row asked for
    values: torch.Tensor
    indices: torch.Tensor

    def entries(self, values: Sequence[Sequence[float]], indices: Sequence[Sequence[int]], token_ids: Sequence[int]):
        """Per report (row, {token id: log-probability}, the chosen token's log-probability), from host
        copies of the tensors: the chosen token first, then the largest that are not it
        (kairyu/engine/engine_loop.py:219-234)."""
        for place, (row, k) in enumerate(zip(self.rows, self.k)):
            chosen = float(values[place][0])
            entry = {int(token_ids[row]): chosen}
            for i in range(k):
                if indices[place][i] >= 0:
                    entry.setdefault(int(indices[place][i]), float(values[place][1 + i]))
            yield row, entry, chosen


class Sampler:
    def __init__(self, vocab_size: int, device: str) -> None:
        self.vocab_size = vocab_size
        self.device = device
        self._report: Optional[LogprobReport] = None
        self._work: Optional[torch.Tensor] = None
        self._is_cuda = str(device).startswith("cuda")
        self._staging: Optional[list] = None  # pinned buffers for the rows' parameters
        self._staging_rows = 0
        self._device_words: Optional[torch.Tensor] = None
        self._next_staging = 0

    def _host(self, values: list, dtype: torch.dtype) -> torch.Tensor:
        tensor = torch.tensor(values, dtype=dtype)
        if self._is_cuda:
            tensor = tensor.pin_memory()
        return tensor.to(self.device, non_blocking=True)

    def _edits(self, rows: Sequence[SamplingRow]) -> Optional[tuple[list[int], list[int], list[float], list[float], list[int]]]:
        e_row: list[int] = []
        e_tok: list[int] = []
        e_mul: list[float] = []
        e_sub: list[float] = []
        e_mask: list[int] = []
        for index, row in enumerate(rows):
            p = row.params
            masked: set[int] = set()
            if row.position < p.min_tokens:
                # kairyu/engine/core/sampler.py:666-699: the whole stop set, EOS included
                for token in (*p.stop_token_ids, *row.eos_token_ids):
                    if 0 <= token < self.vocab_size and token not in masked:
                        masked.add(token)
                        e_row.append(index); e_tok.append(token); e_mul.append(1.0); e_sub.append(0.0); e_mask.append(1)
            has_rep = p.repetition_penalty != 1.0
            has_out = p.frequency_penalty != 0.0 or p.presence_penalty != 0.0
            if not (has_rep or has_out):
                continue
            counts = Counter(row.output_token_ids)
            seen = set(counts)
            if has_rep:
                seen |= set(row.prompt_token_ids)
            for token in seen:
                if token in masked or not 0 <= token < self.vocab_size:
                    continue
                count = counts.get(token, 0)
                sub = p.frequency_penalty * count + (p.presence_penalty if count else 0.0)
                e_row.append(index); e_tok.append(token)
                e_mul.append(p.repetition_penalty if has_rep else 1.0)
                e_sub.append(sub); e_mask.append(0)
        if not e_row:
            return None
        return e_row, e_tok, e_mul, e_sub, e_mask

    def sample(self, logits: torch.Tensor, rows: Sequence[SamplingRow], out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``logits``: [n, vocab] fp32 on the device (edited in place when a row
        has penalties or a min-tokens mask).  Returns int32 token ids [n] on the device
        (in ``out`` when given: a persistent buffer the next step can read them from)."""
        n = logits.shape[0]
        if n != len(rows):
            raise ValueError(f"{n} rows of logits for {len(rows)} sampling rows")
        if out is None:
            out = torch.empty(n, dtype=torch.int32, device=self.device)
        elif out.shape != (n,) or out.dtype != torch.int32 or not out.is_contiguous():
            raise ValueError("out must be a contiguous int32 tensor with one element per row")
        edits = self._edits(rows)
        report_rows = [index for index, row in enumerate(rows) if row.params.logprobs is not None]
        raw = logits
        if report_rows and edits is not None:
            raw = logits.clone()  # the report is of the logits as the model gave them
        if edits is not None:
            e_row, e_tok, e_mul, e_sub, e_mask = edits
            kernels.edit_logits(
                logits,
                self._host(e_row, torch.int32),
                self._host(e_tok, torch.int32),
                self._host(e_mul, torch.float32),
                self._host(e_sub, torch.float32),
                self._host(e_mask, torch.int32),
            )
        if all(row.params.temperature == 0.0 for row in rows):
            kernels.argmax(logits, out)
        else:
            needed = kernels.sample_work_floats(n, self.vocab_size)
            if self._work is None or self._work.numel() < needed:
                self._work = torch.empty(max(needed, kernels.sample_work_floats(8, self.vocab_size)), dtype=torch.float32, device=self.device)
            temperature, top_k, top_p, min_p, seeds = self._row_parameters(rows)
            kernels.sample(logits, self._work, temperature, top_k, top_p, min_p, seeds, out)
        self._report = self._make_report(raw, rows, report_rows, out) if report_rows else None
        return out

    def _make_report(self, raw: torch.Tensor, rows: Sequence[SamplingRow], report_rows: list[int], out: torch.Tensor) -> LogprobReport:
        wanted = [min(max(int(rows[index].params.logprobs), 0), self.vocab_size) for index in report_rows]
        k = max(wanted)
        values = torch.empty((len(report_rows), k + 1), dtype=torch.float32, device=self.device)
        indices = torch.empty((len(report_rows), k), dtype=torch.int32, device=self.device)
        kernels.logprob_report(raw, self._host(report_rows, torch.int32), out, k, values, indices, tokens_by_row=True)
        return LogprobReport(report_rows, wanted, values, indices)

    def take_report(self) -> Optional[LogprobReport]:
        """The report of the last ``sample`` call (None when no row asked for one)."""
        report, self._report = self._report, None
        return report

    def _row_parameters(self, rows: Sequence[SamplingRow]) -> tuple[torch.Tensor, ...]:
        """The rows' parameters on the device: packed into one pinned buffer (a ring of four, so that
        the copy of one step may still be in flight while the next is packed) and sent in one copy."""
        n = len(rows)
        seeds = [as_signed64(mix_seed(row.base_seed(), row.position)) for row in rows]
        if not self._is_cuda:
            return (
                torch.tensor([float(row.params.temperature) for row in rows], dtype=torch.float32),
                torch.tensor([int(row.params.top_k) for row in rows], dtype=torch.int32),
                torch.tensor([float(row.params.top_p) for row in rows], dtype=torch.float32),
                torch.tensor([float(row.params.min_p) for row in rows], dtype=torch.float32),
                torch.tensor(seeds, dtype=torch.int64),
            )
        if self._staging is None or self._staging_rows < n:
            self._staging_rows = max(n, 64)
            words = 6 * self._staging_rows  # seeds (two 32-bit words a row) first: 8-byte aligned
            self._staging = []
            for _ in range(4):
                pinned = torch.empty(words, dtype=torch.int32, pin_memory=True)
                words32 = pinned.numpy()  # numpy views of the pinned words: filling them costs a fifth of what tensor slices do
                self._staging.append((pinned, torch.cuda.Event(), words32, words32.view(np.float32), words32[: 2 * self._staging_rows].view(np.int64)))
            self._device_words = torch.empty(words, dtype=torch.int32, device=self.device)
            self._next_staging = 0
        host, event, as_int, as_float, as_long = self._staging[self._next_staging]
        self._next_staging = (self._next_staging + 1) % len(self._staging)
        event.synchronize()  # the copy that last used this buffer has run
        cap = self._staging_rows
        as_long[:n] = seeds
        as_float[2 * cap : 2 * cap + n] = [row.params.temperature for row in rows]
        as_int[3 * cap : 3 * cap + n] = [min(row.params.top_k, 0x7FFFFFFF) for row in rows]  # beyond the vocabulary either way
        as_float[4 * cap : 4 * cap + n] = [row.params.top_p for row in rows]
        as_float[5 * cap : 5 * cap + n] = [row.params.min_p for row in rows]
        device = self._device_words
        device.copy_(host, non_blocking=True)
        event.record()
        device_float = device.view(torch.float32)
        return (
            device_float[2 * cap : 2 * cap + n],
            device[3 * cap : 3 * cap + n],
            device_float[4 * cap : 4 * cap + n],
            device_float[5 * cap : 5 * cap + n],
            device[: 2 * n].view(torch.int64),
        )
