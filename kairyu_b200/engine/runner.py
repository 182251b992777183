"""The step function: one batch of (request, its next tokens) through the model.

A step runs only the tokens it is given, against the cache earlier steps left,
and returns fp32 logits at the wanted positions.  Rows may be portions of
prompts of any length beside single decoded tokens; a row's tokens continue at
the request's computed length (kairyu/engine/core/prefill.py:17-43 and
kairyu/engine/core/model_runner.py:1833-1962 are the reference's equivalents).

The step's metadata is packed into one pinned int32 buffer and copied to the
device once.  Steps whose rows all carry one token can be replayed from a CUDA
graph captured per (padded batch size, context-length bucket), as
kairyu/engine/core/step_executor.py:591-934 does with its buckets.
"""

from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Any, Hashable, Optional, Sequence

import numpy as np
import torch

from kairyu_b200 import kernels
from kairyu_b200.cache.manager import CacheManager
from kairyu_b200.cache.page_pool import OutOfPages
from kairyu_b200.cache.storage import CacheStorage
from kairyu_b200.engine.workspace import Workspace
from kairyu_b200.parts.base import CacheView, StepContext


@dataclass
class StepEntry:
    """One request's share of a step."""

    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()  # places among ``tokens`` whose logits are wanted
    # The single token of this entry is not known to the host yet: it is element ``future`` of the
    # device tensor of sampled ids given to ``step`` (``tokens`` then holds one placeholder).
    future: Optional[int] = None


class StepError(RuntimeError):
    pass


PORTION_PAD = 16           # a captured step's tokens are padded to a multiple of this (of the page size, if that is smaller)
MAX_PORTION_GRAPHS = 64    # captured shapes of steps kept; the least recently used goes first
PORTION_EVICT_AFTER = 256  # a kept shape gives way to a new one only if it has not come for this many steps
PORTION_CAPTURE_AT = 3     # a shape of step is captured when it comes for this many-th time (a capture costs a dozen replays' gain)


def context_bucket(max_seq_len: int) -> int:
    """Context length a captured decode graph is sized for: the next multiple of an eighth of
    the enclosing power of two (at least 256).  The attention grid of a graph has one block per
    128 keys of this length, so a coarser bucket launches blocks that find nothing to do, and a
    finer one captures more graphs."""
    power = 256
    while power < max_seq_len:
        power *= 2
    step = max(256, power // 8)
    return max(256, -(-max_seq_len // step) * step)


def decode_buckets(max_batch: int) -> list[int]:
    """Padded batch sizes graphs are captured for: 1, 2, 4, 8, 16, 24, 32, then
    every 8 (kairyu/engine/core/graph_buckets.py:9-28)."""
    sizes = [size for size in (1, 2, 4, 8) if size <= max_batch]
    sizes += list(range(16, max_batch + 1, 8))
    if not sizes or sizes[-1] < max_batch:
        sizes.append(max_batch)
    return sizes


@dataclass
class _Graph:
    graph: Any
    meta: torch.Tensor  # static device int32 buffer the graph reads
    logits: torch.Tensor
    generation: int
    layout: dict[str, tuple[int, int]]
    launches: int = 0  # kernels of this package inside the graph
    keepalive: tuple = ()  # tensors the captured kernels read; freeing them would hand their memory to others
    # Host side of the static metadata: an authoritative mirror that is updated in place from
    # step to step (a decode step changes a token, a position and now and then one page per
    # row), which request sits in which row, and a ring of pinned staging buffers so that the
    # copy of step N may still be in flight while step N+1 is prepared.
    mirror: Any = None
    row_state: list = field(default_factory=list)
    staging: list = field(default_factory=list)
    next_staging: int = 0
    last_used: int = 0  # the step that last replayed it (captured steps of prompt portions)


class ModelRunner:
    def __init__(
        self,
        model: Any,
        cache: CacheManager,
        storage: CacheStorage,
        *,
        max_model_len: int,
        decode_mode: str = "eager",
        max_graph_batch: int = 256,
        debug_poison: bool = False,
        check_tables: bool = False,
        portion_graphs: Optional[bool] = None,
        portion_graph_max_tokens: int = 256,
    ) -> None:
        self.model = model
        self.cache = cache
        self.storage = storage
        self.device = model.device
        self.max_model_len = max_model_len
        self.max_pages_per_request = -(-max_model_len // cache.page_size)
        self.decode_mode = decode_mode
        self.max_graph_batch = max_graph_batch
        # Debug aid: pages that were given back since the last step are overwritten with a large
        # finite value before the next one runs, so that a kernel that reads a page its request no
        # longer (or not yet) holds gives logits far off, while keys that are read and masked,
        # as the unwritten tail of a request's last page is, change nothing.
        self.debug_poison = debug_poison
        if debug_poison:
            cache.log_freed_pages = True
        # Per step, on the host: every page a row needs is there, and no page is named twice, in one
        # row or in two, except shared prefix pages, which no row may write
        # (kairyu/engine/core/prefill.py:105-178).  The cache manager guarantees this by
        # construction; the check costs a pass over the tables, so tests turn it on.
        self.check_tables = check_tables
        self.workspace = Workspace(self.device)
        self.graph_workspace = Workspace(self.device)
        self._is_cuda = str(self.device).startswith("cuda")
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        # query-tile sizes the model's mixers want listed with every step (each names its own)
        self._tile_sizes = tuple(sorted({
            int(size) for block in getattr(model, "blocks", ()) for size in getattr(getattr(block, "mixer", None), "query_tile_sizes", lambda: ())()
        }))
        self._views: dict[tuple[int, bool], CacheView] = {}
        for call in model.schedule:
            key = (call.cache_slot, call.writes_cache)
            if key not in self._views:
                self._views[key] = storage.view(call.cache_slot, writes=call.writes_cache)
        self._graphs: dict[tuple[int, int], _Graph] = {}
        self._graph_pool = None
        self._buckets = decode_buckets(max_graph_batch)
        # Steps that hold prompt portions of up to a few hundred tokens are captured too, once the same shape
        # of step has come for the third time: such a step's launches take the host longer (4 ms for 32
        # layers) than the device takes to run them, while a larger step keeps the device busy for longer
        # than the host needs, and a capture (the step once more, and a wait for the device) would only cost.  What a captured step takes from
        # the host is its shape alone: tokens (padded to a multiple of 16 with a filler row on the reserved
        # page), rows, tiles, single-token rows, wanted places, context bucket; everything else is in the
        # device-side description, which is copied before every replay.
        safe = getattr(model, "graph_safe", None)
        capable = self._is_cuda and decode_mode == "cuda_graph" and bool(safe and safe())
        self._portion_pad = min(PORTION_PAD, cache.page_size)  # the filler row lies on the one reserved page
        self.portion_graphs = capable if portion_graphs is None else (bool(portion_graphs) and capable)
        self.portion_graph_max_tokens = portion_graph_max_tokens
        self.portion_workspace = Workspace(self.device, min_rows=portion_graph_max_tokens + PORTION_PAD)
        self._portion_graphs: "OrderedDict[tuple, _Graph]" = OrderedDict()
        self._portion_seen: dict[tuple, int] = {}
        self.counters = {
            "steps": 0, "graph_replays": 0, "graph_captures": 0, "eager_steps": 0, "tokens": 0, "kernel_launches": 0,
            "future_tokens": 0,  # tokens taken from the device because the host had not seen them yet
            "portion_graph_captures": 0, "portion_graph_replays": 0,
        }

    # ------------------------------------------------------------------ host-side packing
    def _prepare_rows(self, entries: Sequence[StepEntry]) -> list[tuple[StepEntry, int, int]]:
        """Checks and page growth; returns (entry, start, seq_len) per row."""
        if not entries:
            raise StepError("a step needs at least one entry")
        seen: set[Hashable] = set()
        rows = []
        vocab = self.model.spec.vocab_size
        for entry in entries:
            if entry.request_id in seen:
                raise StepError(f"request {entry.request_id!r} appears twice in one step")
            seen.add(entry.request_id)
            count = len(entry.tokens)
            if count < 1:
                raise StepError(f"request {entry.request_id!r} brings no tokens")
            if min(entry.tokens) < 0 or max(entry.tokens) >= vocab:
                raise StepError(f"request {entry.request_id!r} has a token id outside [0, {vocab})")
            if any(not 0 <= place < count for place in entry.want):
                raise StepError(f"request {entry.request_id!r} wants a place outside its tokens")
            if entry.future is not None and count != 1:
                raise StepError(f"request {entry.request_id!r}: only a single token can come from the device")
            if entry.request_id not in self.cache:
                self.cache.admit(entry.request_id)
            start = self.cache.get(entry.request_id).num_tokens
            seq_len = start + count
            if seq_len > self.max_model_len:
                raise StepError(
                    f"request {entry.request_id!r} would reach {seq_len} tokens; max_model_len is {self.max_model_len}"
                )
            if not self.cache.ensure_capacity(entry.request_id, seq_len, query_start=start):
                raise OutOfPages(
                    f"no pages left for request {entry.request_id!r} to reach {seq_len} tokens"
                )
            rows.append((entry, start, seq_len))
        if self.check_tables:
            self._check_tables(rows)
        return rows

    def _check_tables(self, rows: Sequence[tuple[StepEntry, int, int]]) -> None:
        page_size = self.cache.page_size
        for group in self.cache.layout.groups:
            owner: dict[int, Hashable] = {}
            for entry, start, seq_len in rows:
                table = self.cache.block_table(entry.request_id, group.index)
                shared = len(self.cache.get(entry.request_id).shared)
                if start < shared * page_size:
                    raise StepError(f"request {entry.request_id!r} would write position {start}, which lies in a shared page")
                needed = -(-seq_len // page_size)
                if len(table) < needed:
                    raise StepError(f"request {entry.request_id!r} has {len(table)} pages in group {group.index}, {needed} are needed")
                first = 0
                if group.spec.window is not None:  # pages the window has passed may be gone
                    first = max(0, (seq_len - len(entry.tokens) + 1 - group.spec.window)) // page_size
                for index in range(first, needed):
                    page = table[index]
                    if page <= 0 or page >= self.cache.num_pages:
                        raise StepError(f"request {entry.request_id!r}: page {page} at place {index} of group {group.index} is not a page a request can hold")
                    if index < shared:
                        if owner.setdefault(page, "the prefix tree") != "the prefix tree":
                            raise StepError(f"page {page} of group {group.index} is shared and also held by {owner[page]!r}")
                        continue
                    if page in owner:
                        raise StepError(f"page {page} of group {group.index} is named by {owner[page]!r} and by {entry.request_id!r}")
                    owner[page] = entry.request_id

    def _pack(
        self,
        rows: Sequence[tuple[StepEntry, int, int]],
        *,
        pad_rows: Optional[int] = None,
        max_pages: Optional[int] = None,
        include_want: bool = True,
        pad_portion: int = 0,
    ) -> tuple[torch.Tensor, dict[str, tuple[int, int]], dict[str, Any]]:
        """One int32 host tensor holding every index array of the step, the
        (offset, length) of each array, and host-side facts."""
        page_size = self.cache.page_size
        groups = self.cache.layout.groups
        num_rows = len(rows)
        padded_rows = pad_rows if pad_rows is not None else num_rows
        if pad_portion:  # one more row of that many tokens at positions 0.. of the reserved page (a captured step's filler)
            padded_rows += 1
        # The per-token arrays are filled as numpy slices (a 2,048-token portion is four slice
        # assignments, not 8,192 list items); the per-row and per-tile arrays are short lists.
        num_tokens = sum(len(entry.tokens) for entry, _, _ in rows) + (padded_rows - num_rows) + max(pad_portion - 1, 0)
        token_ids = np.zeros(num_tokens, dtype=np.int32)
        future_src = np.full(num_tokens, -1, dtype=np.int32)
        positions = np.zeros(num_tokens, dtype=np.int32)
        row_ids = np.zeros(num_tokens, dtype=np.int32)
        qo_indptr = [0]
        seq_lens: list[int] = []
        write_from: list[int] = []
        state_slots: list[int] = []
        want: list[int] = []
        tile_rows: dict[int, list[int]] = {size: [] for size in self._tile_sizes}
        tile_starts: dict[int, list[int]] = {size: [] for size in self._tile_sizes}
        decode_rows: list[int] = []
        decode_tokens: list[int] = []
        base = 0
        for row, (entry, start, seq_len) in enumerate(rows):
            count = len(entry.tokens)
            token_ids[base : base + count] = entry.tokens
            if entry.future is not None:
                future_src[base] = entry.future
            positions[base : base + count] = np.arange(start, seq_len, dtype=np.int32)
            row_ids[base : base + count] = row
            qo_indptr.append(base + count)
            seq_lens.append(seq_len)
            record = self.cache.get(entry.request_id)
            # positions below this lie in pages the request only reads (its shared prefix): the
            # kernels that write keys and values skip them, whatever the step's tokens say
            write_from.append(len(record.shared) * page_size)
            state_slots.append(record.state_slot)
            if include_want:
                want.extend(base + place for place in entry.want)
            if count == 1:
                decode_rows.append(row)
                decode_tokens.append(base)
            else:
                for size in self._tile_sizes:
                    starts = range(0, count, size)
                    tile_rows[size].extend([row] * len(starts))
                    tile_starts[size].extend(starts)
            base += count
        for row in range(num_rows, padded_rows):  # padding rows of a replayed graph: token 0 at position 0
            count = pad_portion if pad_portion and row == padded_rows - 1 else 1
            row_ids[base : base + count] = row
            positions[base : base + count] = np.arange(count, dtype=np.int32)
            qo_indptr.append(base + count)
            seq_lens.append(count)
            write_from.append(0)
            state_slots.append(self.cache.scratch_state_slot)
            if count == 1:
                decode_rows.append(row)
                decode_tokens.append(base)
            else:
                for size in self._tile_sizes:
                    starts = range(0, count, size)
                    tile_rows[size].extend([row] * len(starts))
                    tile_starts[size].extend(starts)
            base += count
        needed_pages = max((-(-seq_len // page_size) for _, _, seq_len in rows), default=1)
        table_width = max_pages if max_pages is not None else needed_pages
        tables = np.full((len(groups), padded_rows, table_width), -1, dtype=np.int32)
        for place, group in enumerate(groups):
            for row, (entry, _, seq_len) in enumerate(rows):
                pages = self.cache.block_table(entry.request_id, group.index)[: -(-seq_len // page_size)]
                tables[place, row, : len(pages)] = pages
            tables[place, num_rows:, :] = 0  # the reserved page
        arrays = {
            "token_ids": token_ids,
            "future_src": future_src,
            "positions": positions,
            "row_ids": row_ids,
            "qo_indptr": qo_indptr,
            "seq_lens": seq_lens,
            "write_from": write_from,
            "state_slots": state_slots,
            "want": want,
            **{f"tile_rows{size}": tile_rows[size] for size in self._tile_sizes},
            **{f"tile_starts{size}": tile_starts[size] for size in self._tile_sizes},
            "decode_rows": decode_rows,
            "decode_tokens": decode_tokens,
            "tables": tables.reshape(-1),
        }
        layout: dict[str, tuple[int, int]] = {}
        total = 0
        for name, values in arrays.items():
            layout[name] = (total, len(values))
            total += len(values)
        host = torch.empty(total, dtype=torch.int32, pin_memory=self._is_cuda)
        flat = host.numpy()
        for name, values in arrays.items():
            offset, length = layout[name]
            if length:
                flat[offset : offset + length] = values
        facts = {
            "num_tokens": num_tokens,
            "num_rows": padded_rows,
            "table_width": table_width,
            "max_seq_len": max(seq_lens),
            "max_portion_seq_len": max((seq_len for (entry, _, seq_len) in rows if len(entry.tokens) > 1), default=0),
            "host_qo_indptr": tuple(qo_indptr),
            "host_seq_lens": tuple(seq_lens),
        }
        return host, layout, facts

    def _context(
        self,
        meta: torch.Tensor,
        layout: dict[str, tuple[int, int]],
        facts: dict[str, Any],
        workspace: Workspace,
    ) -> tuple[StepContext, Optional[torch.Tensor]]:
        def part(name: str) -> torch.Tensor:
            offset, length = layout[name]
            return meta[offset : offset + length]

        num_rows = facts["num_rows"]
        width = facts["table_width"]
        tables = part("tables").view(len(self.cache.layout.groups), num_rows, width)
        ctx = StepContext(
            num_tokens=facts["num_tokens"],
            num_rows=num_rows,
            dtype=self.model.dtype,
            token_ids=part("token_ids"),
            positions=part("positions"),
            row_ids=part("row_ids"),
            qo_indptr=part("qo_indptr"),
            seq_lens=part("seq_lens"),
            write_from=part("write_from"),
            state_slots=part("state_slots"),
            block_tables={group.index: tables[group.index] for group in self.cache.layout.groups},
            host_qo_indptr=facts["host_qo_indptr"],
            host_seq_lens=facts["host_seq_lens"],
            tiles={
                size: (layout[f"tile_rows{size}"][1], part(f"tile_rows{size}"), part(f"tile_starts{size}"))
                for size in self._tile_sizes
            },
            num_decode_rows=layout["decode_rows"][1],
            decode_rows=part("decode_rows"),
            decode_tokens=part("decode_tokens"),
            max_seq_len=facts["max_seq_len"],
            max_portion_seq_len=facts["max_portion_seq_len"],
            workspace=workspace,
            error_flag=self.error_flag,
        )
        want = part("want") if layout["want"][1] else None
        return ctx, want

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry], sampled: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run one batch; returns ``[wanted, vocab]`` fp32 logits on the device,
        in the order of the entries and of their ``want`` lists, or None.
        ``sampled``: device int32 ids that entries with ``future`` set take their token from."""
        rows = self._prepare_rows(entries)
        has_future = any(entry.future is not None for entry in entries)
        if has_future and sampled is None:
            raise StepError("an entry takes its token from the device, but no tensor of sampled ids was given")
        if not has_future:
            sampled = None
        else:
            self.counters["future_tokens"] += sum(1 for entry in entries if entry.future is not None)
        self.storage.zero_state_slots(self.cache.take_fresh_state_slots())
        if self.debug_poison:
            for group, pages in enumerate(self.cache.take_freed_pages()):
                # a page that was handed out again since has not been written yet either
                self.storage.poison_pages(group, pages, value=3.0e4)
        self.counters["steps"] += 1
        self.counters["tokens"] += sum(len(entry.tokens) for entry, _, _ in rows)
        pure_decode = all(len(entry.tokens) == 1 for entry, _, _ in rows)
        if (
            pure_decode
            and self.decode_mode == "cuda_graph"
            and self._is_cuda
            and len(rows) <= self.max_graph_batch
        ):
            logits = self._graph_step(rows, sampled)
        elif self.portion_graphs and sum(len(entry.tokens) for entry, _, _ in rows) <= self.portion_graph_max_tokens:
            logits = self._portion_step(rows, sampled)
        else:
            logits = self._eager_step(rows, sampled)
        for entry, _, seq_len in rows:
            self.cache.advance(entry.request_id, seq_len)
        return logits

    def _patch_tokens(self, meta: torch.Tensor, layout: dict[str, tuple[int, int]], sampled: Optional[torch.Tensor]) -> None:
        if sampled is None:
            return
        offset, length = layout["token_ids"]
        source_at, _ = layout["future_src"]
        kernels.patch_tokens(meta[offset : offset + length], meta[source_at : source_at + length], sampled, self.error_flag)

    def _eager_step(self, rows: Sequence[tuple[StepEntry, int, int]], sampled: Optional[torch.Tensor] = None,
                    as_captured: Optional[tuple[int, int, int]] = None) -> Optional[torch.Tensor]:
        """``as_captured`` = (filler tokens, context bucket, table width): launch the step exactly as a graph
        of its shape would run it (same filler row, same bounds), so that the first time a shape comes and
        every later time give the same bits."""
        if as_captured is None:
            host, layout, facts = self._pack(rows)
        else:
            pad, bucket, width = as_captured
            host, layout, facts = self._pack(rows, pad_portion=pad, max_pages=width)
            facts["max_seq_len"] = bucket
            if facts["max_portion_seq_len"]:
                facts["max_portion_seq_len"] = bucket
        meta = self.workspace.flat("meta", host.numel(), torch.int32)
        meta.copy_(host, non_blocking=True)
        self._patch_tokens(meta, layout, sampled)
        ctx, want = self._context(meta, layout, facts, self.workspace)
        self.counters["eager_steps"] += 1
        before = kernels.launch_count
        logits = self.model.forward(ctx, self._views, want)
        self.counters["kernel_launches"] += kernels.launch_count - before
        return logits

    # ------------------------------------------------------------------ captured steps of prompt portions
    def _portion_shape(self, rows: Sequence[tuple[StepEntry, int, int]]) -> tuple[tuple, int, int, int]:
        """(what a captured step takes from the host, filler tokens, context bucket, table width)."""
        counts = [len(entry.tokens) for entry, _, _ in rows]
        tokens = sum(counts)
        pad = -tokens % self._portion_pad
        if pad:
            counts.append(pad)
        tiles = tuple(sum(-(-count // size) for count in counts if count > 1) for size in self._tile_sizes)
        singles = sum(1 for count in counts if count == 1)
        wanted = sum(len(entry.want) for entry, _, _ in rows)
        bucket = min(context_bucket(max(seq_len for _, _, seq_len in rows)), max(self.max_model_len, 256))
        width = min(self._needed_pages(bucket), self.max_pages_per_request)
        return (tokens + pad, len(counts), tiles, singles, wanted, bucket), pad, bucket, width

    def _portion_step(self, rows: Sequence[tuple[StepEntry, int, int]], sampled: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        shape, pad, bucket, width = self._portion_shape(rows)
        held = self._portion_graphs.get(shape)
        if held is not None and held.generation != self.portion_workspace.generation:
            del self._portion_graphs[shape]  # the workspace has grown since: its buffers are not the ones the graph reads
            held = None
        if held is None:
            seen = self._portion_seen.get(shape, 0) + 1
            if len(self._portion_seen) > 4096:
                self._portion_seen.clear()
            self._portion_seen[shape] = seen
            full = len(self._portion_graphs) >= MAX_PORTION_GRAPHS
            if full:  # the least recently used shape goes only if it has not come for a while: shapes that take turns would evict one another for ever
                oldest = next(iter(self._portion_graphs.values()))
                full = self.counters["steps"] - oldest.last_used < PORTION_EVICT_AFTER
            if seen < PORTION_CAPTURE_AT or full:
                return self._eager_step(rows, sampled, as_captured=(pad, bucket, width))
            return self._capture_portion(shape, rows, sampled, pad, bucket, width)
        self._portion_graphs.move_to_end(shape)
        held.last_used = self.counters["steps"]
        host, layout, _ = self._pack(rows, pad_portion=pad, max_pages=width)
        if layout != held.layout:
            raise StepError("a captured step's description is laid out differently from the one it was captured with")
        held.meta.copy_(host, non_blocking=True)
        self._patch_tokens(held.meta, held.layout, sampled)
        held.graph.replay()
        self.counters["portion_graph_replays"] += 1
        self.counters["kernel_launches"] += held.launches
        return held.logits

    def _capture_portion(self, shape: tuple, rows: Sequence[tuple[StepEntry, int, int]], sampled: Optional[torch.Tensor],
                         pad: int, bucket: int, width: int) -> Optional[torch.Tensor]:
        """Run the step once with the buffers a graph of it will use (that run is the step), then capture it."""
        host, layout, facts = self._pack(rows, pad_portion=pad, max_pages=width)
        facts["max_seq_len"] = bucket
        if facts["max_portion_seq_len"]:
            facts["max_portion_seq_len"] = bucket
        workspace = self.portion_workspace
        meta = torch.zeros(host.numel(), dtype=torch.int32, device=self.device)
        meta.copy_(host, non_blocking=True)
        self._patch_tokens(meta, layout, sampled)
        ctx, want = self._context(meta, layout, facts, workspace)

        def run() -> Optional[torch.Tensor]:
            return self.model.forward(ctx, self._views, want)

        before = kernels.launch_count
        logits = run()
        launches = kernels.launch_count - before
        self.counters["eager_steps"] += 1
        self.counters["kernel_launches"] += launches
        generation = workspace.generation
        torch.cuda.current_stream().synchronize()
        workspace.freeze(True)
        try:
            graph = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            with torch.cuda.graph(graph, pool=self._graph_pool):
                captured = run()
        finally:
            workspace.freeze(False)
        if generation != workspace.generation:
            raise StepError("the workspace of captured steps changed during capture")
        if (logits is None) != (captured is None) or (logits is not None and captured.data_ptr() != logits.data_ptr()):
            raise StepError("a captured step does not leave its logits where the step before it did")
        # graphs captured against buffers that have been replaced since are of no use
        for key in [k for k, g in self._portion_graphs.items() if g.generation != generation]:
            del self._portion_graphs[key]
        while len(self._portion_graphs) >= MAX_PORTION_GRAPHS:
            self._portion_graphs.popitem(last=False)
        self._portion_graphs[shape] = _Graph(graph, meta, logits, generation, dict(layout), launches=launches, keepalive=(ctx, want),
                                             last_used=self.counters["steps"])
        self.counters["portion_graph_captures"] += 1
        return logits

    # ------------------------------------------------------------------ graphs
    def _graph_key(self, num_rows: int, max_seq_len: int) -> tuple[int, int]:
        bucket = next(size for size in self._buckets if size >= num_rows)
        return bucket, min(context_bucket(max_seq_len), max(self.max_model_len, 256))

    def _graph_step(self, rows: Sequence[tuple[StepEntry, int, int]], sampled: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        num_rows = len(rows)
        max_seq_len = max(seq_len for _, _, seq_len in rows)
        key = self._graph_key(num_rows, max_seq_len)
        bucket, context_bucket = key
        held = self._graphs.get(key)
        if held is None or held.generation != self.graph_workspace.generation:
            held = self._capture_padding_graph(key)
        self._update_mirror(held, rows, bucket)
        self._upload(held)
        self._patch_tokens(held.meta, held.layout, sampled)
        held.graph.replay()
        self.counters["graph_replays"] += 1
        self.counters["kernel_launches"] += held.launches
        wanted_rows = [row for row, (entry, _, _) in enumerate(rows) if entry.want]
        if not wanted_rows:
            return None
        if wanted_rows == list(range(num_rows)):
            return held.logits[:num_rows]
        index = torch.tensor(wanted_rows, dtype=torch.long, device=self.device)
        return held.logits.index_select(0, index)

    def capture_decode_graphs(self, max_batch: int, max_context: int) -> int:
        """Capture, ahead of the first request, the decode graphs of every batch bucket up to
        ``max_batch`` rows and every context bucket up to ``max_context`` tokens, so that no step of
        a running engine pays for a capture (a capture runs the step two to three times).
        Returns how many graphs were captured."""
        if self.decode_mode != "cuda_graph" or not self._is_cuda:
            return 0
        captured = 0
        top = min(max_context, self.max_model_len)
        contexts = sorted({self._graph_key(1, length)[1] for length in list(range(1, top + 1, 64)) + [top]})
        limit = max(1, min(max_batch, self.max_graph_batch))
        buckets = [size for size in self._buckets if size < limit] + [next(size for size in self._buckets if size >= limit)]
        # the largest first: its buffers are the workspace's final size, and a workspace that grows
        # afterwards would retire the graphs captured before (the second pass finds nothing to do then)
        for _ in range(2):
            for bucket in reversed(buckets):
                for context in reversed(contexts):
                    held = self._graphs.get((bucket, context))
                    if held is None or held.generation != self.graph_workspace.generation:
                        self._capture_padding_graph((bucket, context))
                        captured += 1
        return captured

    def _capture_padding_graph(self, key: tuple[int, int]) -> _Graph:
        # The graph is captured over padding rows only (token 0 at position 0 of the reserved
        # page, the scratch state slot), so that the capture's warm-up runs touch no request:
        # a mixer with state of its own would otherwise see a request's token several times.
        # Every padded row is "wanted" inside the graph; the caller's wants are picked after.
        bucket, context = key
        host, layout, facts = self._pack((), pad_rows=bucket, max_pages=self.max_pages_per_request, include_want=False)
        facts["max_seq_len"] = context
        held = self._capture(key, host, layout, facts)
        held.mirror = host.numpy().copy()
        held.row_state = [None] * bucket
        return held

    def _needed_pages(self, seq_len: int) -> int:
        return -(-seq_len // self.cache.page_size)

    def _update_mirror(self, held: _Graph, rows: Sequence[tuple[StepEntry, int, int]], bucket: int) -> None:
        """Bring the host mirror of a graph's metadata to this step: per row the token, the
        position, the length, and the pages that were added since the row was last written."""
        mirror = held.mirror
        layout = held.layout
        token_at = layout["token_ids"][0]
        future_at = layout["future_src"][0]
        position_at = layout["positions"][0]
        length_at = layout["seq_lens"][0]
        slot_at = layout["state_slots"][0]
        write_at = layout["write_from"][0]
        table_at = layout["tables"][0]
        width = self.max_pages_per_request
        groups = self.cache.layout.groups
        for row, (entry, start, seq_len) in enumerate(rows):
            record = self.cache.get(entry.request_id)
            mirror[token_at + row] = entry.tokens[0]
            mirror[future_at + row] = -1 if entry.future is None else entry.future
            mirror[position_at + row] = start
            mirror[length_at + row] = seq_len
            mirror[slot_at + row] = record.state_slot
            mirror[write_at + row] = len(record.shared) * self.cache.page_size
            need = self._needed_pages(seq_len)
            state = held.row_state[row]
            # The row's pages may be topped up only for the same admission of the request: an id
            # that was released and admitted again (a preempted request coming back, a reused id)
            # has a new record and new pages, and its row is rewritten whole.
            same = state is not None and state[0] is record
            for group in groups:
                base = table_at + (group.index * bucket + row) * width
                table = record.tables[group.index]
                have = state[1][group.index] if same else None
                if have is None or have > need or group.spec.window is not None:
                    mirror[base : base + width] = -1
                    mirror[base : base + need] = table[:need]
                elif need > have:
                    mirror[base + have : base + need] = table[have:need]
            held.row_state[row] = (record, [need] * len(groups))
        for row in range(len(rows), bucket):
            if held.row_state[row] is not None:  # the row becomes padding: token 0 at position 0 of the reserved page
                mirror[token_at + row] = 0
                mirror[future_at + row] = -1
                mirror[position_at + row] = 0
                mirror[length_at + row] = 1
                mirror[slot_at + row] = self.cache.scratch_state_slot
                mirror[write_at + row] = 0
                for group in groups:
                    base = table_at + (group.index * bucket + row) * width
                    mirror[base : base + width] = 0
                held.row_state[row] = None

    def _upload(self, held: _Graph) -> None:
        if not held.staging:
            for _ in range(4):
                pinned = torch.empty(held.mirror.shape[0], dtype=torch.int32, pin_memory=True)
                held.staging.append((pinned, pinned.numpy(), torch.cuda.Event()))
        pinned, view, event = held.staging[held.next_staging]
        held.next_staging = (held.next_staging + 1) % len(held.staging)
        event.synchronize()  # the copy that last used this buffer has run (a fresh event is complete)
        view[:] = held.mirror
        held.meta.copy_(pinned, non_blocking=True)
        event.record()

    def _capture(self, key: tuple[int, int], host: torch.Tensor, layout: dict, facts: dict) -> _Graph:
        bucket, _ = key
        workspace = self.graph_workspace
        meta = torch.zeros(host.numel(), dtype=torch.int32, device=self.device)
        meta.copy_(host)
        graph_layout = dict(layout)
        # inside the graph every row's single token gives logits
        want_all = torch.arange(bucket, dtype=torch.int32, device=self.device)
        ctx, _ = self._context(meta, graph_layout, facts, workspace)

        def run() -> torch.Tensor:
            return self.model.forward(ctx, self._views, want_all)

        # Warm up on a side stream: buffers reach their size, libraries initialise (twice for the
        # first graph of this runner, once for later ones, whose kernels have all run before).
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2 if self.counters["graph_captures"] == 0 else 1):
                run()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        generation = workspace.generation
        workspace.freeze(True)
        try:
            graph = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            before = kernels.launch_count
            with torch.cuda.graph(graph, pool=self._graph_pool):
                logits = run()
            launches = kernels.launch_count - before
        finally:
            workspace.freeze(False)
        if generation != workspace.generation:
            raise StepError("the graph workspace changed during capture")
        # a grown workspace invalidates graphs captured against the old buffers
        self._graphs = {k: g for k, g in self._graphs.items() if g.generation == generation}
        held = _Graph(graph, meta, logits, generation, graph_layout, launches=launches, keepalive=(ctx, want_all))
        self._graphs[key] = held
        self.counters["graph_captures"] += 1
        return held

    # ------------------------------------------------------------------ errors
    def check_errors(self) -> None:
        """Raise if a kernel saw an index outside its tensors (synchronises)."""
        flag = int(self.error_flag.item())
        if flag:
            self.error_flag.zero_()
            reasons = []
            if flag & 1:
                reasons.append("a block table entry outside the page pool")
            if flag & 2:
                reasons.append("a token id outside the vocabulary")
            if flag & 4:
                reasons.append("a row index outside the batch")
            if flag & 8:
                reasons.append("a position outside the rotary table")
            if flag & 16:
                reasons.append("a copy into shared memory did not complete within its wait limit")
            if flag & 64:
                reasons.append("(the wait was in the TMA-fed decode attention)")
            if flag & 128:
                reasons.append("(the wait was in the tcgen05 prefill attention)")
            if flag & 32:
                reasons.append("a block's shared memory did not start on the 1024-byte boundary its swizzled tiles need")
            raise StepError("a kernel refused an index: " + "; ".join(reasons))
