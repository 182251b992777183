"""Scratch tensors of a step, kept between steps so that a step allocates
nothing and a captured graph sees fixed addresses."""

from __future__ import annotations

import torch


class Workspace:
    def __init__(self, device: str, min_rows: int = 0) -> None:
        """``min_rows``: what a row buffer holds at least from its first allocation on (a workspace whose
        buffers captured graphs point at should not have to grow with the first larger step)."""
        self.device = device
        self.min_rows = min_rows
        self._buffers: dict[tuple[str, int, torch.dtype], torch.Tensor] = {}
        # the views handed out, by (buffer, rows): a step asks for the same few hundred views every time, and
        # slicing a tensor costs as much host time as a third of a kernel launch
        self._views: dict[tuple, torch.Tensor] = {}
        self._frozen = False
        self.generation = 0  # bumps whenever a buffer is (re)allocated

    def buffer(self, tag: str, rows: int, cols: int, dtype: torch.dtype) -> torch.Tensor:
        """A ``[rows, cols]`` view of the buffer named ``tag``; grows (by
        reallocation) when more rows are asked for than ever before."""
        key = (tag, cols, dtype)
        view = self._views.get((key, rows))
        if view is not None:
            return view
        held = self._buffers.get(key)
        if held is None or held.shape[0] < rows:
            if self._frozen:
                raise RuntimeError(
                    f"workspace buffer {tag!r} would have to grow to {rows} rows while a graph is being captured"
                )
            capacity = max(rows, 1, self.min_rows)
            if held is not None:
                capacity = max(capacity, 2 * held.shape[0])
            held = torch.empty((capacity, cols), dtype=dtype, device=self.device)
            self._buffers[key] = held
            self._drop_views(key)
            self.generation += 1
        return self._remember((key, rows), held[:rows])

    def flat(self, tag: str, count: int, dtype: torch.dtype) -> torch.Tensor:
        """A 1-D buffer of ``count`` elements named ``tag``."""
        key = (tag, -1, dtype)
        view = self._views.get((key, count))
        if view is not None:
            return view
        held = self._buffers.get(key)
        if held is None or held.numel() < count:
            if self._frozen:
                raise RuntimeError(f"workspace buffer {tag!r} would have to grow while a graph is being captured")
            capacity = max(count, 1)
            if held is not None:
                capacity = max(capacity, 2 * held.numel())
            held = torch.empty((capacity,), dtype=dtype, device=self.device)
            self._buffers[key] = held
            self._drop_views(key)
            self.generation += 1
        return self._remember((key, count), held[:count])

    def _remember(self, key: tuple, view: torch.Tensor) -> torch.Tensor:
        if len(self._views) >= 4096:  # many sizes over a long run: start over rather than grow without end
            self._views.clear()
        self._views[key] = view
        return view

    def _drop_views(self, key: tuple) -> None:
        """Views of a buffer that has just been replaced point at the old memory."""
        for stale in [k for k in self._views if k[0] == key]:
            del self._views[stale]

    def freeze(self, frozen: bool = True) -> None:
        self._frozen = frozen

    def bytes_held(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._buffers.values())
