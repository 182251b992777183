"""Device tensors behind the cache manager: pages of keys and values per group
and one tensor per per-request state (kairyu/engine/core/kv_pool.py:24-49)."""

from __future__ import annotations

from typing import Sequence

import torch

from kairyu_b200.cache.manager import CacheLayout
from kairyu_b200.parts.base import CacheView

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


class CacheStorage:
    """K and V of group g: ``[slots_in_group, num_pages, page_size, kv_heads, head_dim]``
    (V with the spec's value width where that differs).
    A page of one slot is a contiguous ``[page_size, kv_heads*head_dim]`` tile.
    State tensors: ``[max_requests + 1, *shape]`` each; the last row is the scratch slot that
    padding rows of a decode graph use."""

    def __init__(
        self,
        layout: CacheLayout,
        *,
        num_pages: int,
        page_size: int,
        max_requests: int,
        dtype: torch.dtype,
        device: str,
    ) -> None:
        self.layout = layout
        self.page_size = page_size
        self.num_pages = num_pages
        self.k: list[torch.Tensor] = []
        self.v: list[torch.Tensor] = []
        for group in layout.groups:
            shape = (len(group.slots), num_pages, page_size, group.spec.num_kv_heads)
            if group.spec.head_dim == group.spec.value_dim:
                # one allocation, the values a fixed distance behind the keys: a kernel may then fetch
                # the keys and the values of a run of positions with one strided copy
                both = torch.zeros((2, *shape, group.spec.head_dim), dtype=dtype, device=device)
                self.k.append(both[0])
                self.v.append(both[1])
                continue
            self.k.append(torch.zeros((*shape, group.spec.head_dim), dtype=dtype, device=device))
            self.v.append(torch.zeros((*shape, group.spec.value_dim), dtype=dtype, device=device))
        self.states = [
            torch.zeros((max_requests + 1, *binding.spec.shape), dtype=_STATE_DTYPES[binding.spec.dtype], device=device)
            for binding in layout.states
        ]

    @staticmethod
    def bytes_per_page(layout: CacheLayout, page_size: int, element_size: int) -> int:
        return sum(
            len(group.slots) * page_size * group.spec.num_kv_heads * (group.spec.head_dim + group.spec.value_dim) * element_size
            for group in layout.groups
        )

    def view(self, slot: int, *, writes: bool) -> CacheView:
        view = CacheView(page_size=self.page_size, writes=writes)
        group_index = self.layout.group_of_slot.get(slot)
        if group_index is not None:
            group = self.layout.groups[group_index]
            position = group.slots.index(slot)
            view.k = self.k[group_index][position]
            view.v = self.v[group_index][position]
            view.group = group_index
        states = [tensor for binding, tensor in zip(self.layout.states, self.states) if binding.slot == slot]
        if states:
            view.state = states[0] if len(states) == 1 else states  # type: ignore[assignment]
        return view

    def zero_state_slots(self, slots: Sequence[int]) -> None:
        """A request that takes a slot starts from zero state."""
        if not slots or not self.states:
            return
        index = torch.tensor(list(slots), dtype=torch.long, device=self.states[0].device)
        for tensor in self.states:
            tensor.index_fill_(0, index, 0)

    def poison_pages(self, group: int, pages: Sequence[int], value: float = float("nan")) -> None:
        """Debug aid: overwrite pages that were given back, so a read of stale
        keys shows up as NaN instead of as a plausible number."""
        if not pages:
            return
        index = torch.tensor(list(pages), dtype=torch.long, device=self.k[group].device)
        self.k[group].index_fill_(1, index, value)
        self.v[group].index_fill_(1, index, value)
