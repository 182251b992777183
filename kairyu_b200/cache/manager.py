"""The cache manager: which pages and which state slot each live request holds.

Host-side only; the tensors live in :mod:`kairyu_b200.cache.storage`.

Cache slots (one per schedule call that writes a cache) with equal page
geometry and window form a *group*; each group has its own page pool and its
own block table per request, because a group that keeps every key and a group
that keeps a window of them fill and empty at different rates.  A request's
table for a group maps page index ``position // page_size`` to a physical page,
or -1 once a windowed group has given the page back.

The reference's dense pool is uniform (one table per request,
kairyu/engine/core/radix_kv.py:144-149); groups generalise it the way its
hybrid cache descriptors do (kairyu/engine/core/frontier_cache.py:19-75).

Prefix sharing (``prefix_sharing=True``; off unless asked for).  Whole pages that a request has
filled can be *published* to a tree keyed by their tokens (:mod:`kairyu_b200.cache.prefix`); a
later request whose tokens start the same way is admitted with those pages at the head of its
block tables and starts computing behind them.  A request's table is then ``shared pages ‖ its
own pages``: shared pages are only read (a request writes at positions it computes, and those lie
behind the shared pages), its own pages go back to the pool when it ends unless they were
published, and published pages that no live request reads are taken back, oldest first, when a
pool runs short.  It needs every paged group to keep all keys and no per-request state: a window
gives pages back while the request runs, and state cannot be rebuilt from pages.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Hashable, Mapping, Optional, Sequence

from kairyu_b200.cache.page_pool import OutOfPages, PagePool
from kairyu_b200.cache.prefix import PrefixIndex, PrefixNode
from kairyu_b200.parts.base import PagedKVSpec, StateSpec


@dataclass(frozen=True)
class CacheGroup:
    index: int
    spec: PagedKVSpec
    slots: tuple[int, ...]  # cache slots stored in this group, in storage order


@dataclass(frozen=True)
class StateBinding:
    slot: int  # cache slot
    index: int  # which of the slot's StateSpecs
    spec: StateSpec


@dataclass(frozen=True)
class CacheLayout:
    """Groups of paged slots and the list of per-request state tensors."""

    groups: tuple[CacheGroup, ...]
    states: tuple[StateBinding, ...]
    group_of_slot: Mapping[int, int]

    @classmethod
    def from_slot_specs(cls, slot_specs: Mapping[int, Sequence[Any]]) -> "CacheLayout":
        by_spec: dict[PagedKVSpec, list[int]] = {}
        states: list[StateBinding] = []
        for slot in sorted(slot_specs):
            paged = [s for s in slot_specs[slot] if isinstance(s, PagedKVSpec)]
            if len(paged) > 1:
                raise ValueError(f"cache slot {slot} asks for more than one paged cache")
            if paged:
                by_spec.setdefault(paged[0], []).append(slot)
            for index, spec in enumerate(s for s in slot_specs[slot] if isinstance(s, StateSpec)):
                states.append(StateBinding(slot, index, spec))
        groups = tuple(
            CacheGroup(index, spec, tuple(slots)) for index, (spec, slots) in enumerate(by_spec.items())
        )
        group_of_slot = {slot: group.index for group in groups for slot in group.slots}
        return cls(groups, tuple(states), group_of_slot)


@dataclass
class RequestCache:
    request_id: Hashable
    state_slot: int
    tables: list[list[int]]  # per group: page index -> physical page or -1
    first_live: list[int]  # per group: lowest page index still held
    num_tokens: int = 0  # positions [0, num_tokens) have been computed
    shared: list[PrefixNode] = field(default_factory=list)  # the leading pages it reads from the prefix tree
    num_cached_tokens: int = 0  # how many tokens admission found in the tree


class CacheManager:
    def __init__(
        self,
        layout: CacheLayout,
        *,
        num_pages: int,
        page_size: int,
        max_requests: int,
        reserved_pages: int = 1,
        prefix_sharing: bool = False,
    ) -> None:
        if page_size < 1:
            raise ValueError("page_size must be >= 1")
        if prefix_sharing:
            windowed = [group.index for group in layout.groups if group.spec.window is not None]
            if windowed or layout.states or not layout.groups:
                raise ValueError(
                    "prefix sharing needs paged groups that keep every key and no per-request state; "
                    f"this model has windowed groups {windowed} and {len(layout.states)} state tensors"
                )
        self.layout = layout
        self.page_size = page_size
        self.num_pages = num_pages
        self.pools = [PagePool(num_pages, reserved=reserved_pages) for _ in layout.groups]
        self.max_requests = max_requests
        self._free_state_slots = list(range(max_requests - 1, -1, -1))
        # One state slot beyond the requests' own, as page 0 is reserved among the pages: the
        # padding rows of a replayed decode graph read and write it, so that no live request's
        # state is touched by a row that stands for nobody.
        self.scratch_state_slot = max_requests
        self._requests: dict[Hashable, RequestCache] = {}
        self.fresh_state_slots: list[int] = []  # slots handed out since the storage last zeroed them
        self.prefix: Optional[PrefixIndex] = PrefixIndex(page_size) if prefix_sharing else None
        # Debug aid: with ``log_freed_pages`` every page that goes back to a pool is noted, per
        # group, until ``take_freed_pages`` is called (the step function can then overwrite them).
        self.log_freed_pages = False
        self._freed_log: list[list[int]] = [[] for _ in layout.groups]

    # ------------------------------------------------------------------ queries
    def __contains__(self, request_id: Hashable) -> bool:
        return request_id in self._requests

    def get(self, request_id: Hashable) -> RequestCache:
        return self._requests[request_id]

    @property
    def live_requests(self) -> int:
        return len(self._requests)

    def free_pages(self, group: int = 0) -> int:
        return self.pools[group].num_free

    def available_pages(self, group: int = 0) -> int:
        """Free pages plus published pages that no live request reads (they can be taken back)."""
        unread = self.prefix.num_unread if self.prefix is not None else 0
        return self.pools[group].num_free + unread

    def pages_for(self, num_tokens: int) -> int:
        return -(-num_tokens // self.page_size)

    def _first_needed_page(self, group: CacheGroup, query_start: int) -> int:
        """Lowest page index a query at ``query_start`` (or later) can read."""
        if group.spec.window is None:
            return 0
        return max(0, query_start - group.spec.window + 1) // self.page_size

    def pages_needed(self, request_id: Optional[Hashable], upto: int, query_start: int) -> list[int]:
        """New pages per group to cover positions [.., upto) for queries from ``query_start``."""
        needed = []
        record = self._requests.get(request_id) if request_id is not None else None
        for group in self.layout.groups:
            first = self._first_needed_page(group, query_start)
            last = self.pages_for(upto)
            if record is None:
                needed.append(max(0, last - first))
            else:
                table = record.tables[group.index]
                held = sum(1 for index in range(first, min(last, len(table))) if table[index] >= 0)
                needed.append(max(0, last - first) - held)
        return needed

    def peak_pages(self, num_tokens: int, portion: int = 1) -> list[int]:
        """Per group, the most pages a request of ``num_tokens`` tokens holds at any time when it is
        fed in portions of at most ``portion`` tokens.  A group that keeps every key holds them all;
        a windowed group holds the window behind the portion's first query plus the portion itself
        (one page more for a window that does not start on a page's edge)."""
        whole = self.pages_for(num_tokens)
        return [
            whole if group.spec.window is None else min(whole, self.pages_for(group.spec.window + max(portion, 1)) + 1)
            for group in self.layout.groups
        ]

    def can_hold(self, num_tokens: int, portion: int = 1) -> bool:
        """Whether an empty cache could ever hold a request of this many tokens."""
        return all(pages <= pool.capacity for pages, pool in zip(self.peak_pages(num_tokens, portion), self.pools))

    def held_pages(self, request_id: Hashable) -> tuple[list[int], list[int]]:
        """Per group: (pages the request's tables name, those of them that are its own, that is,
        not read from the prefix tree)."""
        record = self._requests[request_id]
        named = [sum(1 for page in table if page >= 0) for table in record.tables]
        own = [sum(1 for page in table[len(record.shared):] if page >= 0) for table in record.tables]
        return named, own

    # ------------------------------------------------------------------ lifecycle
    def admit(self, request_id: Hashable, tokens: Optional[Sequence[int]] = None) -> RequestCache:
        """Make a request live.  With prefix sharing and its ``tokens`` given, the whole pages the
        tree already holds for them head its block tables and count as computed; at least the
        last token is left to compute, so that the request's first step has logits
        (kairyu/engine/core/scheduler.py:1589-1593)."""
        if request_id in self._requests:
            raise ValueError(f"request {request_id!r} is already live")
        if not self._free_state_slots:
            raise OutOfPages(f"all {self.max_requests} request slots are in use")
        slot = self._free_state_slots.pop()
        self.fresh_state_slots.append(slot)
        record = RequestCache(
            request_id,
            slot,
            tables=[[] for _ in self.layout.groups],
            first_live=[0 for _ in self.layout.groups],
        )
        if self.prefix is not None and tokens is not None and len(tokens) > 1:
            path = self.prefix.match(tokens, max_pages=(len(tokens) - 1) // self.page_size)
            self.prefix.acquire(path)
            record.shared = path
            for group in self.layout.groups:
                record.tables[group.index] = [node.pages[group.index] for node in path]
            record.num_tokens = record.num_cached_tokens = len(path) * self.page_size
        self._requests[request_id] = record
        return record

    def ensure_capacity(self, request_id: Hashable, upto: int, *, query_start: Optional[int] = None) -> bool:
        """Hold pages for positions up to ``upto`` (exclusive) as seen by queries
        from ``query_start`` (default: the request's computed length).  All
        groups or nothing: returns False, changing nothing, if any pool is short."""
        record = self._requests[request_id]
        last = -(-upto // self.page_size)
        # The common case of a decode step: every table already reaches the last page.  (A
        # table is only ever extended together with the allocation of its new entries, and a
        # request's positions only grow, so a table that long covers what can be read.)
        for table in record.tables:
            if len(table) < last:
                break
        else:
            return True
        if query_start is None:
            query_start = record.num_tokens
        needed = self.pages_needed(request_id, upto, query_start)
        short = max(count - pool.num_free for count, pool in zip(needed, self.pools))
        if short > 0:
            if self.prefix is None or short > self.prefix.num_unread:
                return False
            self._take_back(short)
        for group, pool in zip(self.layout.groups, self.pools):
            table = record.tables[group.index]
            first = self._first_needed_page(group, query_start)
            while len(table) < last:
                table.append(-1)
            for index in range(first, last):
                if table[index] < 0:
                    table[index] = pool.allocate(1)[0]
        return True

    def advance(self, request_id: Hashable, num_tokens: int) -> None:
        """Record that positions [0, num_tokens) are computed and give back the
        pages of windowed groups that no later query can read."""
        record = self._requests[request_id]
        if num_tokens < record.num_tokens:
            raise ValueError("a request's computed length cannot shrink")
        record.num_tokens = num_tokens
        for group, pool in zip(self.layout.groups, self.pools):
            if group.spec.window is None:
                continue
            table = record.tables[group.index]
            keep_from = self._first_needed_page(group, num_tokens)
            stale = []
            for index in range(record.first_live[group.index], min(keep_from, len(table))):
                if table[index] >= 0:
                    stale.append(table[index])
                    table[index] = -1
            if stale:
                self._give_back(group.index, stale)
            record.first_live[group.index] = max(record.first_live[group.index], min(keep_from, len(table)))

    def _take_back(self, count: int) -> None:
        """Return ``count`` published pages that nobody reads to every pool."""
        for pages in self.prefix.evict(count):
            for group, page in enumerate(pages):
                self._give_back(group, [page])

    def publish(self, request_id: Hashable, tokens: Sequence[int]) -> int:
        """Make the whole pages this request has computed matchable; ``tokens`` are the tokens
        at its positions.  The request goes on reading them as shared pages.  Where the tree
        already holds a page of the same tokens (another request computed it meanwhile), this
        request keeps its own copy and publishing stops there.  Returns the pages published
        (kairyu/engine/core/radix_kv.py:765-777, 815-889)."""
        if self.prefix is None:
            return 0
        record = self._requests[request_id]
        size = self.page_size
        whole = min(record.num_tokens, len(tokens)) // size
        parent = record.shared[-1] if record.shared else None
        published = 0
        for index in range(len(record.shared), whole):
            key = tuple(tokens[index * size : (index + 1) * size])
            if self.prefix.child(parent, key) is not None:
                break
            pages = tuple(record.tables[group.index][index] for group in self.layout.groups)
            parent = self.prefix.insert(parent, key, pages, readers=1)
            record.shared.append(parent)
            published += 1
        return published

    def release(self, request_id: Hashable) -> None:
        """The request ended (finished, aborted or preempted): its own pages go back to the
        pools; the shared pages it read lose a reader and stay in the tree."""
        record = self._requests.pop(request_id)
        own_from = len(record.shared)
        for group, table in enumerate(record.tables):
            self._give_back(group, [page for page in table[own_from:] if page >= 0])
        if record.shared:
            self.prefix.drop(record.shared)
        self._free_state_slots.append(record.state_slot)

    def block_table(self, request_id: Hashable, group: int) -> list[int]:
        return self._requests[request_id].tables[group]

    def _give_back(self, group: int, pages: Sequence[int]) -> None:
        self.pools[group].free(pages)
        if self.log_freed_pages:
            self._freed_log[group].extend(pages)

    def take_freed_pages(self) -> list[list[int]]:
        freed, self._freed_log = self._freed_log, [[] for _ in self.layout.groups]
        return freed

    def take_fresh_state_slots(self) -> list[int]:
        fresh, self.fresh_state_slots = self.fresh_state_slots, []
        return fresh

    # ------------------------------------------------------------------ invariants
    def check(self) -> None:
        """No page lost, held twice, or freed twice; no state slot shared."""
        for group, pool in zip(self.layout.groups, self.pools):
            pool.check()
            seen: dict[int, Hashable] = {}
            if self.prefix is not None:
                for node in self.prefix.nodes():
                    page = node.pages[group.index]
                    if page in seen or page < pool.reserved:
                        raise AssertionError(f"group {group.index}: page {page} is in the prefix tree twice or reserved")
                    seen[page] = "prefix tree"
            for record in self._requests.values():
                shared = [node.pages[group.index] for node in record.shared]
                if record.tables[group.index][: len(shared)] != shared:
                    raise AssertionError(f"group {group.index}: {record.request_id!r} does not start with its shared pages")
                for page in record.tables[group.index][len(shared) :]:
                    if page < 0:
                        continue
                    if page in seen:
                        raise AssertionError(
                            f"group {group.index}: page {page} held by {seen[page]!r} and {record.request_id!r}"
                        )
                    if page < pool.reserved:
                        raise AssertionError(f"group {group.index}: reserved page {page} handed out")
                    seen[page] = record.request_id
            if len(seen) != pool.num_held:
                raise AssertionError(
                    f"group {group.index}: pool holds {pool.num_held} pages, requests hold {len(seen)}"
                )
        if self.prefix is not None:
            self.prefix.check()
            readers: dict[int, int] = {}
            for record in self._requests.values():
                for node in record.shared:
                    readers[id(node)] = readers.get(id(node), 0) + 1
            for node in self.prefix.nodes():
                if node.readers != readers.get(id(node), 0):
                    raise AssertionError("a prefix page's reader count does not match the requests that read it")
        slots = [record.state_slot for record in self._requests.values()]
        if len(set(slots)) != len(slots):
            raise AssertionError("two requests share a state slot")
        if sorted(slots + self._free_state_slots) != list(range(self.max_requests)):
            raise AssertionError("a state slot was lost or duplicated")
