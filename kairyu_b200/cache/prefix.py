"""Prefix sharing: a tree of whole pages keyed by the tokens they hold.

A node is one page index of every paged group (the same positions in each): its key is the
``page_size`` tokens at those positions, its parent the page before.  Only whole pages are shared,
so a request's partly filled last page is always its own and nothing is ever copied on write
(kairyu/engine/core/radix_kv.py:1-11).  A node counts the live requests that read it; a node that
none reads stays in the tree, to be matched again or to be taken back, oldest unread leaf first,
when pages run short (radix_kv.py:488-539).  A request holds a whole path from the root, so a
node's count is never below its children's: every node with count zero can be taken back, leaves
first.

Host-side only; it never touches a tensor.
"""

from __future__ import annotations

import heapq
from typing import Optional, Sequence


class PrefixNode:
    __slots__ = ("parent", "key", "pages", "children", "readers", "stamp", "alive")

    def __init__(self, parent: Optional["PrefixNode"], key: tuple[int, ...], pages: tuple[int, ...]) -> None:
        self.parent = parent
        self.key = key
        self.pages = pages  # one physical page per paged group
        self.children: dict[tuple[int, ...], PrefixNode] = {}
        self.readers = 0
        self.stamp = 0
        self.alive = True


class PrefixIndex:
    def __init__(self, page_size: int) -> None:
        self.page_size = page_size
        self.root = PrefixNode(None, (), ())
        self._clock = 0
        self._heap: list[tuple[int, int, PrefixNode]] = []  # (stamp, tiebreak, node): candidates to take back
        self._pushed = 0
        self.num_nodes = 0
        self.num_unread = 0  # nodes no live request reads: each can be taken back
        self.counters = {"inserted_pages": 0, "evicted_pages": 0}

    # ------------------------------------------------------------------ internals
    def _touch(self, node: PrefixNode) -> None:
        self._clock += 1
        node.stamp = self._clock

    def _offer(self, node: PrefixNode) -> None:
        """Put a node that nobody reads and nothing hangs below on the take-back heap."""
        if node.alive and node.readers == 0 and not node.children and node is not self.root:
            self._pushed += 1
            heapq.heappush(self._heap, (node.stamp, self._pushed, node))
            if len(self._heap) > 4 * self.num_nodes + 64:  # mostly entries of nodes that changed since
                self._heap = [entry for entry in self._heap if self._current(entry)]
                heapq.heapify(self._heap)

    @staticmethod
    def _current(entry: tuple[int, int, PrefixNode]) -> bool:
        stamp, _, node = entry
        return node.alive and node.readers == 0 and not node.children and node.stamp == stamp

    # ------------------------------------------------------------------ lookups
    def match(self, tokens: Sequence[int], max_pages: Optional[int] = None) -> list[PrefixNode]:
        """The longest path of whole pages that ``tokens`` starts with (at most ``max_pages``)."""
        size = self.page_size
        limit = len(tokens) // size
        if max_pages is not None:
            limit = min(limit, max_pages)
        path: list[PrefixNode] = []
        node = self.root
        for index in range(limit):
            child = node.children.get(tuple(tokens[index * size : (index + 1) * size]))
            if child is None:
                break
            path.append(child)
            node = child
        return path

    # ------------------------------------------------------------------ readers
    def acquire(self, path: Sequence[PrefixNode]) -> None:
        for node in path:
            if node.readers == 0:
                self.num_unread -= 1
            node.readers += 1
            self._touch(node)

    def drop(self, path: Sequence[PrefixNode]) -> None:
        for node in reversed(path):
            if node.readers < 1:
                raise ValueError("a prefix page was dropped more often than it was acquired")
            node.readers -= 1
            self._touch(node)
            if node.readers == 0:
                self.num_unread += 1
                self._offer(node)

    # ------------------------------------------------------------------ growth and shrinkage
    def child(self, parent: Optional[PrefixNode], key: tuple[int, ...]) -> Optional[PrefixNode]:
        return (parent or self.root).children.get(key)

    def insert(self, parent: Optional[PrefixNode], key: tuple[int, ...], pages: tuple[int, ...], *, readers: int) -> PrefixNode:
        """Hang a new page below ``parent`` (None: the root); the caller has checked that no
        child has this key.  ``readers``: 1 if the inserting request keeps reading it, else 0."""
        above = parent or self.root
        if len(key) != self.page_size:
            raise ValueError(f"a prefix page holds {self.page_size} tokens, got {len(key)}")
        if key in above.children:
            raise ValueError("this page of tokens is already in the tree")
        if above is not self.root and readers > above.readers:
            raise ValueError("a page cannot have more readers than the page before it")
        node = PrefixNode(above, key, pages)
        node.readers = readers
        above.children[key] = node
        self._touch(node)
        self.num_nodes += 1
        self.counters["inserted_pages"] += 1
        if readers == 0:
            self.num_unread += 1
            self._offer(node)
        return node

    def evict(self, count: int) -> list[tuple[int, ...]]:
        """Take back up to ``count`` nodes, oldest unread leaf first; returns their pages."""
        freed: list[tuple[int, ...]] = []
        while len(freed) < count and self._heap:
            entry = heapq.heappop(self._heap)
            if not self._current(entry):
                continue  # the node changed after it was offered
            node = entry[2]
            parent = node.parent
            del parent.children[node.key]
            node.alive = False
            self.num_nodes -= 1
            self.num_unread -= 1
            self.counters["evicted_pages"] += 1
            freed.append(node.pages)
            self._offer(parent)
        return freed

    # ------------------------------------------------------------------ invariants
    def nodes(self) -> list[PrefixNode]:
        found: list[PrefixNode] = []
        stack = list(self.root.children.values())
        while stack:
            node = stack.pop()
            found.append(node)
            stack.extend(node.children.values())
        return found

    def check(self) -> None:
        nodes = self.nodes()
        if len(nodes) != self.num_nodes:
            raise AssertionError(f"the tree has {len(nodes)} nodes, its count says {self.num_nodes}")
        unread = sum(1 for node in nodes if node.readers == 0)
        if unread != self.num_unread:
            raise AssertionError(f"{unread} nodes are unread, the count says {self.num_unread}")
        for node in nodes:
            if not node.alive:
                raise AssertionError("a removed node is still in the tree")
            if node.readers < 0:
                raise AssertionError("a node has a negative reader count")
            if node.parent is not self.root and node.parent.readers < node.readers:
                raise AssertionError("a node has more readers than the page before it")
        # every unread leaf can be found by evict()
        offered = {id(entry[2]) for entry in self._heap if self._current(entry)}
        for node in nodes:
            if node.readers == 0 and not node.children and id(node) not in offered:
                raise AssertionError("an unread leaf is missing from the take-back heap")
