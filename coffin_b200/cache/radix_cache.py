"""Radix prefix cache over KV blocks, with delta-net state snapshots.

A trie whose edges are whole token blocks (64 tokens).  A node owns one reference on its KV
block and may carry a snapshot of the linear-attention state taken right after the block's
last token.  For a hybrid model a prefix is only reusable up to a node that has a snapshot
(the recurrent state cannot be rebuilt from KV), so ``match_prefix(require_states=True)``
returns the deepest such node.  Image prompts salt the block keys with the digests of the
images that overlap the block, so equal placeholder tokens with different pixels never match.
Snapshots are the expensive part (tens of MB each) and are kept under an LRU budget; blocks are
evicted leaf-first, least recently used first, and only when nothing but the cache holds them.
Reference: ``cache/radix_cache.py:79-161`` (media ids), ``:235-318`` (match), ``:387-451``
(insert), ``:555-577`` (snapshot budget), ``:579-716`` (evict / stats).
"""
from __future__ import annotations

import hashlib
import itertools
from typing import Any, Iterable, Sequence

from .paged_cache import BlockPool


def media_signature(digests: Iterable[str]) -> str:
    h = hashlib.sha256()
    for d in digests:
        h.update(d.encode())
    return h.hexdigest()[:16]


def media_ids_for(n_tokens: int, block_size: int, mm: Any | None) -> list[str]:
    """Per-block salt strings: the signature of the images overlapping each block ("" if none).

    ``mm`` needs ``spans`` (``[(start, end), ...]`` absolute token ranges, prompt order) and
    ``digests`` (one per span), or a single ``digest`` for all spans.
    """
    nblk = n_tokens // block_size
    if mm is None or not getattr(mm, "spans", None):
        return [""] * nblk
    spans = list(mm.spans)
    digests = list(getattr(mm, "digests", None) or [getattr(mm, "digest", "")] * len(spans))
    out = []
    for b in range(nblk):
        lo, hi = b * block_size, (b + 1) * block_size
        hit = [d for (s, e), d in zip(spans, digests) if s < hi and e > lo]
        out.append(media_signature(hit) if hit else "")
    return out


class RadixNode:
    __slots__ = ("key", "parent", "children", "block", "state", "tick", "depth")

    def __init__(self, key, parent: "RadixNode | None", block: int, depth: int) -> None:
        self.key = key
        self.parent = parent
        self.children: dict[Any, RadixNode] = {}
        self.block = block
        self.state: Any | None = None
        self.tick = 0
        self.depth = depth          # blocks from the root, i.e. tokens = depth * block_size


class RadixCache:
    def __init__(self, pool: BlockPool, max_snapshots: int = 8) -> None:
        self.pool = pool
        self.bs = pool.block_size
        self.max_snapshots = max_snapshots
        self.root = RadixNode(None, None, -1, 0)
        self._clock = itertools.count(1)
        self.n_nodes = 0
        self.n_queries = self.n_hits = 0
        self.tokens_queried = self.tokens_hit = 0
        self.n_evicted = 0

    # ------------------------------------------------------------------ helpers
    def _keys(self, tokens: Sequence[int], n_blocks: int, mm: Any | None) -> list[tuple]:
        salts = media_ids_for(n_blocks * self.bs, self.bs, mm)
        return [(tuple(tokens[b * self.bs:(b + 1) * self.bs]), salts[b]) for b in range(n_blocks)]

    def _touch(self, node: RadixNode) -> None:
        t = next(self._clock)
        while node is not None and node is not self.root:
            node.tick = t
            node = node.parent

    def _nodes(self) -> list[RadixNode]:
        out, stack = [], list(self.root.children.values())
        while stack:
            n = stack.pop()
            out.append(n)
            stack.extend(n.children.values())
        return out

    # ------------------------------------------------------------------ lookup
    def match_prefix(self, tokens: Sequence[int], require_states: bool = True, mm: Any | None = None
                     ) -> tuple[list[int], int, Any | None]:
        """Longest cached prefix of ``tokens`` that leaves at least one token to compute.

        Returns ``(blocks, n_tokens, state)``; every returned block has been incref'ed for the
        caller.  With ``require_states`` the match ends at the deepest node holding a snapshot
        (``state`` is that snapshot), else at the deepest matching node (``state`` None).
        """
        self.n_queries += 1
        self.tokens_queried += len(tokens)
        limit = max(0, (len(tokens) - 1) // self.bs)
        node, path = self.root, []
        for key in self._keys(tokens, limit, mm):
            child = node.children.get(key)
            if child is None:
                break
            path.append(child)
            node = child
        if require_states:
            while path and path[-1].state is None:
                path.pop()
        if not path:
            return [], 0, None
        self._touch(path[-1])
        blocks = [n.block for n in path]
        for b in blocks:
            self.pool.incref(b)
        self.n_hits += 1
        self.tokens_hit += len(blocks) * self.bs
        return blocks, len(blocks) * self.bs, path[-1].state

    # ------------------------------------------------------------------ insert
    def insert(self, tokens: Sequence[int], blocks: Sequence[int], states: dict[int, Any] | None = None,
               mm: Any | None = None) -> int:
        """Publish the full blocks of a computed sequence.

        ``blocks[i]`` holds tokens ``[i*bs, (i+1)*bs)``; ``states`` maps a token count (a multiple
        of the block size) to the snapshot taken after that many tokens.  Existing nodes keep
        their block (the caller's duplicate stays private); new nodes take a reference.
        Returns the number of new nodes.
        """
        n_blocks = min(len(tokens) // self.bs, len(blocks))
        node, created = self.root, 0
        for i, key in enumerate(self._keys(tokens, n_blocks, mm)):
            child = node.children.get(key)
            if child is None:
                child = RadixNode(key, node, blocks[i], i + 1)
                self.pool.incref(blocks[i])
                node.children[key] = child
                self.n_nodes += 1
                created += 1
            node = child
            if states and (i + 1) * self.bs in states and child.state is None:
                child.state = states[(i + 1) * self.bs]
        if node is not self.root:
            self._touch(node)
        self._trim_states()
        return created

    def _trim_states(self) -> None:
        holders = [n for n in self._nodes() if n.state is not None]
        if len(holders) <= self.max_snapshots:
            return
        holders.sort(key=lambda n: (n.tick, -n.depth))
        for n in holders[: len(holders) - self.max_snapshots]:
            n.state = None

    # ------------------------------------------------------------------ eviction
    def evictable(self) -> int:
        return sum(1 for n in self._nodes() if self.pool.ref[n.block] == 1)

    def evict(self, n_blocks: int) -> int:
        """Free up to ``n_blocks`` blocks held only by the cache, leaves first, LRU first."""
        freed = 0
        while freed < n_blocks:
            leaves = [n for n in self._nodes() if not n.children and self.pool.ref[n.block] == 1]
            if not leaves:
                break
            leaves.sort(key=lambda n: n.tick)
            for n in leaves:
                if freed >= n_blocks:
                    break
                del n.parent.children[n.key]
                self.pool.decref(n.block)
                n.state = None
                self.n_nodes -= 1
                self.n_evicted += 1
                freed += 1
        return freed

    def reserve(self, n_blocks: int) -> bool:
        """Make sure ``n_blocks`` are free, evicting cached blocks if needed."""
        short = n_blocks - self.pool.free_blocks
        if short > 0:
            self.evict(short)
        return self.pool.free_blocks >= n_blocks

    def clear(self) -> None:
        for n in self._nodes():
            self.pool.decref(n.block)
            n.state = None
        self.root.children.clear()
        self.n_nodes = 0

    def stats(self) -> dict:
        return {"nodes": self.n_nodes, "snapshots": sum(1 for n in self._nodes() if n.state is not None),
                "queries": self.n_queries, "hits": self.n_hits, "tokens_queried": self.tokens_queried,
                "tokens_hit": self.tokens_hit, "evicted": self.n_evicted,
                "hit_rate": self.tokens_hit / self.tokens_queried if self.tokens_queried else 0.0}
