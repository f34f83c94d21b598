"""Block ownership: one pool, one radix tree, the model's copy/snapshot hooks.

Everything that hands out or takes back KV blocks goes through here, so that the batched
engine and the single-stream prefix engine share one id space (reference:
``engine/block_manager.py:31-213``).
"""
from __future__ import annotations

from typing import Any

from ..cache.paged_cache import BlockPool, OutOfBlocks, SeqBlocks
from ..cache.radix_cache import RadixCache


class BlockManager:
    def __init__(self, model, num_blocks: int | None = None, block_size: int = 64, max_snapshots: int = 8,
                 prefix_cache: bool = True) -> None:
        self.model = model
        n = num_blocks or getattr(model, "num_blocks")
        self.pool = BlockPool(n, block_size, reserved=1)       # block 0: padding target
        self.radix = RadixCache(self.pool, max_snapshots)
        self.prefix_cache = prefix_cache
        self.n_cow = 0

    @classmethod
    def attach(cls, model, num_blocks=None, block_size=64, max_snapshots=8, prefix_cache=True) -> "BlockManager":
        return cls(model, num_blocks, block_size, max_snapshots, prefix_cache)

    def _copy(self, src: int, dst: int) -> None:
        self.n_cow += 1
        self.model.copy_block(src, dst)

    def new_table(self) -> SeqBlocks:
        return SeqBlocks(self.pool, self._copy)

    # ------------------------------------------------------------------ prefix reuse
    def match_prefix(self, tokens, mm: Any | None = None, require_states: bool = True):
        if not self.prefix_cache:
            return [], 0, None
        return self.radix.match_prefix(tokens, require_states=require_states, mm=mm)

    def insert(self, tokens, blocks, states=None, mm: Any | None = None) -> int:
        if not self.prefix_cache:
            return 0
        return self.radix.insert(tokens, blocks, states, mm)

    # ------------------------------------------------------------------ capacity
    def ensure_blocks(self, table: SeqBlocks, n_tokens: int) -> bool:
        """Reserve room for ``n_tokens`` more tokens, evicting cached blocks if the pool is
        short.  Returns False (nothing reserved beyond what fit) when even eviction cannot
        make room; the caller then preempts a sequence."""
        need = table.blocks_needed(n_tokens)
        if need > self.pool.free_blocks and not self.radix.reserve(need):
            return False
        try:
            table.reserve(n_tokens)
        except OutOfBlocks:
            return False
        return True

    def release(self, table: SeqBlocks | None) -> None:
        if table is not None:
            table.free()

    def stats(self) -> dict:
        return {"blocks": self.pool.num_blocks, "free": self.pool.free_blocks, "used": self.pool.used_blocks,
                "cow": self.n_cow, "prefix": self.radix.stats()}
