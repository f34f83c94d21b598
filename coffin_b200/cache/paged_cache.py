"""Block bookkeeping of the paged KV pool: reference counts, free list, copy-on-write.

The KV tensors themselves live in the model (``[layers, blocks * 64, nkv, hd]``) and are
addressed by block id through per-row block tables handed to the kernels; this module only
decides which block ids a sequence owns.  Blocks are shared between sequences and the radix
prefix cache by reference count; a sequence that must write into a shared tail block first
gets a private copy (``SeqBlocks.reserve`` calls the model's ``copy_block``).
Reference: ``cache/paged_cache.py:78-251`` (pool, alloc/incref/decref/copy_block) and
``:461-577`` (``SeqKV.reserve/commit/free``); there the pool also stores int8 KV and a device
``pos2slot`` table, which the block-table kernels here make unnecessary.
"""
from __future__ import annotations

from typing import Callable

BLOCK_SIZE = 64


class OutOfBlocks(RuntimeError):
    """The pool cannot satisfy an allocation even after the caller's eviction attempt."""


class BlockPool:
    def __init__(self, num_blocks: int, block_size: int = BLOCK_SIZE, reserved: int = 0) -> None:
        """``reserved`` low block ids are never handed out (block 0 can serve as the padding
        target of unused block-table entries)."""
        if num_blocks <= reserved:
            raise ValueError("pool needs at least one allocatable block")
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.reserved = reserved
        self.ref = [0] * num_blocks
        self._free = list(range(num_blocks - 1, reserved - 1, -1))   # pop() yields low ids first

    @property
    def free_blocks(self) -> int:
        return len(self._free)

    @property
    def used_blocks(self) -> int:
        return self.num_blocks - self.reserved - len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfBlocks("no free KV block")
        b = self._free.pop()
        assert self.ref[b] == 0
        self.ref[b] = 1
        return b

    def incref(self, block: int) -> None:
        assert self.ref[block] > 0, f"incref of free block {block}"
        self.ref[block] += 1

    def decref(self, block: int) -> None:
        assert self.ref[block] > 0, f"decref of free block {block}"
        self.ref[block] -= 1
        if self.ref[block] == 0:
            self._free.append(block)

    def shared(self, block: int) -> bool:
        return self.ref[block] > 1

    def check(self) -> None:
        """Invariant check used by tests: free list and counts agree."""
        free = set(self._free)
        assert len(free) == len(self._free), "duplicate entry in the free list"
        for b in range(self.reserved, self.num_blocks):
            assert (self.ref[b] == 0) == (b in free), f"block {b}: ref {self.ref[b]} vs free list"


class SeqBlocks:
    """Block table of one sequence.

    ``length`` tokens are committed; ``reserve(n)`` makes the table long enough for ``n`` more
    tokens and un-shares the block that will be written first.
    """

    def __init__(self, pool: BlockPool, copy_block: Callable[[int, int], None] | None = None) -> None:
        self.pool = pool
        self.copy_block = copy_block
        self.table: list[int] = []
        self.length = 0

    def adopt(self, blocks: list[int], length: int) -> None:
        """Start from shared prefix blocks (already incref'ed for this sequence)."""
        assert not self.table and length <= len(blocks) * self.pool.block_size
        self.table = list(blocks)
        self.length = length

    def blocks_needed(self, n: int) -> int:
        bs = self.pool.block_size
        need = (self.length + n + bs - 1) // bs - len(self.table)
        cow = 1 if (self.table and self.length % bs and self.length // bs < len(self.table)
                    and self.pool.shared(self.table[self.length // bs])) else 0
        return max(0, need) + cow

    def reserve(self, n: int) -> None:
        """Room for ``n`` more tokens. Raises ``OutOfBlocks`` without side effects on the table
        length (blocks already appended stay owned and are reused by the retry)."""
        bs = self.pool.block_size
        first = self.length // bs
        if first < len(self.table) and self.pool.shared(self.table[first]):
            # the block that receives the next token is shared: private copy first
            fresh = self.pool.alloc()
            if self.copy_block is not None and self.length % bs:
                self.copy_block(self.table[first], fresh)
            self.pool.decref(self.table[first])
            self.table[first] = fresh
        while len(self.table) * bs < self.length + n:
            self.table.append(self.pool.alloc())

    def commit(self, n: int) -> None:
        self.length += n
        assert self.length <= len(self.table) * self.pool.block_size

    def truncate(self, length: int) -> None:
        """Drop tokens beyond ``length`` (speculative rollback) and the blocks they alone used."""
        bs = self.pool.block_size
        keep = (length + bs - 1) // bs
        for b in self.table[keep:]:
            self.pool.decref(b)
        del self.table[keep:]
        self.length = length

    def free(self) -> None:
        for b in self.table:
            self.pool.decref(b)
        self.table = []
        self.length = 0
