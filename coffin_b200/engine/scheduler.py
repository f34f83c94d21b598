"""Continuous-batching scheduler: who runs in the next forward, and as what.

One engine step is either a *decode* step (every RUNNING sequence advances one token, rows
padded to a bucket) or a *prefill* step (one quantum of prompt tokens of one or more admitted
sequences).  The two never mix in one forward (the kernels for the two regimes differ), and
they alternate while both kinds of work exist, so a long prompt cannot starve running
streams and running streams cannot starve admission.  A sequence is admitted when a state
slot is free; KV blocks are claimed chunk by chunk, so admission never over-commits the
pool, and when the pool runs dry the most recently arrived running sequence is preempted
and later recomputed.  Reference: ``engine/scheduler.py:144-427``.
"""
from __future__ import annotations

import collections
import dataclasses
import time

from .config import EngineConfig
from .sequence import Sequence, SequenceStatus

PREEMPT_COOLDOWN = 1


@dataclasses.dataclass
class Batch:
    kind: str                                   # "decode" | "prefill" | "idle"
    seqs: list[Sequence] = dataclasses.field(default_factory=list)
    chunks: list[int] = dataclasses.field(default_factory=list)   # prefill: tokens per sequence


class Scheduler:
    def __init__(self, cfg: EngineConfig) -> None:
        self.cfg = cfg
        self.waiting: collections.deque[Sequence] = collections.deque()
        self.prefilling: list[Sequence] = []
        self.running: list[Sequence] = []
        self.free_slots = list(range(cfg.max_num_seqs - 1, -1, -1))
        self._last_kind = "decode"
        self._hold_since: float | None = None

    # ------------------------------------------------------------------ queue ops
    def add(self, seq: Sequence) -> None:
        seq.status = SequenceStatus.WAITING
        self.waiting.append(seq)

    def has_work(self) -> bool:
        return bool(self.waiting or self.prefilling or self.running)

    def _has_room(self) -> bool:
        return bool(self.free_slots)

    def _admit(self) -> Sequence | None:
        if not self.waiting or not self._has_room():
            return None
        seq = self.waiting.popleft()
        seq.slot = self.free_slots.pop()
        seq.status = SequenceStatus.PREFILLING
        self.prefilling.append(seq)
        return seq

    # ------------------------------------------------------------------ policy
    def schedule(self) -> Batch:
        """Pick the next forward. Admits waiting sequences into free slots first."""
        newly = []
        while True:
            s = self._admit()
            if s is None:
                break
            newly.append(s)
        self.admitted = newly
        want_prefill = bool(self.prefilling)
        want_decode = bool(self.running)
        if want_prefill and (not want_decode or self._last_kind == "decode"):
            return self._schedule_prefill()
        if want_decode:
            if self._hold_for_batch():
                return Batch("idle")
            self._last_kind = "decode"
            for s in self.running:
                s.cooldown = max(0, s.cooldown - 1)
            return Batch("decode", list(self.running))
        return Batch("idle")

    def _hold_for_batch(self) -> bool:
        """Optionally hold a lone decode for a few ms so that a burst of arrivals shares its
        steps (``batch_window_ms``)."""
        w = self.cfg.batch_window_ms
        if w <= 0 or len(self.running) != 1 or not self.waiting:
            self._hold_since = None
            return False
        now = time.monotonic()
        if self._hold_since is None:
            self._hold_since = now
        if (now - self._hold_since) * 1e3 < w:
            return True
        self._hold_since = None
        return False

    def _schedule_prefill(self) -> Batch:
        budget = self.cfg.max_num_batched_tokens
        quantum = min(self.cfg.prefill_quantum, self.cfg.chunk)
        seqs, chunks = [], []
        for s in self.prefilling:
            if budget <= 0:
                break
            n = min(s.remaining_prefill, quantum, budget)
            if n <= 0:
                continue
            seqs.append(s)
            chunks.append(n)
            budget -= n
        self._last_kind = "prefill"
        return Batch("prefill", seqs, chunks)

    # ------------------------------------------------------------------ transitions
    def prefill_done(self, seq: Sequence) -> None:
        self.prefilling.remove(seq)
        seq.status = SequenceStatus.RUNNING
        seq.cooldown = PREEMPT_COOLDOWN
        self.running.append(seq)

    def finish(self, seq: Sequence, reason: str) -> None:
        for lst in (self.running, self.prefilling):
            if seq in lst:
                lst.remove(seq)
        try:
            self.waiting.remove(seq)
        except ValueError:
            pass
        if seq.slot is not None:
            self.free_slots.append(seq.slot)
            seq.slot = None
        seq.finish(reason)

    def expire(self, now: float | None = None) -> list[Sequence]:
        """Sequences past their deadline (the caller finishes them with reason ``timeout``)."""
        now = now if now is not None else time.monotonic()
        return [s for s in list(self.waiting) + self.prefilling + self.running if s.over_budget(now)]

    def preempt_victim(self, exclude: Sequence | None = None) -> Sequence | None:
        """Latest-arrived resident sequence that is not cooling down (LIFO keeps the oldest
        streams making progress)."""
        cands = [s for s in self.running + self.prefilling if s is not exclude and s.cooldown == 0]
        if not cands:
            cands = [s for s in self.running + self.prefilling if s is not exclude]
        return max(cands, key=lambda s: s.arrival) if cands else None

    def park(self, seq: Sequence) -> None:
        """Move a preempted sequence back to the head of the waiting queue."""
        for lst in (self.running, self.prefilling):
            if seq in lst:
                lst.remove(seq)
        if seq.slot is not None:
            self.free_slots.append(seq.slot)
        seq.park_preempted()
        seq.resume()
        self.waiting.appendleft(seq)

    def stats(self) -> dict:
        return {"waiting": len(self.waiting), "prefilling": len(self.prefilling), "running": len(self.running),
                "free_slots": len(self.free_slots)}
