"""Request state: sampling parameters, the sequence object and its status machine.

WAITING -> PREFILLING -> RUNNING -> FINISHED, with PREEMPTED as the parking state of a
sequence whose blocks were taken back (it re-enters as WAITING and recomputes its prompt
plus the tokens generated so far).  Reference: ``engine/sequence.py:27-241``.
"""
from __future__ import annotations

import dataclasses
import enum
import itertools
import time
from typing import Any

from ..cache.paged_cache import SeqBlocks


class SequenceStatus(enum.Enum):
    WAITING = "waiting"
    PREFILLING = "prefilling"
    RUNNING = "running"
    PREEMPTED = "preempted"
    FINISHED = "finished"


@dataclasses.dataclass
class SamplingParams:
    temperature: float = 0.0
    max_tokens: int = 256
    ignore_eos: bool = False
    eos: tuple[int, ...] = ()
    deadline: float | None = None       # absolute time.monotonic() limit
    seed: int | None = None
    spec_k: int = -1                    # speculative draft length: -1 = the engine's default, 0 = off

    def __post_init__(self) -> None:
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")


_ids = itertools.count()


class Sequence:
    def __init__(self, prompt: list[int], params: SamplingParams, mm: Any | None = None,
                 request_id: str | None = None) -> None:
        if not prompt:
            raise ValueError("empty prompt")
        self.seq_id = next(_ids)
        self.request_id = request_id or f"req-{self.seq_id}"
        self.prompt = list(prompt)
        self.params = params
        self.mm = mm
        self.output: list[int] = []
        self.status = SequenceStatus.WAITING
        self.finish_reason: str | None = None
        self.slot: int | None = None            # model state slot while resident
        self.blocks: SeqBlocks | None = None
        self.num_computed = 0                   # tokens whose KV/state are in the model
        self.cached_tokens = 0                  # of which came from the prefix cache
        self.pending_logits = None              # logits of the last computed position
        self.arrival = time.monotonic()
        self.first_token_time: float | None = None
        self.finish_time: float | None = None
        self.n_preempted = 0
        self.cooldown = 0                       # engine steps before it may be preempted again
        self.snap_marks: dict[int, Any] = {}    # token count -> delta-net snapshot (for the cache)
        self.rope_delta = 0
        # speculative decoding (greedy rows): host-side drafter and its acceptance counters
        self.drafter = None
        self.drafter_seen = 0                   # tokens of all_tokens the drafter has observed
        self.spec_drafted = 0
        self.spec_accepted = 0
        self.spec_steps = 0

    # tokens the model must have seen before the next sample: prompt + generated so far
    @property
    def all_tokens(self) -> list[int]:
        return self.prompt + self.output

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def remaining_prefill(self) -> int:
        """Tokens still to run through prefill: everything except the position that samples."""
        return self.num_tokens - self.num_computed

    @property
    def finished(self) -> bool:
        return self.status is SequenceStatus.FINISHED

    def over_budget(self, now: float | None = None) -> bool:
        d = self.params.deadline
        return d is not None and (now if now is not None else time.monotonic()) > d

    def park_preempted(self) -> None:
        """Forget device residency; generated tokens are kept and recomputed on resume."""
        self.status = SequenceStatus.PREEMPTED
        self.slot = None
        self.blocks = None
        self.num_computed = 0
        self.cached_tokens = 0
        self.pending_logits = None
        self.snap_marks = {}
        self.n_preempted += 1

    def resume(self) -> None:
        self.status = SequenceStatus.WAITING

    def finish(self, reason: str) -> None:
        self.status = SequenceStatus.FINISHED
        self.finish_reason = reason
        self.finish_time = time.monotonic()
