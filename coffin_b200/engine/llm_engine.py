"""``LLMEngine``: request lifecycle around the scheduler, the block manager and the runner.

``add_request`` queues a sequence; every ``step()`` runs exactly one forward (a decode step of
all running rows, or one prefill quantum) and returns the tokens it produced.  Capacity is
claimed lazily: before a decode step every row reserves room for one more token, and when the
pool (after evicting cached blocks) cannot provide it the latest-arrived sequence is preempted
and recomputed later.  A run of steps that makes no progress raises instead of spinning.
Reference: ``engine/llm_engine.py:113-657`` (``step`` l.206-240, ``_check_progress`` l.242,
``_make_room_for_decode/_preempt`` l.388-473).
"""
from __future__ import annotations

import dataclasses
import os
import time
from typing import Any, Iterable, Iterator

from .block_manager import BlockManager
from .config import EngineConfig
from .model_runner import ModelRunner
from .scheduler import Scheduler
from .sequence import SamplingParams, Sequence, SequenceStatus

NO_PROGRESS_LIMIT = 200
#: ``COFFIN_DEBUG_STEP=1``: every 50 steps print what the scheduler really holds (reference
#: ``engine/llm_engine.py:27-32``).
DEBUG_STEP = bool(os.environ.get("COFFIN_DEBUG_STEP"))
DEBUG_STEP_EVERY = 50


@dataclasses.dataclass
class StepOutput:
    seq: Sequence
    token: int | None
    finished: bool


class LLMEngine:
    def __init__(self, model, cfg: EngineConfig | None = None, bm: BlockManager | None = None) -> None:
        self.cfg = cfg or EngineConfig()
        if self.cfg.spec_sparse_k > 0:
            raise NotImplementedError("spec_sparse_k > 0 (batched verify over the k best history blocks of a row) needs a "
                                      "masked multi-query verify kernel that does not exist; pass spec_sparse_k=0")
        self.model = model
        slots = getattr(model, "num_slots", self.cfg.max_num_seqs)
        # a model may carry fewer rows per step than the configuration asks for (state slots, or the
        # bucket limit of a multi-rank model): clamp instead of failing in the middle of a step
        rows = getattr(model, "max_decode_rows", None)
        limit = min(slots, rows) if rows else slots
        if limit < self.cfg.max_num_seqs:
            print(f"[engine] max_num_seqs {self.cfg.max_num_seqs} -> {limit} (model limit)", flush=True)
            self.cfg = dataclasses.replace(self.cfg, max_num_seqs=limit)
        self.bm = bm or BlockManager(model, getattr(model, "num_blocks", None), self.cfg.block_size,
                                     self.cfg.snapshots, self.cfg.prefix_cache)
        self.scheduler = Scheduler(self.cfg)
        self.runner = ModelRunner(model, self.bm, self.cfg)
        self.runner.live_seqs = lambda: self.scheduler.prefilling + self.scheduler.running
        self.max_seq = min(self.cfg.max_seq, getattr(model, "max_seq", self.cfg.max_seq))
        self._stall = 0
        self.n_steps = 0
        self.n_preempt = 0
        self.n_finished = 0

    @classmethod
    def build(cls, model, cfg: EngineConfig | None = None) -> "LLMEngine":
        eng = cls(model, cfg)
        if eng.cfg.graph and hasattr(model, "capture"):
            for m in (1,):
                model.capture(m)
        return eng

    def warmup(self) -> float:
        """Pay the one-time costs before the first request: a prefill chunk (workspaces, kernel attributes)
        on a scratch slot and the CUDA graph of every decode bucket the configuration can reach.  Without
        it the first few dozen requests of a busy server wait behind seven graph captures (their TTFT was
        2-4 s in a 16 request/s run whose steady state is 20 ms).  Returns the seconds spent; a model
        without graphs or on the CPU only runs the prefill."""
        t0 = time.monotonic()
        m = self.model
        dev = getattr(m, "device", None)
        if (not hasattr(m, "prefill") or not hasattr(m, "zero_state") or self.scheduler.has_work()
                or getattr(dev, "type", "cpu") != "cuda"):
            return 0.0
        if max(getattr(m, "tp_world", 1), getattr(m, "ep_world", 1), getattr(m, "pp_world", 1)) > 1:
            return 0.0          # multi-rank steps are collective: the ranks warm up with their first request
        import torch
        n = max(1, min(self.cfg.chunk, getattr(m, "max_chunk", self.cfg.chunk), self.max_seq - 1))
        per = -(-n // self.cfg.block_size)
        blocks = getattr(m, "max_blocks_per_seq", per)
        if per > blocks or per + 1 > getattr(m, "num_blocks", per + 1):
            return 0.0
        table = torch.arange(1, per + 1, dtype=torch.int32, device=dev)      # pages nobody owns yet: their contents are never read
        vocab = int(getattr(getattr(m, "cfg", None), "vocab_size", 2))
        with torch.no_grad():
            for size in sorted({n, min(n, 64)}, reverse=True):
                m.zero_state(0)
                m.prefill(torch.ones(size, dtype=torch.int64, device=dev) % vocab, 0, 0, table[:-(-size // self.cfg.block_size)],
                          want_logits=False)
            m.zero_state(0)
            if self.cfg.graph and hasattr(m, "capture") and getattr(dev, "type", "cpu") == "cuda":
                buckets = getattr(m, "BUCKETS_ALL", None) or (1, 2, 4, 8, 16, 32, 64)
                for M in buckets:
                    if M <= max(1, self.cfg.max_num_seqs) * 2 - 1 and M <= getattr(m, "max_decode_rows", M):
                        try:
                            m.capture(M)
                        except (NotImplementedError, ValueError):
                            break
            if dev is not None and getattr(dev, "type", "cpu") == "cuda":
                torch.cuda.synchronize(dev)
        return time.monotonic() - t0

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt: list[int], params: SamplingParams | None = None, mm: Any | None = None,
                    request_id: str | None = None) -> Sequence:
        params = params or SamplingParams()
        if len(prompt) >= self.max_seq:
            raise ValueError(f"prompt of {len(prompt)} tokens does not fit the {self.max_seq}-token window")
        if params.deadline is None and self.cfg.max_seconds > 0:
            params = dataclasses.replace(params, deadline=time.monotonic() + self.cfg.max_seconds)
        seq = Sequence(prompt, params, mm, request_id)
        self.scheduler.add(seq)
        return seq

    def abort(self, seq: Sequence, reason: str = "abort") -> None:
        if not seq.finished:
            self._release(seq, reason)

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    # ------------------------------------------------------------------ the step
    def step(self) -> list[StepOutput]:
        out: list[StepOutput] = []
        self.n_steps += 1
        for seq in self.scheduler.expire():
            self._release(seq, "timeout")
            out.append(StepOutput(seq, None, True))
        batch = self.scheduler.schedule()
        if DEBUG_STEP and self.n_steps % DEBUG_STEP_EVERY == 0:
            print(self.debug_line(batch.kind), flush=True)
        for seq in self.scheduler.admitted:
            self.runner.begin_prefill(seq)
        progressed = False
        if batch.kind == "prefill":
            progressed = self._run_prefill(batch, out)
        elif batch.kind == "decode":
            progressed = self._run_decode(batch.seqs, out)
        self._check_progress(progressed or bool(out), batch.kind)
        return out

    def debug_line(self, kind: str = "") -> str:
        """One line with the scheduler's queues and the free blocks; printed every 50th step under
        ``COFFIN_DEBUG_STEP``."""
        sch = self.scheduler
        return (f"[step] n={self.n_steps} kind={kind} running={len(sch.running)} prefilling={len(sch.prefilling)} "
                f"waiting={len(sch.waiting)} max_seqs={self.cfg.max_num_seqs} free_slots={len(sch.free_slots)} "
                f"free_blocks={self.bm.pool.free_blocks} stall={self._stall}")

    def _check_progress(self, progressed: bool, kind: str) -> None:
        if progressed or kind == "idle" and not self.scheduler.has_work():
            self._stall = 0
            return
        self._stall += 1
        if self._stall >= NO_PROGRESS_LIMIT:
            raise RuntimeError(f"engine made no progress in {NO_PROGRESS_LIMIT} steps: "
                               f"{self.scheduler.stats()} {self.bm.stats()}")

    # ------------------------------------------------------------------ prefill
    def _run_prefill(self, batch, out: list[StepOutput]) -> bool:
        progressed = False
        todo = [(seq, n) for seq, n in zip(batch.seqs, batch.chunks)
                if not seq.finished and seq.status is SequenceStatus.PREFILLING]
        if not todo:
            return False
        done = self.runner.prefill_many([s for s, _ in todo], [n for _, n in todo])
        for seq, _n in todo:
            if done.get(seq.seq_id, 0) == 0:
                # no room even for one chunk: take blocks back from someone else
                victim = self.scheduler.preempt_victim(exclude=seq)
                if victim is not None and victim.status is not SequenceStatus.FINISHED:
                    self._preempt(victim)
                continue
            if seq.finished or seq.status is not SequenceStatus.PREFILLING:
                continue                                  # preempted by an earlier sequence of this batch
            progressed = True
            if seq.remaining_prefill == 0:
                self.runner.finish_prefill(seq)
                self.scheduler.prefill_done(seq)
                tok = self.runner.sample([seq], seq.pending_logits.reshape(1, -1))[0]
                seq.pending_logits = None
                if seq.first_token_time is None:
                    seq.first_token_time = time.monotonic()
                self._commit(seq, tok, out)
        return progressed

    # ------------------------------------------------------------------ decode
    def _run_decode(self, seqs: list[Sequence], out: list[StepOutput]) -> bool:
        ready = []
        for seq in list(seqs):
            if seq.finished or seq.status is not SequenceStatus.RUNNING:
                continue
            while not self.bm.ensure_blocks(seq.blocks, 1):
                victim = self.scheduler.preempt_victim(exclude=None)
                if victim is None:
                    break
                self._preempt(victim)
                if victim is seq:
                    break
            if seq.status is SequenceStatus.RUNNING:
                ready.append(seq)
        ready = [s for s in ready if s.status is SequenceStatus.RUNNING]
        if not ready:
            return False
        tokens = [s.output[-1] for s in ready]
        if self._run_spec(ready, tokens, out):
            return True
        logits = self.runner.decode(ready, tokens)
        greedy = getattr(self.runner, "_last_next", None)
        picked = self.runner.sample(ready, logits, greedy)
        for seq, tok in zip(ready, picked):
            self._commit(seq, tok, out)
        return True

    def _run_spec(self, ready: list[Sequence], tokens: list[int], out: list[StepOutput]) -> bool:
        """Speculative step: when a greedy row has drafts (and the configuration allows it), verify all
        rows' drafts in one pass and commit, per row, the model's own tokens for the accepted prefix
        plus one.  Speculation only changes speed: a draft is accepted only if it equals the model's
        arg-max, so the tokens are those of plain greedy decoding.  Returns False when a plain step
        should run instead (no drafts, no room for the draft window)."""
        if not (self.cfg.spec_k > 0 or any(s.params.spec_k > 0 for s in ready)):
            return False
        drafts = self.runner.draft(ready)
        if drafts is None:
            return False
        C = self.runner.spec_width(drafts)
        for seq in ready:
            if seq.num_computed + C > self.max_seq or not self.bm.ensure_blocks(seq.blocks, C):
                return False
        new_tokens, first_logits = self.runner.spec_step(ready, tokens, drafts, C)
        sampled = [s for s in ready if s.params.temperature > 0]
        if sampled:
            idx = [i for i, s in enumerate(ready) if s.params.temperature > 0]
            picked = self.runner.sample(sampled, first_logits[idx])
            for i, tok in zip(idx, picked):
                new_tokens[i] = [tok]
        for seq, toks in zip(ready, new_tokens):
            for tok in toks:
                self._commit(seq, tok, out)
                if seq.finished:
                    break
        return True

    def _preempt(self, seq: Sequence) -> None:
        self.n_preempt += 1
        self.bm.release(seq.blocks)
        self.scheduler.park(seq)

    # ------------------------------------------------------------------ commit / release
    def _commit(self, seq: Sequence, tok: int, out: list[StepOutput]) -> None:
        p = seq.params
        if not p.ignore_eos and tok in p.eos:
            self._release(seq, "stop")
            out.append(StepOutput(seq, None, True))
            return
        seq.output.append(tok)
        reason = None
        if len(seq.output) >= p.max_tokens:
            reason = "length"
        elif seq.num_tokens >= self.max_seq:
            reason = "window"
        if reason:
            self._release(seq, reason)
        out.append(StepOutput(seq, tok, reason is not None))

    def _release(self, seq: Sequence, reason: str) -> None:
        self.bm.release(seq.blocks)
        seq.blocks = None
        self.runner.forget(seq)
        self.scheduler.finish(seq, reason)
        self.n_finished += 1

    # ------------------------------------------------------------------ conveniences
    def generate(self, prompts: Iterable[list[int]], params: SamplingParams | None = None) -> list[Sequence]:
        seqs = [self.add_request(p, params) for p in prompts]
        while any(not s.finished for s in seqs):
            self.step()
        return seqs

    def stream(self, seq: Sequence) -> Iterator[int]:
        """Yield the tokens of ``seq`` as the engine produces them (drives ``step`` itself)."""
        sent = 0
        while True:
            while sent < len(seq.output):
                yield seq.output[sent]
                sent += 1
            if seq.finished:
                return
            self.step()

    def reset(self) -> None:
        """Drop every request and the prefix cache (the recovery path after a failed step)."""
        for seq in list(self.scheduler.waiting) + self.scheduler.prefilling + self.scheduler.running:
            self.bm.release(seq.blocks)
            seq.blocks = None
            self.scheduler.finish(seq, "reset")
        self.bm.radix.clear()
        self._stall = 0

    def stats(self) -> dict:
        return {"steps": self.n_steps, "finished": self.n_finished, "preempted": self.n_preempt,
                "queue": self.scheduler.stats(), "blocks": self.bm.stats(), "runner": self.runner.stats()}
