"""``ModelRunner``: turns scheduler decisions into model calls.

It owns nothing but staging: token tensors, block tables, sampling.  A model is anything with
the slot/block-table interface of ``models.qwen35.model.Qwen35Model`` (``prefill``,
``set_rows``/``decode``, ``zero_state``/``snapshot_state``/``restore_state``, ``copy_block``,
``sample``); the CPU twin in ``oracle/engine_model.py`` and the fake models of the tests
implement the same calls.  Reference: ``engine/model_runner.py:216-924`` (chunked prefill
l.331-515, prefix insertion l.517-571, batched decode l.829-879, sampling l.900-924).
"""
from __future__ import annotations

import random
import time

import torch

from . import debug
from .block_manager import BlockManager
from .config import EngineConfig
from .sequence import Sequence

BATCH_BUCKETS = (1, 2, 4, 8, 16, 32, 64)


class ModelRunner:
    def __init__(self, model, bm: BlockManager, cfg: EngineConfig) -> None:
        self.model = model
        self.bm = bm
        self.cfg = cfg
        self.device = getattr(model, "device", torch.device("cpu"))
        self.block_size = bm.pool.block_size
        self._rng: dict[int, random.Random] = {}
        self.n_prefill_tokens = 0
        self.n_decode_steps = 0
        self.n_cached_tokens = 0
        self.n_spec_steps = self.n_spec_drafted = self.n_spec_accepted = 0
        self.n_prefill_groups = 0
        # device status words (bounded waits that ran out): queued after every model call, looked at
        # after the next synchronisation (the token read-back in ``sample``)
        self._poll = getattr(model, "poll_status", None)
        self._check = getattr(model, "check_status", None)

    live_seqs = None      # callable returning the sequences that hold blocks (set by the engine; used by the debug checks)

    def live(self) -> list:
        return list(self.live_seqs()) if self.live_seqs is not None else []

    # ------------------------------------------------------------------ admission
    def begin_prefill(self, seq: Sequence) -> None:
        """Give a freshly admitted sequence its block table; reuse a cached prefix if one
        matches (KV blocks by reference, delta-net state restored from the snapshot)."""
        seq.blocks = self.bm.new_table()
        toks = seq.all_tokens
        blocks, n, state = self.bm.match_prefix(toks, seq.mm)
        if debug.PC_TRACE:
            print(f"[pctrace] seq={seq.seq_id} prompt={len(toks)} matched={n} blocks={len(blocks) if n else 0} "
                  f"snapshot={'yes' if state is not None else 'no'}", flush=True)
        if n:
            seq.blocks.adopt(blocks, n)
            self.model.restore_state(seq.slot, state)
            seq.num_computed = n
            seq.cached_tokens = n
            self.n_cached_tokens += n
        else:
            self.model.zero_state(seq.slot)
            seq.num_computed = 0
            seq.cached_tokens = 0
        seq.snap_marks = {}

    # ------------------------------------------------------------------ prefill
    def _chunk_end(self, seq: Sequence, n: int) -> int:
        """End of the next chunk: at most ``n`` tokens, cut at the next snapshot boundary and at
        the last block boundary before the sampling position (so that the longest reusable
        prefix of this prompt gets a state snapshot)."""
        start, total = seq.num_computed, seq.num_tokens
        end = min(total, start + n, start + self.cfg.chunk)
        if self.bm.prefix_cache:
            iv = max(self.block_size, self.cfg.snapshot_interval // self.block_size * self.block_size)
            nxt = (start // iv + 1) * iv
            tail = (total - 1) // self.block_size * self.block_size
            for cut in (nxt, tail):
                if start < cut < end:
                    end = cut
        return end

    def prefill_chunk(self, seq: Sequence, n: int) -> int:
        """Run up to ``n`` more tokens of ``seq``.  Returns the tokens computed (0 = no room)."""
        done = 0
        while done < n and seq.remaining_prefill > 0:
            start = seq.num_computed
            end = self._chunk_end(seq, n - done)
            T = end - start
            if not self.bm.ensure_blocks(seq.blocks, T):
                break
            toks = seq.all_tokens[start:end]
            last = end == seq.num_tokens
            embeds = cos_sin = None
            if seq.mm is not None:
                embeds, cos_sin = self._mm_chunk(seq, toks, start, end)
            if debug.KV_TRACE:
                debug.check_block_alias(self.live(), self.block_size, "prefill", {seq.seq_id: T}, verbose=True)
            t0 = time.perf_counter() if debug.PREFILL_TRACE else 0.0
            logits = self.model.prefill(self._tokens(toks), start, seq.slot, self._table(seq),
                                        embeds=embeds, cos_sin=cos_sin, want_logits=last)
            if debug.PREFILL_TRACE:
                debug.prefill_trace(seq, start, end, t0, self.device)
            if self._poll is not None:
                self._poll()
            self._chunk_done(seq, end, logits)
            done += T
        return done

    def _chunk_done(self, seq: Sequence, end: int, logits) -> None:
        """Bookkeeping after the tokens ``[num_computed, end)`` of ``seq`` ran."""
        T = end - seq.num_computed
        last = end == seq.num_tokens
        seq.blocks.commit(T)
        seq.num_computed = end
        self.n_prefill_tokens += T
        if last:
            seq.pending_logits = logits
        if self.bm.prefix_cache and end % self.block_size == 0 and not last:
            iv = max(self.block_size, self.cfg.snapshot_interval // self.block_size * self.block_size)
            tail = (seq.num_tokens - 1) // self.block_size * self.block_size
            if end % iv == 0 or end == tail:
                seq.snap_marks[end] = self.model.snapshot_state(seq.slot)

    def prefill_many(self, seqs: list[Sequence], budgets: list[int]) -> dict[int, int]:
        """Run the scheduled prefill quanta of several sequences.  Chunks of text-only sequences share
        forwards (``model.prefill_group``: one GEMM over the stacked rows per projection), so a burst of
        short prompts costs about one pass over the weights instead of one per prompt.  Chunks are still
        cut at snapshot boundaries, so a sequence may take part in several rounds of one call.
        Returns ``{seq_id: tokens computed}`` (0 = no room for that sequence)."""
        done = {s.seq_id: 0 for s in seqs}
        group_fn = getattr(self.model, "prefill_group", None)
        text = [s for s in seqs if s.mm is None]
        if group_fn is None or len(text) < 2 or not self.cfg.group_prefill:
            for s, n in zip(seqs, budgets):
                done[s.seq_id] = self.prefill_chunk(s, n)
            return done
        budget = {s.seq_id: n for s, n in zip(seqs, budgets)}
        for s in seqs:
            if s.mm is not None:
                done[s.seq_id] = self.prefill_chunk(s, budget[s.seq_id])
        cap = getattr(self.model, "max_chunk", self.cfg.chunk)
        stuck: set[int] = set()
        while True:
            group, total = [], 0
            for s in text:
                left = budget[s.seq_id] - done[s.seq_id]
                if left <= 0 or s.remaining_prefill <= 0 or s.seq_id in stuck:
                    continue
                end = self._chunk_end(s, left)
                T = end - s.num_computed
                if total + T > cap:
                    continue
                if not self.bm.ensure_blocks(s.blocks, T):
                    stuck.add(s.seq_id)
                    continue
                group.append((s, end))
                total += T
            if not group:
                break
            items = [(self._tokens(s.all_tokens[s.num_computed:end]), s.num_computed, s.slot, self._table(s)) for s, end in group]
            want = [end == s.num_tokens for s, end in group]
            outs = group_fn(items, want_logits=want)
            if self._poll is not None:
                self._poll()
            self.n_prefill_groups += 1
            for (s, end), lg in zip(group, outs):
                done[s.seq_id] += end - s.num_computed
                self._chunk_done(s, end, lg)
        return done

    def finish_prefill(self, seq: Sequence) -> None:
        """Publish the computed prompt blocks (and their snapshots) to the prefix cache."""
        if self.bm.prefix_cache and seq.snap_marks:
            self.bm.insert(seq.all_tokens[:seq.num_computed], seq.blocks.table, seq.snap_marks, seq.mm)
        seq.snap_marks = {}

    def _mm_chunk(self, seq: Sequence, toks, start: int, end: int):
        mm = seq.mm
        embeds = cos_sin = None
        if getattr(mm, "embeds", None) is not None:
            x = self.model.embed_tokens(self._tokens(toks))
            embeds = mm.scatter_into(x, start, end)
        if getattr(mm, "positions", None) is not None:
            pos3 = mm.positions[:, start:end]
            L = mm.positions.shape[1]
            if end > L:
                # a preempted sequence re-prefills prompt + generated tokens: positions were built for the
                # prompt only, the text after it continues on all three axes at index + rope_delta
                tail = torch.arange(max(start, L), end, dtype=pos3.dtype) + int(mm.rope_delta)
                pos3 = torch.cat([pos3, tail.unsqueeze(0).expand(3, -1).to(pos3.device)], dim=1)
            cos_sin = self.model.mrope_rows(pos3)
            seq.rope_delta = int(mm.rope_delta)
        return embeds, cos_sin

    def _tokens(self, toks) -> torch.Tensor:
        t = torch.tensor(toks, dtype=torch.int64)
        if self.device.type == "cuda":
            return t.pin_memory().to(self.device, non_blocking=True)
        return t

    def _table(self, seq: Sequence) -> torch.Tensor:
        t = torch.tensor(seq.blocks.table, dtype=torch.int32)
        return t.to(self.device) if self.device.type == "cuda" else t

    # ------------------------------------------------------------------ decode
    def decode(self, seqs: list[Sequence], tokens: list[int]) -> torch.Tensor:
        """One decode step: ``tokens[i]`` is fed to ``seqs[i]`` at position ``num_computed``.
        Blocks must already be reserved.  Returns logits ``[len(seqs), vocab]``."""
        n = len(seqs)
        cap = BATCH_BUCKETS[-1]
        if debug.KV_TRACE:
            debug.check_block_alias(self.live() or seqs, self.block_size, "decode", verbose=True)
        if hasattr(self.model, "full_logits"):
            # a tensor-parallel step gathers the full-vocabulary logits only when a row samples from them
            self.model.full_logits = any(s.params.temperature > 0 for s in seqs)
        if n > cap:
            # more rows than the widest bucket: run them in groups (each group is one model step)
            parts, nxts = [], []
            for g0 in range(0, n, cap):
                grp = seqs[g0:g0 + cap]
                M = self.model.bucket_for(len(grp))
                self.model.set_rows(M, tokens[g0:g0 + cap], [s.num_computed for s in grp], [s.slot for s in grp],
                                    [s.blocks.table for s in grp], [s.rope_delta for s in grp])
                nx, lg = self.model.decode(M, graph=self.cfg.graph)
                parts.append(lg[:len(grp)].clone())
                nxts.append(nx[:len(grp)].clone())
            nxt, logits = torch.cat(nxts), torch.cat(parts)
        else:
            M = self.model.bucket_for(n)
            self.model.set_rows(M, tokens, [s.num_computed for s in seqs], [s.slot for s in seqs],
                                [s.blocks.table for s in seqs], [s.rope_delta for s in seqs])
            nxt, logits = self.model.decode(M, graph=self.cfg.graph)
        if self._poll is not None:
            self._poll()
        for s in seqs:
            s.blocks.commit(1)
            s.num_computed += 1
        self.n_decode_steps += 1
        self._last_next = nxt
        return logits[:n]

    # ------------------------------------------------------------------ speculative decoding
    @property
    def spec_capable(self) -> bool:
        return hasattr(self.model, "verify_batch") and hasattr(self.model, "commit_batch")

    def spec_k_of(self, seq: Sequence) -> int:
        """Draft length of a row: the request's own ``spec_k`` or the engine default; rows that sample
        with a temperature cannot be verified by arg-max and never draft."""
        if seq.params.temperature > 0 or not self.spec_capable:
            return 0
        k = seq.params.spec_k if seq.params.spec_k >= 0 else self.cfg.spec_k
        if seq.num_tokens < self.cfg.spec_min_ctx:
            return 0
        return max(0, min(7, int(k)))

    def draft(self, seqs: list[Sequence]) -> list[list[int]] | None:
        """Drafts per row from the rows' suffix drafters (``None`` when no row proposes anything, in
        which case a plain decode step is the better step)."""
        from ..utils.suffix import SuffixDrafter
        if len(seqs) > self.SPEC_MAX_ROWS or not (self.cfg.spec_batch or len(seqs) == 1):
            return None
        drafts, any_draft = [], False
        for s in seqs:
            k = self.spec_k_of(s)
            if k <= 0:
                drafts.append([])
                continue
            if s.drafter is None:
                s.drafter, s.drafter_seen = SuffixDrafter(), 0
            toks = s.all_tokens
            if s.drafter_seen < len(toks):
                s.drafter.observe(toks[s.drafter_seen:])
                s.drafter_seen = len(toks)
            room = self.model.max_seq - s.num_tokens - 1 if hasattr(self.model, "max_seq") else k
            d = s.drafter.draft(min(k, max(0, room)))
            drafts.append(d)
            any_draft = any_draft or bool(d)
        return drafts if any_draft else None

    SPEC_MAX_ROWS = 8

    @staticmethod
    def spec_width(drafts: list[list[int]]) -> int:
        need = max(len(d) for d in drafts) + 1
        for w in (2, 4, 8):
            if need <= w:
                return w
        return 8

    def spec_step(self, seqs: list[Sequence], tokens: list[int], drafts: list[list[int]], C: int):
        """One verify pass over all rows: row ``i`` feeds its pending token and its drafts (padded to
        ``C`` tokens).  Returns ``(new_tokens, first_logits)``: per row the model's own greedy tokens for
        the accepted prefix plus one (``new_tokens[i]`` has ``accepted + 1`` entries), and the logits of
        every row's first position (what a temperature row samples from).  The delta-net states
        advance by exactly the accepted tokens; KV rows of rejected positions are overwritten later."""
        rows, fed_all = [], []
        for s, tok, d in zip(seqs, tokens, drafts):
            fed = [tok] + list(d[:C - 1])
            fed_all.append(fed)
            rows.append((fed + [fed[-1]] * (C - len(fed)), s.num_computed, s.slot, s.blocks.table, s.rope_delta))
        logits = self.model.verify_batch(rows)                     # [n, C, vocab]
        if self._poll is not None:
            self._poll()
        preds = logits.argmax(-1).tolist()                         # the read-back synchronises with the pass
        if self._check is not None:
            self._check()
        new_tokens, steps = [], []
        for s, fed, p in zip(seqs, fed_all, preds):
            a = 0
            while a < len(fed) - 1 and fed[a + 1] == p[a]:
                a += 1
            new_tokens.append([int(t) for t in p[:a + 1]])
            steps.append(a + 1)
            if len(fed) > 1:
                s.spec_steps += 1
                s.spec_drafted += len(fed) - 1
                s.spec_accepted += a
                self.n_spec_drafted += len(fed) - 1
                self.n_spec_accepted += a
        self.model.commit_batch([s.slot for s in seqs], steps)
        for s, n in zip(seqs, steps):
            s.blocks.commit(n)
            s.num_computed += n
        self.n_decode_steps += 1
        self.n_spec_steps += 1
        return new_tokens, logits[:, 0]

    # ------------------------------------------------------------------ sampling
    def sample(self, seqs: list[Sequence], logits: torch.Tensor, greedy_tokens: torch.Tensor | None = None) -> list[int]:
        """Greedy rows take the argmax (already computed on the device by the decode step when
        ``greedy_tokens`` is given); temperature rows are drawn by inverse CDF from a uniform
        produced by the sequence's own seeded generator, so every tensor-parallel rank picks the
        same token without a broadcast."""
        picked = self._sample(seqs, logits, greedy_tokens)     # the read-back synchronises with the step
        if self._check is not None:
            self._check()
        return picked

    def _sample(self, seqs: list[Sequence], logits: torch.Tensor, greedy_tokens: torch.Tensor | None) -> list[int]:
        temps = [s.params.temperature for s in seqs]
        if all(t <= 0 for t in temps):
            if greedy_tokens is not None:
                return [int(v) for v in greedy_tokens[:len(seqs)].tolist()]
            return [int(v) for v in self.model.sample(logits, None, None).tolist()]
        us = []
        for s in seqs:
            rng = self._rng.get(s.seq_id)
            if rng is None:
                rng = self._rng[s.seq_id] = random.Random(s.params.seed if s.params.seed is not None else s.seq_id)
            us.append(rng.random())
        return [int(v) for v in self.model.sample(logits, temps, us).tolist()]

    def forget(self, seq: Sequence) -> None:
        self._rng.pop(seq.seq_id, None)

    def stats(self) -> dict:
        return {"prefill_tokens": self.n_prefill_tokens, "decode_steps": self.n_decode_steps,
                "cached_tokens": self.n_cached_tokens, "prefill_groups": self.n_prefill_groups,
                "spec": {"steps": self.n_spec_steps, "drafted": self.n_spec_drafted, "accepted": self.n_spec_accepted}}
