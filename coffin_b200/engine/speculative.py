"""Speculative decoding: draft a few tokens cheaply, verify them in one model pass.

Drafts come from the host-side ``SuffixDrafter`` (or any object with ``observe``/``draft``, such
as the MTP head's drafter).  One ``model.verify`` pass scores the last sampled token plus the
drafts; the longest prefix of drafts that equals the model's own greedy choices is accepted, the
model's choice after it comes for free, and ``model.commit`` advances the delta-net state by
exactly the accepted tokens (KV rows of rejected positions are simply overwritten later).  Greedy
output is therefore the same as plain decoding up to kernel rounding.
Reference: ``models/qwen35/model.py:1832-1950`` (``spec_step`` / ``spec_generate``),
``docs/FACTS-RUNTIME.md:31-43`` (when it pays off).
"""
from __future__ import annotations

import torch

from ..utils.suffix import SuffixDrafter

WIDTHS = (2, 4, 8)


class SpeculativeDecoder:
    def __init__(self, model, k: int = 3, drafter=None, slot: int = 0) -> None:
        self.model = model
        self.k = max(1, min(7, k))
        self.drafter = drafter or SuffixDrafter()
        self.slot = slot
        self.n_steps = self.n_drafted = self.n_accepted = self.n_plain = 0

    def _width(self, n_draft: int) -> int:
        for w in WIDTHS:
            if n_draft + 1 <= w:
                return w
        return WIDTHS[-1]

    def _table(self, table: list[int]) -> torch.Tensor:
        return torch.tensor(table, dtype=torch.int32, device=getattr(self.model, "device", "cpu"))

    def verify_only(self, table: list[int], tokens: list[int], pos: int) -> torch.Tensor:
        """One verify pass that accepts everything (timing aid of the ``verify`` op)."""
        logits = self.model.verify(tokens, pos, self.slot, self._table(table))
        self.model.commit(self.slot, len(tokens))
        return logits

    def step(self, table: list[int], tok: int, pos: int) -> list[int]:
        """Advance by at least one token. ``tok`` is the last sampled token (not yet run) at
        position ``pos``.  Returns the new tokens (the last one is the next ``tok``)."""
        ctx = getattr(self.drafter, "draft_ctx", None)            # model-based drafters (MTP head) need the context
        drafts = ctx(table, tok, pos, self.k) if ctx is not None else self.drafter.draft(self.k)
        room = getattr(self.model, "max_seq", 1 << 30) - pos - 1
        drafts = drafts[:max(0, min(len(drafts), room - 1))]
        self.n_steps += 1
        if not drafts:
            self.n_plain += 1
            self.model.set_rows(1, [tok], [pos], [self.slot], [table])
            nxt, _ = self.model.decode(1, graph=False)
            new = [int(nxt[0])]
            self.drafter.observe(new)
            if hasattr(self.drafter, "after_decode"):
                self.drafter.after_decode()
            return new
        W = self._width(len(drafts))
        drafts = drafts[:W - 1]
        fed = [tok] + drafts
        pad = W - len(fed)
        logits = self.model.verify(fed + [fed[-1]] * pad, pos, self.slot, self._table(table))
        preds = [int(t) for t in logits[:len(fed)].argmax(-1).tolist()]
        a = 0
        while a < len(drafts) and drafts[a] == preds[a]:
            a += 1
        self.n_drafted += len(drafts)
        self.n_accepted += a
        self.model.commit(self.slot, a + 1)          # the fed token plus the accepted drafts
        new = preds[:a + 1]
        self.drafter.observe(new)
        if hasattr(self.drafter, "after_verify"):
            self.drafter.after_verify(table, fed, a, pos)
        return new

    def generate(self, prompt: list[int], table: list[int], logits: torch.Tensor, n: int) -> list[int]:
        """Greedy generation of ``n`` tokens after a prefill that produced ``logits``."""
        tok = int(logits.argmax())
        self.drafter.reset()
        self.drafter.observe(list(prompt) + [tok])
        out, pos = [tok], len(prompt)
        while len(out) < n:
            new = self.step(table, tok, pos)
            pos += len(new)
            out.extend(new)
            tok = new[-1]
        return out[:n]

    def stats(self) -> dict:
        return {"steps": self.n_steps, "plain_steps": self.n_plain, "drafted": self.n_drafted,
                "accepted": self.n_accepted,
                "accept_rate": round(self.n_accepted / self.n_drafted, 4) if self.n_drafted else 0.0}
