"""MTP draft head: a one-layer gated-attention model that predicts the token after next.

Input of a draft step is the token just sampled and the main model's last-layer residual stream
(before the final norm) of the position that produced it:
``x = fc([norm_e(embed(tok)), norm_h(h_prev)])`` -> one attention layer with its own KV pool ->
SwiGLU -> final norm (which is also the ``h_prev`` of the next chained draft) -> shared lm_head.
The head is run as a second, one-layer instance of the device model whose input is injected
instead of gathered, so it reuses every decode kernel and the block tables of the main sequence
(same block ids, separate pool).  Reference: ``models/qwen35/mtp.py:56-111`` (weights),
``:160-186`` (chained drafts), ``:214-273`` (prefill of its KV).
"""
from __future__ import annotations

import dataclasses

import torch

from ...config import FULL, ModelConfig
from ...ops import kernels as K
from ...weights.init import LM


def has_mtp(sd: dict) -> bool:
    return "mtp.fc.weight" in sd


def _inner_state_dict(sd: dict) -> dict:
    out = {LM + "embed_tokens.weight": sd[LM + "embed_tokens.weight"], LM + "norm.weight": sd["mtp.norm.weight"]}
    if "lm_head.weight" in sd:
        out["lm_head.weight"] = sd["lm_head.weight"]
    for k, v in sd.items():
        if k.startswith("mtp.layers.0."):
            out[LM + "layers.0." + k[len("mtp.layers.0."):]] = v
    return out


class MTPHead:
    def __init__(self, main, sd: dict) -> None:
        from .model import Qwen35Model
        c: ModelConfig = main.cfg
        cfg1 = dataclasses.replace(c, num_hidden_layers=1, layer_types=(FULL,), num_experts=0,
                                   intermediate_size=sd["mtp.layers.0.mlp.gate_proj.weight"].shape[0], name=c.name + "-mtp")
        self.main = main
        self.inner = Qwen35Model(cfg1, _inner_state_dict(sd), device=main.device, max_seq=main.max_seq,
                                 num_slots=1, num_blocks=main.num_blocks, max_chunk=main.max_chunk)
        self.inner.embed = main.embed           # share, do not duplicate
        if "lm_head.weight" not in sd:
            self.inner.lm_head = main.lm_head
        dev, bf = main.device, torch.bfloat16
        self.fc = sd["mtp.fc.weight"].to(dev, bf).contiguous()                       # [H, 2H]
        self.g_e = (1.0 + sd["mtp.pre_fc_norm_embedding.weight"].float()).to(dev).contiguous()
        self.g_h = (1.0 + sd["mtp.pre_fc_norm_hidden.weight"].float()).to(dev).contiguous()
        H = c.hidden_size
        self._cat = torch.zeros(8, 2 * H, dtype=bf, device=dev)
        self._x = torch.zeros(8, H, dtype=bf, device=dev)
        self.n_drafted = 0

    def _inject(self, tokens: torch.Tensor, h_prev: torch.Tensor) -> torch.Tensor:
        """``fc([norm(embed(tok)), norm(h_prev)])`` for ``T`` rows (T <= 8 per call)."""
        T, H = tokens.numel(), self.main.cfg.hidden_size
        e = K.embed_gather(self.main.embed, tokens)
        cat = self._cat[:T]
        K.rmsnorm(e, self.g_e, self.main.eps, out=cat[:, :H])
        K.rmsnorm(h_prev.reshape(T, H).to(torch.bfloat16), self.g_h, self.main.eps, out=cat[:, H:])
        x = self._x[:T]
        K.gemv(self.fc, cat.contiguous(), x)
        return x

    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor, h_prev: torch.Tensor, pos0: int, block_table: torch.Tensor) -> None:
        """Fill the head's KV for prompt positions: row ``t`` pairs token ``t + 1`` of the prompt
        with the main hidden of position ``t`` (``tokens`` are already shifted by the caller)."""
        T = tokens.numel()
        xs = []
        for s in range(0, T, 8):
            xs.append(self._inject(tokens[s:s + 8], h_prev[s:s + 8]).clone())
        self.inner.prefill(tokens, pos0, 0, block_table, embeds=torch.cat(xs), want_logits=False)

    @torch.no_grad()
    def draft(self, tok: int, h_prev: torch.Tensor, pos: int, block_table: list[int], k: int) -> list[int]:
        """``k`` chained greedy drafts after ``tok`` (sampled at position ``pos``, not yet run by the
        main model). KV rows the head writes at ``pos ..`` are overwritten by later calls."""
        out = []
        m = self.inner
        t = torch.tensor([tok], dtype=torch.int64, device=m.device)
        h = h_prev.reshape(1, -1)
        for i in range(k):
            x = self._inject(t, h)
            m.set_rows(1, [0], [pos + i], [0], [block_table])
            m.input_hidden = x
            nxt, _ = m.decode(1, graph=False)
            m.input_hidden = None
            h = m.final_hidden(1)
            t = nxt.clone()
            out.append(int(nxt[0]))
        self.n_drafted += k
        return out


class MTPDrafter:
    """Adapter that lets ``engine.speculative.SpeculativeDecoder`` draft with the MTP head.

    The head keeps its own KV: head position ``p`` pairs token ``p + 1`` with the main model's hidden
    of position ``p``.  ``prime`` fills it from a prefilled prompt, ``draft_ctx`` chains ``k`` greedy
    drafts from the last sampled token, ``after_verify`` rewrites the head rows of the accepted
    tokens with the main model's hiddens (while drafting they were written with the head's own) and
    ``after_decode`` picks up the hidden of a plain step.  Reference: ``models/qwen35/model.py:
    1832-1950`` (``spec_step``), ``models/qwen35/mtp.py`` (head and its cache)."""

    def __init__(self, head: MTPHead) -> None:
        self.head = head
        self.h: torch.Tensor | None = None

    # the suffix-drafter protocol (history is not needed here)
    def reset(self) -> None:
        self.h = None

    def observe(self, tokens) -> None:
        pass

    def draft(self, k: int) -> list[int]:
        return []

    def prime(self, prompt: torch.Tensor, pos0: int, table: torch.Tensor) -> None:
        """After the main model prefilled ``prompt`` (the chunk starting at ``pos0`` whose residual
        stream is still in ``main.last_prenorm``)."""
        main = self.head.main
        T = prompt.numel()
        pre = main.last_prenorm[:T]
        if T > 1:
            self.head.prefill(prompt[1:], pre[:-1], pos0, table)
        self.h = pre[T - 1].clone()

    def draft_ctx(self, table: list[int], tok: int, pos: int, k: int) -> list[int]:
        if self.h is None or pos < 1:
            return []
        return self.head.draft(tok, self.h, pos - 1, table, k)

    def after_verify(self, table: list[int], fed: list[int], accepted: int, pos: int) -> None:
        main = self.head.main
        hid = main.verify_hidden()
        if accepted > 0:
            bt = torch.tensor(table, dtype=torch.int32, device=main.device)
            toks = torch.tensor(fed[1:accepted + 1], dtype=torch.int64, device=main.device)
            self.head.prefill(toks, hid[:accepted], pos, bt)
        self.h = hid[accepted].clone()

    def after_decode(self) -> None:
        self.h = self.head.main.final_hidden(1, normed=False)[0].clone()
