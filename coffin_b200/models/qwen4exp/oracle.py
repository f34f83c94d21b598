"""fp32 CPU oracle of the Qwen4-exp text model: the numerical reference every sm_100a kernel of the
family is tested against.

It states the math directly, one token row at a time where that is clearest:

* hyper-connection (``models/qwen4exp/gated_residual.py:48-478`` in the reference): grouped
  zero-centred RMSNorm of the ``hc`` residual lanes, a low-rank read gate
  ``sigmoid(up(silu(down(n) / hc)))`` whose gated lanes are *averaged* into the mixer input, and a
  scalar write gate ``2 * sigmoid(inject(n) / hc)`` per lane for the mixer output;
* QSA (``models/qwen4exp/qsa.py:416-1305``): the indexer scores blocks of ``ratio`` consecutive
  visible tokens (mean of the raw index keys, normed, rotated at the block's first position) with
  ``sum_heads relu(q . k) / sqrt(d)``, keeps the ``budget / ratio`` best blocks plus the ragged
  tail, and gated GQA attention runs over the kept tokens only.  A query that sees at most
  ``full_select_factor * topk`` blocks attends to everything (the reference's full-select path,
  applied here per query);
* PLE (``models/qwen4exp/ngram.py:530-949``): hashed 2..n-gram ids -> embedding rows -> a
  per-lane gated value plus a dilated causal depthwise conv, added to all lanes before the layer;
* the delta-net and MoE layers are the Qwen3.5 ones (``oracle/ops.py``) with a selectable output
  gate.
"""
from __future__ import annotations

import dataclasses
import math

import torch
import torch.nn.functional as F

from ...oracle import ops as O
from .config import LINEAR, Qwen4Config
from .ngram import NGramHasher

LM = "model.language_model."


def grouped_rms_norm(x: torch.Tensor, w: torch.Tensor, group: int, eps: float) -> torch.Tensor:
    """Zero-centred RMSNorm over groups of ``group`` channels: ``x [..., G*group]``, ``w`` same width."""
    xf = x.float().reshape(*x.shape[:-1], -1, group)
    n = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return n.flatten(-2) * (1.0 + w.float())


def hyper_read(x: torch.Tensor, p: dict, prefix: str, cfg: Qwen4Config):
    """``x [T, hc*H]`` -> ``(mixed [T, H], inject [T, hc] | None)``."""
    hc, H = cfg.hc_count, cfg.hidden_size
    n = grouped_rms_norm(x, p[prefix + "hc_norm.weight"], H, cfg.rms_norm_eps)
    low = F.silu(n @ p[prefix + "input_mix_weight_down.weight"].float().t() / hc)
    gate = torch.sigmoid(low @ p[prefix + "input_mix_weight_up.weight"].float().t())
    mixed = (gate * n).reshape(-1, hc, H).mean(1)
    key = prefix + "block_inject_weight.weight"
    inject = 2.0 * torch.sigmoid(n @ p[key].float().t() / hc) if key in p else None
    return mixed, inject


def hyper_write(x: torch.Tensor, out: torch.Tensor, inject: torch.Tensor, cfg: Qwen4Config) -> torch.Tensor:
    """``x + out (x) inject``: the mixer output written into every lane with that lane's gate."""
    return x + (out.float()[:, None, :] * inject[:, :, None]).flatten(1)


def dilated_conv_silu(w: torch.Tensor, x: torch.Tensor, hist: torch.Tensor, dilation: int):
    """Causal depthwise conv: taps ``w [C, k]`` (oldest first) ``dilation`` rows apart over
    ``hist [span, C] ++ x [T, C]``, then SiLU.  Returns the outputs and the new history."""
    k = w.shape[1]
    span = dilation * (k - 1)
    seq = torch.cat([hist.float(), x.float()], 0)
    T = x.shape[0]
    out = torch.zeros(T, x.shape[1])
    for j in range(k):
        out += seq[j * dilation:j * dilation + T] * w[:, j].float()
    return F.silu(out), seq[seq.shape[0] - span:].clone()


def qsa_block_keys(raw: torch.Tensor, k_norm_w: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, ratio: int,
                   rot: int, eps: float) -> torch.Tensor:
    """Block keys of the complete blocks of ``raw [S, d]``: mean -> zero-centred norm -> rotary at
    the block's first position.  ``cos/sin [S, rot]``."""
    nb = raw.shape[0] // ratio
    pooled = raw[:nb * ratio].float().reshape(nb, ratio, -1).mean(1)
    pooled = O.rms_norm(pooled, 1.0 + k_norm_w.float(), eps)
    starts = torch.arange(nb) * ratio
    return O.apply_rope(pooled[:, None, :], cos[starts], sin[starts], rot)[:, 0]


def qsa_select(iq: torch.Tensor, bkeys: torch.Tensor, n_visible: int, cfg: Qwen4Config) -> torch.Tensor:
    """Bool keep-mask ``[n_visible]`` for one query: ``iq [n_heads, d]`` normed + rotated index
    queries, ``bkeys [>= n_visible // ratio, d]``."""
    ratio, topk = cfg.indexer_compress_ratio, cfg.block_topk
    nb = n_visible // ratio
    keep = torch.zeros(n_visible, dtype=torch.bool)
    keep[nb * ratio:] = True
    if nb <= topk * cfg.full_select_factor or nb <= topk:
        keep[:] = True
        return keep
    s = torch.relu(iq.float() @ bkeys[:nb].float().t()).sum(0) / math.sqrt(iq.shape[-1])
    # ties (relu leaves many exact zeros) go to the lowest block index: a rule the kernels can match
    for b in torch.sort(s, descending=True, stable=True).indices[:topk].tolist():
        keep[b * ratio:(b + 1) * ratio] = True
    return keep


@dataclasses.dataclass
class DraftIndexPlan:
    """Block selection shared along one draft chain: the head selects on draft step 0 and later steps
    attend to the same blocks (``models/qwen4exp/mtp.py:63-128`` of the reference; only block numbers are
    reused, the ragged tail after the last complete block is always visible).  The reuse holds only
    while no further block has completed since step 0 - a step that crosses a block boundary selects
    again and records anew, so the visible set never silently loses a block.  ``used`` counts the steps
    that attended through the recorded selection."""
    enabled: bool = True
    blocks: torch.Tensor | None = None          # bool [n_complete_blocks] kept at the recording step
    n_blocks: int = -1
    used: int = 0

    def before_step(self, step: int):
        if step < 0:
            raise ValueError(f"draft step index must be >= 0, got {step}")
        if not self.enabled or step == 0 or self.blocks is None:
            return None
        return self.blocks

    def record(self, keep_row: torch.Tensor, position: int, cfg) -> None:
        ratio = cfg.indexer_compress_ratio
        nb = (position + 1) // ratio
        self.n_blocks = nb
        self.blocks = keep_row[:nb * ratio].reshape(nb, ratio).all(1) if nb else torch.zeros(0, dtype=torch.bool)

    def keep_rows(self, blocks: torch.Tensor, pos: torch.Tensor, S: int, cfg):
        """Keep-mask ``[T, S]`` from the recorded blocks, or ``None`` when a row's block count differs
        from the recorded one (select again)."""
        ratio = cfg.indexer_compress_ratio
        keep = torch.zeros(pos.numel(), S, dtype=torch.bool)
        for t, p_ in enumerate(pos.tolist()):
            nb = (p_ + 1) // ratio
            if nb != self.n_blocks:
                return None
            keep[t, :nb * ratio] = blocks.repeat_interleave(ratio)
            keep[t, nb * ratio:p_ + 1] = True
        self.used += 1
        return keep


@dataclasses.dataclass
class Qwen4State:
    n: int = 0
    conv: dict = dataclasses.field(default_factory=dict)        # layer -> [C, k-1]
    rec: dict = dataclasses.field(default_factory=dict)         # layer -> [nv, dk, dv]
    k: dict = dataclasses.field(default_factory=dict)           # layer -> [S, nkv, hd]
    v: dict = dataclasses.field(default_factory=dict)
    ik: dict = dataclasses.field(default_factory=dict)          # layer -> raw index keys [S, d]
    ple_ctx: dict = dataclasses.field(default_factory=dict)     # layer -> list[int]
    ple_hist: dict = dataclasses.field(default_factory=dict)    # layer -> [span, hc*H]
    pos3: torch.Tensor | None = None                            # [3, n] rotary positions (t, h, w) of every token so far

    def clone(self) -> "Qwen4State":
        c = Qwen4State(self.n)
        for name in ("conv", "rec", "k", "v", "ik", "ple_hist"):
            setattr(c, name, {i: t.clone() for i, t in getattr(self, name).items()})
        c.ple_ctx = {i: list(t) for i, t in self.ple_ctx.items()}
        c.pos3 = None if self.pos3 is None else self.pos3.clone()
        return c


class Qwen4Oracle:
    def __init__(self, cfg: Qwen4Config, sd: dict[str, torch.Tensor]) -> None:
        self.cfg = cfg
        self.p = {k: (v.float() if isinstance(v, torch.Tensor) and v.is_floating_point() else v) for k, v in sd.items()}
        self.hashers = {li: NGramHasher(cfg, cfg.ple_index(li)) for li in range(cfg.num_hidden_layers)
                        if cfg.ple_index(li) is not None}
        self.last_selected: dict[int, torch.Tensor] = {}

    def new_state(self) -> Qwen4State:
        return Qwen4State()

    # ------------------------------------------------------------------ pieces
    def _cos_sin(self, pos: torch.Tensor):
        """``pos [L]`` (the same index on every axis) or ``[3, L]`` (t, h, w of image tokens)."""
        c = self.cfg
        if pos.dim() == 2 and not c.mrope_section:
            pos = pos[0]
        if c.mrope_section:
            p3 = pos if pos.dim() == 2 else pos.reshape(1, -1).expand(3, -1)
            return O.mrope_cos_sin(p3, c.rotary_dim, c.rope_theta, c.mrope_section)
        inv = O.inv_freq(c.rotary_dim, c.rope_theta)
        f = pos.float()[:, None] * inv[None, :]
        return torch.cat([f.cos(), f.cos()], -1), torch.cat([f.sin(), f.sin()], -1)

    def _ple(self, li: int, x: torch.Tensor, tokens: torch.Tensor, st: Qwen4State) -> torch.Tensor:
        c, p = self.cfg, self.p
        q = f"{LM}layers.{li}.ple."
        hc, H = c.hc_count, c.hidden_size
        ctx = st.ple_ctx.get(li) or [c.eos_token_id] * c.ple_context_len
        ids = self.hashers[li].ids(tokens.tolist(), ctx)                         # [T, heads]
        tw = p[q + "ple_embedding.ngram_embedding.weight"]
        if isinstance(tw, list):                 # row shards of a real checkpoint (mapped host views)
            from .ngram import ShardedNGramTable
            emb = ShardedNGramTable(list(tw), "cpu").gather(ids).float()
        else:
            emb = tw[ids].flatten(1)             # [T, E]
        key = grouped_rms_norm(emb @ p[q + "key_proj.weight"].t(), p[q + "norm_key.weight"], H, c.rms_norm_eps)
        val = emb @ p[q + "value_proj.weight"].t()                               # [T, H]
        qry = grouped_rms_norm(x, p[q + "norm_query.weight"], H, c.rms_norm_eps)
        g = (key.reshape(-1, hc, H) * qry.reshape(-1, hc, H)).sum(-1, keepdim=True) / math.sqrt(H)
        g = g.abs().clamp_min(1e-6).sqrt() * g.sign()
        gv = (torch.sigmoid(g) * val[:, None, :]).flatten(1)                     # [T, hc*H]
        gvn = grouped_rms_norm(gv, p[q + "norm_conv.weight"], H, c.rms_norm_eps)
        hist = st.ple_hist.get(li)
        if hist is None:
            hist = torch.zeros(c.ple_conv_state_len, hc * H)
        conv, st.ple_hist[li] = dilated_conv_silu(p[q + "conv1d.weight"].reshape(hc * H, -1), gvn, hist, c.ple_conv_dilation)
        st.ple_ctx[li] = (ctx + tokens.tolist())[-c.ple_context_len:]
        return gv + conv

    def _gdn(self, li: int, h: torch.Tensor, st: Qwen4State) -> torch.Tensor:
        c, p = self.cfg, self.p
        q = f"{LM}layers.{li}.linear_attn."
        T = h.shape[0]
        qkv = h @ p[q + "in_proj_qkv.weight"].t()
        z = h @ p[q + "in_proj_z.weight"].t()
        b = h @ p[q + "in_proj_b.weight"].t()
        a = h @ p[q + "in_proj_a.weight"].t()
        conv_state = st.conv.get(li)
        if conv_state is None:
            conv_state = torch.zeros(c.lin_conv_dim, c.linear_conv_kernel_dim - 1)
        conv, st.conv[li] = O.conv1d_silu_seq(p[q + "conv1d.weight"].reshape(c.lin_conv_dim, -1), qkv, conv_state)
        nk, nv, dk, dv = c.linear_num_key_heads, c.linear_num_value_heads, c.linear_key_head_dim, c.linear_value_head_dim
        qq = conv[:, :c.lin_kdim].reshape(T, nk, dk)
        kk = conv[:, c.lin_kdim:2 * c.lin_kdim].reshape(T, nk, dk)
        vv = conv[:, 2 * c.lin_kdim:].reshape(T, nv, dv)
        qn, kn, beta, g = O.gdn_head_prep(qq, kk, b, a, p[q + "A_log"], p[q + "dt_bias"], c.lin_rep)
        state = st.rec.get(li)
        if state is None:
            state = st.rec[li] = torch.zeros(nv, dk, dv)
        o = (O.delta_chunked if T > 1 else O.delta_recurrent)(qn, kn, vv, beta, g, state)
        zz = z.reshape(T, nv, dv)
        gate = F.silu(zz) if c.output_gate_type == "silu" else torch.sigmoid(zz)
        o = O.rms_norm(o, p[q + "norm.weight"], c.rms_norm_eps) * gate
        return o.reshape(T, nv * dv) @ p[q + "out_proj.weight"].t()

    def _qsa(self, li, h: torch.Tensor, st: Qwen4State, pos: torch.Tensor, cos, sin, prefix: str | None = None,
             reuse: torch.Tensor | None = None) -> torch.Tensor:
        """``li`` keys the K / V / index-key history in ``st`` (the draft head uses the key ``"mtp"``);
        ``reuse`` (bool ``[T, S]``) replaces the block selection by a given keep-mask."""
        c, p = self.cfg, self.p
        q = (prefix if prefix is not None else f"{LM}layers.{li}.") + "self_attn."
        T = h.shape[0]
        nh, nkv, hd, rot = c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.rotary_dim
        ni, di = c.indexer_n_heads, c.indexer_head_dim
        qg = (h @ p[q + "q_proj.weight"].t()).reshape(T, nh, 2 * hd)
        qq, gate = qg[..., :hd], qg[..., hd:]
        kk = (h @ p[q + "k_proj.weight"].t()).reshape(T, nkv, hd)
        vv = (h @ p[q + "v_proj.weight"].t()).reshape(T, nkv, hd)
        qq = O.apply_rope(O.rms_norm(qq, 1.0 + p[q + "q_norm.weight"], c.rms_norm_eps), cos, sin, rot)
        kk = O.apply_rope(O.rms_norm(kk, 1.0 + p[q + "k_norm.weight"], c.rms_norm_eps), cos, sin, rot)
        iqk = h @ p[q + "indexer.index_qk_proj.weight"].t()
        iq = O.rms_norm(iqk[:, :ni * di].reshape(T, ni, di), 1.0 + p[q + "indexer.q_layernorm.weight"], c.rms_norm_eps)
        iq = O.apply_rope(iq, cos, sin, rot)
        raw = iqk[:, ni * di:]
        st.k[li] = torch.cat([st.k[li], kk]) if li in st.k else kk
        st.v[li] = torch.cat([st.v[li], vv]) if li in st.v else vv
        st.ik[li] = torch.cat([st.ik[li], raw]) if li in st.ik else raw
        S = st.k[li].shape[0]
        allcos, allsin = self._cos_sin(st.pos3[:, :S] if (st.pos3 is not None and li != "mtp") else torch.arange(S))
        bkeys = qsa_block_keys(st.ik[li], p[q + "indexer.k_layernorm.weight"], allcos, allsin, c.indexer_compress_ratio,
                               rot, c.rms_norm_eps)
        keep = torch.zeros(T, S, dtype=torch.bool)
        for t in range(T):
            nvis = int(pos[t]) + 1
            keep[t, :nvis] = qsa_select(iq[t], bkeys, nvis, c) if reuse is None else reuse[t, :nvis]
        self.last_selected[li] = keep
        o = O.gated_attention(qq, gate, st.k[li], st.v[li], pos, hd ** -0.5, keep=keep)
        return o.reshape(T, nh * hd) @ p[q + "o_proj.weight"].t()

    def _moe(self, li, h: torch.Tensor, prefix: str | None = None) -> torch.Tensor:
        c, p = self.cfg, self.p
        m = (prefix if prefix is not None else f"{LM}layers.{li}.") + "mlp."
        shared = (p[m + "shared_expert.gate_proj.weight"], p[m + "shared_expert.up_proj.weight"],
                  p[m + "shared_expert.down_proj.weight"], p[m + "shared_expert_gate.weight"])
        return O.moe_ffn(h, p[m + "gate.weight"], p[m + "experts.gate_up_proj"], p[m + "experts.down_proj"],
                         c.num_experts_per_tok, c.norm_topk_prob, shared)

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def lanes(self, tokens: torch.Tensor, st: Qwen4State, embeds: torch.Tensor | None = None,
              pos3: torch.Tensor | None = None) -> torch.Tensor:
        """The ``hc`` residual lanes ``[T, hc*H]`` after the last layer; ``st`` advances by ``T``.
        ``embeds`` replaces the token embeddings (image tokens carry the vision tower's output),
        ``pos3 [3, T]`` the rotary positions (default: the token index on every axis).  Causality and
        the block structure of the sparse attention always follow the token index."""
        c, p = self.cfg, self.p
        T = tokens.numel()
        pos = torch.arange(st.n, st.n + T)
        if pos3 is None:
            pos3 = pos.reshape(1, -1).expand(3, -1)
        st.pos3 = pos3.clone() if st.pos3 is None else torch.cat([st.pos3, pos3], 1)
        cos, sin = self._cos_sin(pos3)
        e = p[LM + "embed_tokens.weight"][tokens.long()] if embeds is None else embeds.float()
        x = e.repeat(1, c.hc_count)
        for li, kind in enumerate(c.layer_types):
            lp = f"{LM}layers.{li}."
            if li in self.hashers:
                x = x + self._ple(li, x, tokens, st)
            mixed, inject = hyper_read(x, p, lp + "attn_hyper_connection.", c)
            out = self._gdn(li, mixed, st) if kind == LINEAR else self._qsa(li, mixed, st, pos, cos, sin)
            x = hyper_write(x, out, inject, c)
            mixed, inject = hyper_read(x, p, lp + "mlp_hyper_connection.", c)
            x = hyper_write(x, self._moe(li, mixed), inject, c)
        st.n += T
        return x

    # ------------------------------------------------------------------ draft head (MTP)
    @property
    def has_mtp(self) -> bool:
        return "mtp.fc_embedding.weight" in self.p

    @torch.no_grad()
    def mtp_run(self, next_tokens: torch.Tensor, lanes: torch.Tensor, mst: Qwen4State, add_embedding: bool = True,
                plan: "DraftIndexPlan | None" = None, step: int = 0):
        """One pass of the draft head over ``T`` rows at positions ``mst.n ..``: row ``t`` sees the main
        model's un-collapsed lanes at its position (``lanes [T, hc*H]``; on later draft steps the head's
        own ``multi`` output) and the token that FOLLOWS that position (``next_tokens [T]``), and
        predicts the token after it.  Returns ``(sample [T, H], multi [T, hc*H])``; ``mst`` holds the
        head's own K / V / index keys (nothing is shared with a main layer) and advances by ``T``.

        Structure (``models/qwen4exp/mtp.py:146-330`` of the reference): the embedding goes through a
        zero-centred RMSNorm of width ``H`` and ``fc_embedding``; the lanes through ONE RMSNorm over the
        whole ``hc*H`` width and ``fc_hidden`` applied to every lane; the projected embedding is added to
        every lane with unit weight only when ``add_embedding`` (prefill / append rows and draft step 0
        - adding it on the chained steps would stack it into the stream again); then one QSA + MoE
        layer without n-gram injection and the head's own final mixer, which has no write gate."""
        c, p = self.cfg, self.p
        hc, H = c.hc_count, c.hidden_size
        T = next_tokens.numel()
        pos = torch.arange(mst.n, mst.n + T)
        cos, sin = self._cos_sin(pos)
        e = p[LM + "embed_tokens.weight"][next_tokens.long()]
        e = O.rms_norm(e, 1.0 + p["mtp.pre_fc_norm_embedding.weight"], c.rms_norm_eps) @ p["mtp.fc_embedding.weight"].t()
        n = O.rms_norm(lanes.float(), 1.0 + p["mtp.pre_fc_norm_hidden.weight"], c.rms_norm_eps)
        x = (n.reshape(T, hc, H) @ p["mtp.fc_hidden.weight"].t()).flatten(1)
        if add_embedding:
            x = x + e.repeat(1, hc)
        lp = "mtp.layers.0."
        mixed, inject = hyper_read(x, p, lp + "attn_hyper_connection.", c)
        reuse = plan.before_step(step) if plan is not None else None
        keep = None
        if reuse is not None:
            keep = plan.keep_rows(reuse, pos, mst.k["mtp"].shape[0] + T if "mtp" in mst.k else T, c)
        out = self._qsa("mtp", mixed, mst, pos, cos, sin, prefix=lp, reuse=keep)
        if plan is not None and keep is None:
            plan.record(self.last_selected["mtp"][-1], int(pos[-1]), c)
        x = hyper_write(x, out, inject, c)
        mixed, inject = hyper_read(x, p, lp + "mlp_hyper_connection.", c)
        x = hyper_write(x, self._moe("mtp", mixed, prefix=lp), inject, c)
        mst.n += T
        return hyper_read(x, p, "mtp.hyper_connection_mixer.", c)[0], x

    def head(self, hidden: torch.Tensor) -> torch.Tensor:
        return hidden @ self.p.get("lm_head.weight", self.p[LM + "embed_tokens.weight"]).t()

    @torch.no_grad()
    def spec_generate(self, prompt: list[int], max_new: int, k: int = 3, index_reuse: bool = True, draft_hook=None):
        """Greedy speculative decoding with the draft head, stated as plainly as possible: the head's
        K/V follow the main model's position by position (row ``i`` pairs the lanes at position ``i``
        with token ``i + 1``), ``k`` drafts are chained from the last committed position, the main
        model scores ``[last, d1..dk]`` in one pass and the longest agreeing prefix is kept.  The
        result equals plain greedy decoding token for token.  ``draft_hook(position, drafts)`` may
        replace the drafts of a round (``position``: where the first draft would land).
        Returns ``(tokens, stats)``."""
        st, mst = self.new_state(), self.new_state()
        toks = torch.tensor(prompt)
        lanes = self.lanes(toks, st)
        logits = self.head(hyper_read(lanes, self.p, LM + "hyper_connection_mixer.", self.cfg)[0])
        out = [int(logits[-1].argmax())]
        stats = {"rounds": 0, "drafted": 0, "accepted": 0, "index_reuse": 0}
        # rows 0..n-2 of the prompt build the head's history; the row of the last prompt position is
        # appended together with the first draft below (its "next token" is out[-1])
        if len(prompt) > 1:
            self.mtp_run(toks[1:], lanes[:-1], mst)
        pend_lanes, pend_next = lanes[-1:], [out[-1]]          # rows not yet appended to the head
        while len(out) < max_new:
            stats["rounds"] += 1
            plan = DraftIndexPlan(enabled=index_reuse)
            sample, multi = self.mtp_run(torch.tensor(pend_next), pend_lanes, mst, plan=plan, step=0)
            base = mst.clone()                                  # the head's state at the committed length
            drafts = [int(self.head(sample[-1:])[0].argmax())]
            multi = multi[-1:]
            for step in range(1, k):
                sample, multi = self.mtp_run(torch.tensor(drafts[-1:]), multi, mst, add_embedding=False, plan=plan, step=step)
                drafts.append(int(self.head(sample)[0].argmax()))
            mst = base                                          # the chain's K/V rows are dropped
            if draft_hook is not None:                          # a caller may replace the drafts (tests of the accept paths)
                drafts = list(draft_hook(len(prompt) + len(out), drafts))[:k]
            stats["drafted"] += k
            stats["index_reuse"] += plan.used
            snap = st.clone()
            seq = torch.tensor([out[-1]] + drafts)
            v_lanes = self.lanes(seq, st)
            picked = self.head(hyper_read(v_lanes, self.p, LM + "hyper_connection_mixer.", self.cfg)[0]).argmax(-1).tolist()
            a = 0
            while a < len(drafts) and picked[a] == drafts[a]:
                a += 1
            stats["accepted"] += a
            if a < len(drafts):                                            # roll the main model back to the accepted prefix
                st = snap
                v_lanes = self.lanes(seq[:a + 1], st)
            new = drafts[:a] + [picked[a]]
            out.extend(new)
            pend_lanes, pend_next = v_lanes[:a + 1], new
        stats["acceptance"] = stats["accepted"] / max(stats["drafted"], 1)
        return out[:max_new], stats

    def hidden(self, tokens: torch.Tensor, st: Qwen4State, **kw) -> torch.Tensor:
        x = self.lanes(tokens, st, **kw)
        return hyper_read(x, self.p, LM + "hyper_connection_mixer.", self.cfg)[0]

    def forward(self, tokens: torch.Tensor, st: Qwen4State, **kw) -> torch.Tensor:
        """Logits ``[T, vocab]``."""
        w = self.p.get("lm_head.weight", self.p[LM + "embed_tokens.weight"])
        return self.hidden(tokens, st, **kw) @ w.t()
