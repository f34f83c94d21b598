"""CPU fp32 model of the Qwen3.5-style hybrid: the logits oracle.

One class, no kernels, no caches beyond plain tensors.  It runs a whole sequence or one
token at a time through the same code, so prefill-vs-decode agreement of the sm_100a
engine can be checked against a single definition.  The layer structure follows the
reference model (``models/qwen35/blocks.py:112-225``: pre-norm mixer, residual,
pre-norm FFN, residual; ``models/qwen35/linear_attn.py:358-396``;
``models/qwen35/full_attn.py:303-369``; ``models/qwen35/moe.py:508-559``;
``models/qwen35/mtp.py:56-186``), computed in fp32 throughout.
"""
from __future__ import annotations

import dataclasses

import torch

from ..config import LINEAR, ModelConfig
from ..weights.init import LM
from . import ops as O


@dataclasses.dataclass
class OracleState:
    """Per-sequence state: conv windows + recurrent states of the linear layers, K/V of
    the attention layers (position order), number of tokens seen."""
    conv: dict[int, torch.Tensor]
    rec: dict[int, torch.Tensor]
    k: dict[int, torch.Tensor]
    v: dict[int, torch.Tensor]
    length: int = 0

    def clone(self) -> "OracleState":
        return OracleState({i: t.clone() for i, t in self.conv.items()},
                           {i: t.clone() for i, t in self.rec.items()},
                           {i: t.clone() for i, t in self.k.items()},
                           {i: t.clone() for i, t in self.v.items()}, self.length)


class OracleModel:
    """fp32 reference forward.  ``sd`` uses the HF key layout (``weights/init.py``)."""

    def __init__(self, cfg: ModelConfig, sd: dict[str, torch.Tensor], kv_int8: bool = False,
                 chunked_gdn: bool = False) -> None:
        self.cfg = cfg
        self.sd = {k: v.float() if v.is_floating_point() else v for k, v in sd.items()}
        self.kv_int8 = kv_int8
        self.chunked_gdn = chunked_gdn
        self.has_mtp = "mtp.fc.weight" in self.sd

    # ---- state ------------------------------------------------------------
    def new_state(self) -> OracleState:
        c = self.cfg
        conv, rec, k, v = {}, {}, {}, {}
        for i, t in enumerate(c.layer_types):
            if t == LINEAR:
                conv[i] = torch.zeros(c.lin_conv_dim, c.linear_conv_kernel_dim - 1)
                rec[i] = torch.zeros(c.linear_num_value_heads, c.linear_key_head_dim,
                                     c.linear_value_head_dim)
            else:
                k[i] = torch.zeros(0, c.num_key_value_heads, c.head_dim)
                v[i] = torch.zeros(0, c.num_key_value_heads, c.head_dim)
        if self.has_mtp:
            k[-1] = torch.zeros(0, c.num_key_value_heads, c.head_dim)
            v[-1] = torch.zeros(0, c.num_key_value_heads, c.head_dim)
        return OracleState(conv, rec, k, v, 0)

    # ---- pieces -----------------------------------------------------------
    def _norm(self, x, key):
        return O.rms_norm(x, 1.0 + self.sd[key], self.cfg.rms_norm_eps)

    def _linear_attn(self, i: int, x: torch.Tensor, st: OracleState, p: str | None = None) -> torch.Tensor:
        c, sd = self.cfg, self.sd
        p = p or f"{LM}layers.{i}.linear_attn."
        T = x.shape[0]
        qkv = x @ sd[p + "in_proj_qkv.weight"].t()
        z = x @ sd[p + "in_proj_z.weight"].t()
        b = x @ sd[p + "in_proj_b.weight"].t()
        a = x @ sd[p + "in_proj_a.weight"].t()
        conv_w = sd[p + "conv1d.weight"].reshape(c.lin_conv_dim, c.linear_conv_kernel_dim)
        conv, st.conv[i] = O.conv1d_silu_seq(conv_w, qkv, st.conv[i])
        nk, nv, dk, dv = (c.linear_num_key_heads, c.linear_num_value_heads,
                          c.linear_key_head_dim, c.linear_value_head_dim)
        q = conv[:, :c.lin_kdim].reshape(T, nk, dk)
        k = conv[:, c.lin_kdim:2 * c.lin_kdim].reshape(T, nk, dk)
        v = conv[:, 2 * c.lin_kdim:].reshape(T, nv, dv)
        qn, kn, beta, g = O.gdn_head_prep(q, k, b, a, sd[p + "A_log"], sd[p + "dt_bias"], c.lin_rep)
        scan = O.delta_chunked if (self.chunked_gdn and T > 1) else O.delta_recurrent
        o = scan(qn, kn, v, beta, g, st.rec[i])                          # [T, nv, dv]
        o = O.rms_norm_gated(o, sd[p + "norm.weight"], z.reshape(T, nv, dv), c.rms_norm_eps)
        return o.reshape(T, nv * dv) @ sd[p + "out_proj.weight"].t()

    def _full_attn(self, i: int, x: torch.Tensor, st: OracleState, cos, sin, pos,
                   p: str | None = None) -> torch.Tensor:
        c, sd = self.cfg, self.sd
        p = p or f"{LM}layers.{i}.self_attn."
        T = x.shape[0]
        nh, nkv, hd = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        qg = (x @ sd[p + "q_proj.weight"].t()).reshape(T, nh, 2 * hd)
        q, gate = qg[..., :hd], qg[..., hd:]
        k = (x @ sd[p + "k_proj.weight"].t()).reshape(T, nkv, hd)
        v = (x @ sd[p + "v_proj.weight"].t()).reshape(T, nkv, hd)
        q = O.rms_norm(q, 1.0 + sd[p + "q_norm.weight"], c.rms_norm_eps)
        k = O.rms_norm(k, 1.0 + sd[p + "k_norm.weight"], c.rms_norm_eps)
        q = O.apply_rope(q, cos, sin, c.rotary_dim)
        k = O.apply_rope(k, cos, sin, c.rotary_dim)
        if self.kv_int8:
            kq, ks = O.quant_rows_int8(k)
            vq, vs = O.quant_rows_int8(v)
            k, v = kq.float() * ks[..., None], vq.float() * vs[..., None]
        st.k[i] = torch.cat([st.k[i], k], 0)
        st.v[i] = torch.cat([st.v[i], v], 0)
        o = O.gated_attention(q, gate, st.k[i], st.v[i], pos, hd ** -0.5)
        return o.reshape(T, nh * hd) @ sd[p + "o_proj.weight"].t()

    def _ffn(self, p: str, x: torch.Tensor) -> torch.Tensor:
        c, sd = self.cfg, self.sd
        if (p + "gate.weight") in sd:
            shared = None
            if (p + "shared_expert.gate_proj.weight") in sd:
                shared = (sd[p + "shared_expert.gate_proj.weight"], sd[p + "shared_expert.up_proj.weight"],
                          sd[p + "shared_expert.down_proj.weight"], sd[p + "shared_expert_gate.weight"])
            return O.moe_ffn(x, sd[p + "gate.weight"], sd[p + "experts.gate_up_proj"],
                             sd[p + "experts.down_proj"], c.num_experts_per_tok, c.norm_topk_prob, shared)
        h = O.silu_mul(x @ sd[p + "gate_proj.weight"].t(), x @ sd[p + "up_proj.weight"].t())
        return h @ sd[p + "down_proj.weight"].t()

    def embed(self, tokens: torch.Tensor) -> torch.Tensor:
        return self.sd[LM + "embed_tokens.weight"][tokens.long()]

    def head(self, h: torch.Tensor) -> torch.Tensor:
        w = self.sd.get("lm_head.weight", self.sd[LM + "embed_tokens.weight"])
        return h @ w.t()

    def _cos_sin(self, pos: torch.Tensor, positions3: torch.Tensor | None):
        c = self.cfg
        if positions3 is None:
            positions3 = pos.reshape(1, -1).expand(3, -1)
        return O.mrope_cos_sin(positions3, c.rotary_dim, c.rope_theta, c.mrope_section)

    # ---- forward ------------------------------------------------------------
    def hidden(self, tokens: torch.Tensor, st: OracleState, embeds: torch.Tensor | None = None,
               positions3: torch.Tensor | None = None, rope_delta: int = 0) -> torch.Tensor:
        """Final-norm hidden states ``[T, H]`` for ``tokens`` appended to ``st``.

        ``embeds`` overrides the token embeddings (image rows already scattered);
        ``positions3 [3, T]`` gives mRoPE positions; otherwise the rotary position is the
        token index plus ``rope_delta``.
        """
        c = self.cfg
        T = tokens.shape[0]
        pos = torch.arange(st.length, st.length + T)
        cos, sin = self._cos_sin(pos + rope_delta, positions3)
        x = self.embed(tokens) if embeds is None else embeds.float()
        for i, t in enumerate(c.layer_types):
            p = f"{LM}layers.{i}."
            h = self._norm(x, p + "input_layernorm.weight")
            if t == LINEAR:
                x = x + self._linear_attn(i, h, st)
            else:
                x = x + self._full_attn(i, h, st, cos, sin, pos)
            x = x + self._ffn(p + "mlp.", self._norm(x, p + "post_attention_layernorm.weight"))
        self._last_prenorm = x
        st.length += T
        return self._norm(x, LM + "norm.weight")

    def forward(self, tokens: torch.Tensor, st: OracleState, **kw) -> torch.Tensor:
        """Logits ``[T, vocab]``."""
        return self.head(self.hidden(tokens, st, **kw))

    @torch.no_grad()
    def generate(self, prompt: list[int], n: int, st: OracleState | None = None
                 ) -> tuple[list[int], torch.Tensor]:
        """Greedy decode ``n`` tokens. Returns the tokens and the logits ``[n, vocab]``
        each token was picked from."""
        st = st or self.new_state()
        logits = self.forward(torch.tensor(prompt), st)[-1]
        toks, rows = [], []
        for _ in range(n):
            rows.append(logits)
            t = int(logits.argmax())
            toks.append(t)
            logits = self.forward(torch.tensor([t]), st)[-1]
        return toks, torch.stack(rows)

    # ---- MTP draft head ---------------------------------------------------
    def mtp_forward(self, tokens: torch.Tensor, hidden_prev: torch.Tensor, st: OracleState,
                    pos: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """Draft head: ``fc([norm(embed(tok)), norm(h_prev)])`` -> one gated-attention layer
        with its own KV (``st.k[-1]``) -> SwiGLU -> norm -> shared lm_head.

        ``tokens[t]`` is the token at position ``pos[t] + 1`` (the one just sampled) and
        ``hidden_prev[t]`` the main model's pre-head hidden at ``pos[t]``.  Returns
        ``(logits, hidden)`` for the token after.
        """
        sd = self.sd
        e = self._norm(self.embed(tokens), "mtp.pre_fc_norm_embedding.weight")
        h = self._norm(hidden_prev.float(), "mtp.pre_fc_norm_hidden.weight")
        x = torch.cat([e, h], -1) @ sd["mtp.fc.weight"].t()
        cos, sin = self._cos_sin(pos, None)
        p = "mtp.layers.0."
        x = x + self._full_attn(-1, self._norm(x, p + "input_layernorm.weight"), st, cos, sin,
                                pos, p + "self_attn.")
        x = x + self._ffn(p + "mlp.", self._norm(x, p + "post_attention_layernorm.weight"))
        hn = self._norm(x, "mtp.norm.weight")
        return self.head(hn), hn
