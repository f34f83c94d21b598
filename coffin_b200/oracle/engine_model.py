"""CPU twin of the device model: same slot / block-table interface, fp32 PyTorch math.

The engine (scheduler, block manager, radix cache, runner) is written against the interface of
``models.qwen35.model.Qwen35Model``.  This class implements that interface with the oracle ops
and a real paged KV pool in host memory, so that the whole engine — prefix reuse, copy-on-write,
preemption, chunked prefill — runs end to end on a machine without a GPU, and so that the device
model can be compared with it call for call.  (The reference tests its engine with a fake model
whose "KV" is the token list, ``tests/test_chunked_prefill.py:53-304``; this twin computes real
logits.)
"""
from __future__ import annotations

import torch

from ..config import LINEAR, ModelConfig
from ..weights.init import LM
from . import ops as O

BLOCK = 64
BUCKETS = (1, 2, 4, 8, 16, 32, 64)


class OracleEngineModel:
    def __init__(self, cfg: ModelConfig, sd: dict[str, torch.Tensor], max_seq: int = 1024, num_slots: int = 4,
                 num_blocks: int | None = None, max_chunk: int = 2048, pp_first: bool = True,
                 pp_last: bool = True) -> None:
        self.cfg = cfg
        self.pp_first, self.pp_last = pp_first, pp_last
        self.lane = 0
        self.input_hidden = None
        self._lanes: dict = {}
        self.sd = {k: v.float() if v.is_floating_point() else v for k, v in sd.items()}
        self.device = torch.device("cpu")
        self.max_seq, self.num_slots, self.max_chunk = max_seq, num_slots, max_chunk
        self.max_blocks_per_seq = (max_seq + BLOCK - 1) // BLOCK
        self.num_blocks = num_blocks or self.max_blocks_per_seq * num_slots + 1
        c = cfg
        self.lin_ids = {li: j for j, li in enumerate(c.linear_layers)}
        self.full_ids = {li: j for j, li in enumerate(c.full_layers)}
        self.state = torch.zeros(len(self.lin_ids), num_slots, c.linear_num_value_heads, c.linear_key_head_dim,
                                 c.linear_value_head_dim)
        self.conv = torch.zeros(len(self.lin_ids), num_slots, c.lin_conv_dim, c.linear_conv_kernel_dim - 1)
        self.kpool = torch.zeros(len(self.full_ids), self.num_blocks * BLOCK, c.num_key_value_heads, c.head_dim)
        self.vpool = torch.zeros_like(self.kpool)
        self._rows: dict | None = None
        self.n_prefill_calls = 0
        self.n_decode_calls = 0

    # ------------------------------------------------------------------ state hooks
    def zero_state(self, slot: int) -> None:
        self.state[:, slot].zero_()
        self.conv[:, slot].zero_()

    def snapshot_state(self, slot: int):
        return self.state[:, slot].clone(), self.conv[:, slot].clone()

    def restore_state(self, slot: int, snap) -> None:
        self.state[:, slot].copy_(snap[0])
        self.conv[:, slot].copy_(snap[1])

    def copy_block(self, src: int, dst: int) -> None:
        s, d = src * BLOCK, dst * BLOCK
        self.kpool[:, d:d + BLOCK] = self.kpool[:, s:s + BLOCK]
        self.vpool[:, d:d + BLOCK] = self.vpool[:, s:s + BLOCK]

    @staticmethod
    def bucket_for(n: int) -> int:
        for m in BUCKETS:
            if n <= m:
                return m
        raise ValueError(f"{n} rows exceed the largest decode bucket")

    def embed_tokens(self, tokens: torch.Tensor) -> torch.Tensor:
        return self.sd[LM + "embed_tokens.weight"][tokens.long()]

    def mrope_rows(self, positions3: torch.Tensor):
        c = self.cfg
        return O.mrope_cos_sin(positions3, c.rotary_dim, c.rope_theta, c.mrope_section)

    # ------------------------------------------------------------------ forward
    def _norm(self, x, key):
        return O.rms_norm(x, 1.0 + self.sd[key], self.cfg.rms_norm_eps)

    def _forward(self, x: torch.Tensor, pos0: int, slot: int, table: torch.Tensor, cos, sin) -> torch.Tensor:
        """Hidden states (pre final norm) of ``T`` consecutive tokens of one sequence."""
        c, sd = self.cfg, self.sd
        T = x.shape[0]
        pos = torch.arange(pos0, pos0 + T)
        slots = table.long()[pos // BLOCK] * BLOCK + pos % BLOCK
        allpos = torch.arange(0, pos0 + T)
        allslots = table.long()[allpos // BLOCK] * BLOCK + allpos % BLOCK
        for li, kind in enumerate(c.layer_types):
            p = f"{LM}layers.{li}."
            h = self._norm(x, p + "input_layernorm.weight")
            if kind == LINEAR:
                j, q = self.lin_ids[li], p + "linear_attn."
                qkv = h @ sd[q + "in_proj_qkv.weight"].t()
                z = h @ sd[q + "in_proj_z.weight"].t()
                b = h @ sd[q + "in_proj_b.weight"].t()
                a = h @ sd[q + "in_proj_a.weight"].t()
                cw = sd[q + "conv1d.weight"].reshape(c.lin_conv_dim, -1)
                conv, new = O.conv1d_silu_seq(cw, qkv, self.conv[j, slot])
                self.conv[j, slot] = new
                nk, nv, dk, dv = (c.linear_num_key_heads, c.linear_num_value_heads, c.linear_key_head_dim,
                                  c.linear_value_head_dim)
                qq = conv[:, :c.lin_kdim].reshape(T, nk, dk)
                kk = conv[:, c.lin_kdim:2 * c.lin_kdim].reshape(T, nk, dk)
                vv = conv[:, 2 * c.lin_kdim:].reshape(T, nv, dv)
                qn, kn, beta, g = O.gdn_head_prep(qq, kk, b, a, sd[q + "A_log"], sd[q + "dt_bias"], c.lin_rep)
                st = self.state[j, slot]
                o = (O.delta_chunked if T > 1 else O.delta_recurrent)(qn, kn, vv, beta, g, st)
                o = O.rms_norm_gated(o, sd[q + "norm.weight"], z.reshape(T, nv, dv), c.rms_norm_eps)
                x = x + o.reshape(T, nv * dv) @ sd[q + "out_proj.weight"].t()
            else:
                j, q = self.full_ids[li], p + "self_attn."
                nh, nkv, hd = c.num_attention_heads, c.num_key_value_heads, c.head_dim
                qg = (h @ sd[q + "q_proj.weight"].t()).reshape(T, nh, 2 * hd)
                qq, gate = qg[..., :hd], qg[..., hd:]
                kk = (h @ sd[q + "k_proj.weight"].t()).reshape(T, nkv, hd)
                vv = (h @ sd[q + "v_proj.weight"].t()).reshape(T, nkv, hd)
                qq = O.apply_rope(O.rms_norm(qq, 1.0 + sd[q + "q_norm.weight"], c.rms_norm_eps), cos, sin, c.rotary_dim)
                kk = O.apply_rope(O.rms_norm(kk, 1.0 + sd[q + "k_norm.weight"], c.rms_norm_eps), cos, sin, c.rotary_dim)
                self.kpool[j, slots] = kk
                self.vpool[j, slots] = vv
                o = O.gated_attention(qq, gate, self.kpool[j, allslots], self.vpool[j, allslots], pos, hd ** -0.5)
                x = x + o.reshape(T, nh * hd) @ sd[q + "o_proj.weight"].t()
            hn = self._norm(x, p + "post_attention_layernorm.weight")
            m = p + "mlp."
            if (m + "gate.weight") in sd:
                shared = None
                if (m + "shared_expert.gate_proj.weight") in sd:
                    shared = (sd[m + "shared_expert.gate_proj.weight"], sd[m + "shared_expert.up_proj.weight"],
                              sd[m + "shared_expert.down_proj.weight"], sd[m + "shared_expert_gate.weight"])
                x = x + O.moe_ffn(hn, sd[m + "gate.weight"], sd[m + "experts.gate_up_proj"], sd[m + "experts.down_proj"],
                                  c.num_experts_per_tok, c.norm_topk_prob, shared)
            else:
                x = x + O.silu_mul(hn @ sd[m + "gate_proj.weight"].t(), hn @ sd[m + "up_proj.weight"].t()) \
                    @ sd[m + "down_proj.weight"].t()
        return x

    def _head(self, x: torch.Tensor) -> torch.Tensor:
        w = self.sd.get("lm_head.weight", self.sd[LM + "embed_tokens.weight"])
        return self._norm(x, LM + "norm.weight") @ w.t()

    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor, pos0: int, slot: int, block_table: torch.Tensor,
                embeds: torch.Tensor | None = None, cos_sin=None, want_logits: bool = True, want_hidden: bool = False):
        self.n_prefill_calls += 1
        c = self.cfg
        T = tokens.numel()
        x = self.embed_tokens(tokens) if embeds is None else embeds.float()
        if cos_sin is None:
            pos = torch.arange(pos0, pos0 + T)
            cos, sin = O.mrope_cos_sin(pos.reshape(1, -1).expand(3, -1), c.rotary_dim, c.rope_theta, c.mrope_section)
        else:
            cos, sin = cos_sin
        x = self._forward(x, pos0, slot, block_table, cos, sin)
        self.last_prenorm = x
        if not self.pp_last:
            return None
        self.last_hidden = self._norm(x, LM + "norm.weight") if want_hidden else None
        return self._head(x[-1:])[0] if want_logits else None

    @torch.no_grad()
    def prefill_group(self, items: list[tuple], want_logits: list[bool] | None = None, **kw) -> list:
        """Chunks of several sequences (``(tokens, pos0, slot, block_table)`` each); the twin runs them one
        after the other, which is what the stacked forward of the device model computes."""
        self.n_group_calls = getattr(self, "n_group_calls", 0) + 1
        want = want_logits if want_logits is not None else [True] * len(items)
        return [self.prefill(t, p0, slot, bt, want_logits=w) for (t, p0, slot, bt), w in zip(items, want)]

    def set_rows(self, M, tokens, positions, slots, block_tables, rope_deltas=None) -> None:
        self._rows = dict(tokens=list(tokens), positions=list(positions), slots=list(slots),
                          tables=[list(t) for t in block_tables],
                          deltas=list(rope_deltas) if rope_deltas else [0] * len(tokens),
                          next=torch.zeros(M, dtype=torch.int64), hidden=torch.zeros(M, self.cfg.hidden_size))
        self._lanes[(M, self.lane)] = self._rows

    def _row_buffers(self, M: int) -> dict:
        return self._lanes[(M, self.lane)]

    def stage_hidden(self, M: int) -> torch.Tensor:
        """Residual stream after this stage's layers for the rows of the last decode step."""
        return self._row_buffers(M)["hidden"]

    def advance_rows(self, M: int) -> None:
        r = self._row_buffers(M)
        n = len(r["tokens"])
        r["tokens"] = [int(t) for t in r["next"][:n]]
        r["positions"] = [p + 1 for p in r["positions"]]

    @torch.no_grad()
    def decode(self, M: int, graph: bool = True):
        self.n_decode_calls += 1
        r, c = self._lanes.get((M, self.lane), self._rows), self.cfg
        n = len(r["tokens"])
        logits = torch.zeros(M, c.vocab_size)
        for i in range(n):
            pos = r["positions"][i]
            rp = torch.tensor([pos + r["deltas"][i]])
            cos, sin = O.mrope_cos_sin(rp.reshape(1, -1).expand(3, -1), c.rotary_dim, c.rope_theta, c.mrope_section)
            if self.input_hidden is not None:
                x = self.input_hidden[i:i + 1].float()
            else:
                x = self.embed_tokens(torch.tensor([r["tokens"][i]]))
            x = self._forward(x, pos, r["slots"][i], torch.tensor(r["tables"][i], dtype=torch.int32), cos, sin)
            r["hidden"][i] = x[0]
            if self.pp_last:
                logits[i] = self._head(x)[0]
        r["next"] = logits.argmax(-1)
        return r["next"], logits

    @torch.no_grad()
    def verify_batch(self, rows: list[tuple]) -> torch.Tensor:
        """Logits ``[R, C, vocab]`` of ``C`` consecutive tokens of each row ``(tokens, pos0, slot,
        block_table, rope_delta)``; the delta-net states are restored afterwards and ``commit_batch``
        replays each row's accepted prefix."""
        c = self.cfg
        self._verify = []
        out = []
        for tokens, pos0, slot, block_table, rope_delta in rows:
            table = block_table.clone() if isinstance(block_table, torch.Tensor) else torch.tensor(list(block_table), dtype=torch.int32)
            snap = self.snapshot_state(slot)
            self._verify.append((list(tokens), pos0, table, rope_delta, snap, slot))
            T = len(tokens)
            pos = torch.arange(pos0, pos0 + T) + rope_delta
            cos, sin = O.mrope_cos_sin(pos.reshape(1, -1).expand(3, -1), c.rotary_dim, c.rope_theta, c.mrope_section)
            x = self._forward(self.embed_tokens(torch.tensor(list(tokens))), pos0, slot, table, cos, sin)
            out.append(self._head(x))
            self.restore_state(slot, snap)
        return torch.stack(out)

    def commit_batch(self, slots: list[int], steps: list[int]) -> None:
        c = self.cfg
        for (tokens, pos0, table, delta, snap, slot0), slot, n_accept in zip(self._verify, slots, steps):
            assert slot == slot0
            self.restore_state(slot, snap)
            if n_accept > 0:
                pos = torch.arange(pos0, pos0 + n_accept) + delta
                cos, sin = O.mrope_cos_sin(pos.reshape(1, -1).expand(3, -1), c.rotary_dim, c.rope_theta, c.mrope_section)
                self._forward(self.embed_tokens(torch.tensor(tokens[:n_accept])), pos0, slot, table, cos, sin)

    def verify(self, tokens: list[int], pos0: int, slot: int, block_table: torch.Tensor, rope_delta: int = 0) -> torch.Tensor:
        return self.verify_batch([(tokens, pos0, slot, block_table, rope_delta)])[0]

    def commit(self, slot: int, n_accept: int) -> None:
        self.commit_batch([slot], [n_accept])

    def sample(self, logits: torch.Tensor, temps, us) -> torch.Tensor:
        """Greedy when ``temps`` is None; else per-row inverse-CDF sampling with uniforms ``us``
        (rows with temperature <= 0 stay greedy)."""
        if temps is None:
            return logits.argmax(-1)
        out = []
        for i, (t, u) in enumerate(zip(temps, us)):
            if t <= 0:
                out.append(int(logits[i].argmax()))
                continue
            cdf = torch.softmax(logits[i].double() / t, -1).cumsum(0)
            idx = int(torch.searchsorted(cdf, torch.tensor(u * float(cdf[-1]), dtype=torch.float64), right=True))
            out.append(min(idx, logits.shape[1] - 1))
        return torch.tensor(out)
