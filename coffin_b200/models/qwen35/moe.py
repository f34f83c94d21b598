"""Routed mixture-of-experts FFN (top-k softmax routing + one shared expert with a sigmoid gate).

Decode: router logits (one GEMV whose last row is the shared-expert gate vector), a router kernel
(fp32 softmax, top-k, renormalise), two grouped tensor-core GEMVs over the selected experts
(gate/up with fused SwiGLU, then down), the shared expert's two GEMVs and one combine kernel -
8 launches, all graph-capturable, no host round trip.  Prefill sorts the (token, expert) slots by
expert and runs the experts' tcgen05 GEMMs over their row segments.
Reference: ``models/qwen35/moe.py:508-559`` (route, shared expert), ``:561-730`` (dispatch,
grouped projections, merge), kernels ``backends/corex/kernels/moe_grouped*.cu``, ``moe_dispatch.cu``.
"""
from __future__ import annotations

import dataclasses

import torch

import os

from ...config import ModelConfig
from ...ops import kernels as K

# Routed experts of an int8 checkpoint stay int8 (slot GEMV with in-kernel activation quantisation in decode,
# grouped kind::i8 tcgen05 GEMM in prefill).  COFFIN_MOE_I8_GROUPED=0: expand the stacks to bf16 at load.
I8_GROUPED = os.environ.get("COFFIN_MOE_I8_GROUPED", "1") != "0"
PREFILL_CACHE_BYTES = int(float(os.environ.get("COFFIN_MOE_PREFILL_CACHE_GB", "64")) * (1 << 30))
CACHE_HEADROOM = 16 << 30      # HBM that must stay free after an expansion is kept
_cache_used = 0                # bytes of bf16 expansions kept by the process


def keep_expansion(t: torch.Tensor) -> bool:
    """Account a bf16 expansion of int4 weights that its owner wants to keep for later prefill calls;
    False when the budget or the free HBM says it has to be redone per call."""
    global _cache_used
    size = t.numel() * t.element_size()
    if not t.is_cuda or _cache_used + size > PREFILL_CACHE_BYTES or torch.cuda.mem_get_info(t.device)[0] < CACHE_HEADROOM:
        return False
    _cache_used += size
    return True


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


@dataclasses.dataclass
class MoEWeights:
    cfg: ModelConfig
    router: torch.Tensor          # [pad8(E + 1), H]: expert rows, then the shared-expert gate vector
    gate_up: torch.Tensor         # [E, 2I, H]
    down: torch.Tensor            # [E, H, I]
    sh_gu: torch.Tensor | None    # [2S, H]
    sh_down: torch.Tensor | None  # [H, S]
    e_lo: int = 0                 # expert parallel: this rank holds experts [e_lo, e_hi)
    e_hi: int = 0
    ep_world: int = 1
    bufs: dict = dataclasses.field(default_factory=dict)
    _expanded: dict = dataclasses.field(default_factory=dict)   # id(W4 stack) -> kept bf16 expansion

    @classmethod
    def from_state_dict(cls, cfg: ModelConfig, sd: dict, p: str, dev, ep_rank: int = 0, ep_world: int = 1,
                        quant: str = "none"):
        """Expert parallel (``ep_world > 1``): the routed experts are split by contiguous range
        (reference ``expert_range``, ``models/qwen35/parallel.py:238-259``) and the shared expert by
        intermediate columns, so every rank's partial output sums to the full layer output."""
        bf = torch.bfloat16
        E = cfg.num_experts
        rows = [sd[p + "gate.weight"].to(dev, bf)]
        has_shared = (p + "shared_expert.gate_proj.weight") in sd
        if has_shared:
            rows.append(sd[p + "shared_expert_gate.weight"].to(dev, bf).reshape(1, -1))
        n = sum(r.shape[0] for r in rows)
        if _pad8(n) != n:
            rows.append(torch.zeros(_pad8(n) - n, cfg.hidden_size, dtype=bf, device=dev))
        gu, dn = sd[p + "experts.gate_up_proj"], sd[p + "experts.down_proj"]
        if E % ep_world:
            raise ValueError(f"num_experts={E} is not divisible by expert-parallel world {ep_world}")
        per = E // ep_world
        e_lo, e_hi = ep_rank * per, (ep_rank + 1) * per
        from ...weights.quant import QWeight, W4A8Weight
        from .model import QW, QW4
        # a state dict read with an expert-parallel filter already holds only this rank's experts
        presliced = tuple(sd.get("__ep_shard__", ())) == (ep_rank, ep_world) and ep_world > 1
        s_lo, s_hi = (0, per) if presliced else (e_lo, e_hi)

        def experts(t):
            """bf16 stack, or W4A8 codes + scales when the checkpoint (or ``quant``) says so."""
            if isinstance(t, W4A8Weight):
                part = W4A8Weight(t.packed[s_lo:s_hi], t.scale[s_lo:s_hi], t.k, t.group_size)
                return QW4(*part.to(dev).to_nk())
            if isinstance(t, QWeight):
                if I8_GROUPED and t.k % 16 == 0 and t.n % 8 == 0:
                    return QW(t.wq[s_lo:s_hi].to(dev), t.scale[s_lo:s_hi].to(dev))
                # a depth the int8 kernels cannot take (or the switch): expanded once at load
                t = (t.wq[s_lo:s_hi].to(dev).float() * t.scale[s_lo:s_hi].to(dev).float()[..., None]).to(bf)
                s0, s1 = 0, t.shape[0]
            else:
                s0, s1 = s_lo, s_hi
            t = t[s0:s1].to(dev, bf)
            if quant == "w4a8" and t.shape[-1] % 128 == 0:
                return QW4.quantize(t)
            return t.contiguous()

        gu, dn = experts(gu), experts(dn)
        if isinstance(gu, QW) != isinstance(dn, QW):
            # the expert kernels take one storage for the pair: the int8 one is expanded
            def widen(st):
                return (st.wq.float() * st.scale[..., None]).to(bf).contiguous() if isinstance(st, QW) else st
            gu, dn = widen(gu), widen(dn)
        if isinstance(gu, QW4) != isinstance(dn, QW4):
            # one stack cannot be stored as int4 (its reduction length is not a whole number of groups):
            # both stay bf16, the expert kernels take one storage for the pair
            def expand(st):
                if not isinstance(st, QW4):
                    return st
                E_, N_, half = st.wq.shape
                return K.w4_dequant(st.wq.reshape(E_ * N_, half), st.scale.reshape(E_ * N_, -1)).reshape(E_, N_, half * 2)
            gu, dn = expand(gu), expand(dn)
        sh_gu = sh_down = None
        if has_shared:
            from ...weights.quant import QWeight

            def dense(t):            # the shared expert is small: quantised storage is expanded to bf16
                return t.dequant(bf) if isinstance(t, (W4A8Weight, QWeight)) else t

            sg, su = dense(sd[p + "shared_expert.gate_proj.weight"]), dense(sd[p + "shared_expert.up_proj.weight"])
            sdn = dense(sd[p + "shared_expert.down_proj.weight"])
            S = sg.shape[0]
            if S % ep_world:
                raise ValueError("shared expert width must divide by the expert-parallel world")
            c0, c1 = ep_rank * (S // ep_world), (ep_rank + 1) * (S // ep_world)
            sh_gu = torch.cat([sg[c0:c1].to(dev, bf), su[c0:c1].to(dev, bf)]).contiguous()
            sh_down = sdn[:, c0:c1].to(dev, bf).contiguous()
        return cls(cfg, torch.cat(rows).contiguous(), gu, dn, sh_gu, sh_down, e_lo, e_hi, ep_world)

    def tensors(self) -> list[torch.Tensor]:
        return [t for t in (self.router, self.gate_up, self.down, self.sh_gu, self.sh_down) if t is not None]

    @property
    def w4(self) -> bool:
        return hasattr(self.gate_up, "wq") and self.gate_up.wq.dtype == torch.uint8

    @property
    def i8(self) -> bool:
        return hasattr(self.gate_up, "wq") and self.gate_up.wq.dtype == torch.int8

    def _expert(self, stack, e: int) -> torch.Tensor:
        """bf16 ``[rows, K]`` weights of local expert ``e`` (expanded from W4 storage for a prefill GEMM)."""
        if isinstance(stack, torch.Tensor):
            return stack[e]
        if stack.wq.dtype == torch.int8:
            return (stack.wq[e].float() * stack.scale[e][:, None]).to(torch.bfloat16)
        return K.w4_dequant(stack.wq[e], stack.scale[e])

    def _stack(self, stack) -> torch.Tensor:
        """bf16 ``[E, rows, K]`` weights of all local experts.  W4 storage is expanded on the first prefill
        and the expansion is kept while HBM allows (``COFFIN_MOE_PREFILL_CACHE_GB``, default 64, and at least
        ``CACHE_HEADROOM`` bytes left free): decode streams the int4 codes (bandwidth), prefill multiplies
        the bf16 copy on the tensor cores (compute) - expanding 1.6 GB per layer on every call cost three
        times the expert GEMMs themselves.  Without room the expansion is redone per call."""
        if isinstance(stack, torch.Tensor):
            return stack
        hit = self._expanded.get(id(stack))
        if hit is not None:
            return hit
        E, N, half = stack.wq.shape
        out = K.w4_dequant(stack.wq.reshape(E * N, half), stack.scale.reshape(E * N, -1)).reshape(E, N, half * 2)
        kept = keep_expansion(out)
        if kept:
            self._expanded[id(stack)] = out
        from ...engine import debug
        if debug.WQ_TRACE:
            debug.wq_expand(out.shape, kept)
        return out

    # ------------------------------------------------------------------ buffers
    def _b(self, T: int, dev) -> dict:
        b = self.bufs.get(T)
        if b is None:
            c, bf = self.cfg, torch.bfloat16
            k, H, I = c.num_experts_per_tok, c.hidden_size, c.moe_intermediate_size
            b = {"normed": torch.zeros(T, H, dtype=bf, device=dev),
                 "logits": torch.zeros(T, self.router.shape[0], dtype=torch.float32, device=dev),
                 "idx": torch.zeros(T, k, dtype=torch.int32, device=dev),
                 "w": torch.zeros(T, k, dtype=torch.float32, device=dev),
                 "xrow": torch.arange(T, dtype=torch.int32, device=dev).repeat_interleave(k).contiguous(),
                 "inter": torch.zeros(T * k, I, dtype=bf, device=dev),
                 "irow": torch.arange(T * k, dtype=torch.int32, device=dev),
                 "y": torch.zeros(T * k, H, dtype=bf, device=dev)}
            if self.sh_gu is not None:
                S = self.sh_gu.shape[0] // 2
                b["sh_inter"] = torch.zeros(T, S, dtype=bf, device=dev)
                b["sh_out"] = torch.zeros(T, H, dtype=bf, device=dev)
            self.bufs[T] = b
        return b

    # ------------------------------------------------------------------ decode (graph-capturable)
    def forward_decode(self, cur, h, nxt, post_gain, out, model, M: int) -> None:
        """``nxt = cur + h``; ``out = moe(rmsnorm(nxt))`` for ``M`` rows (the caller swaps
        ``cur``/``nxt`` and carries ``out`` into the next layer's norm)."""
        c = self.cfg
        b = self._b(M, cur.device)
        E, k = c.num_experts, c.num_experts_per_tok
        K.rmsnorm(cur, post_gain, model.eps, out=b["normed"], add=h, res_out=nxt)
        tp = model.tp if self.ep_world > 1 or model.tp_force else None
        self._experts(b, M, out, tp=tp, push_site=model.ep_site if tp is not None else -1)

    def _experts(self, b: dict, T: int, out: torch.Tensor, tp=None, push_site: int = -1) -> None:
        c = self.cfg
        E, k, H, I = c.num_experts, c.num_experts_per_tok, c.hidden_size, c.moe_intermediate_size
        normed = b["normed"][:T]
        # router logits: up to 8 rows go through the GEMV (fp32 logits); more rows are one tensor-core GEMM
        # (eight 8-row GEMV launches per layer were a fifth of a 64-row step)
        wide = T > 8
        if wide:
            if "logits_bf" not in b:
                b["logits_bf"] = torch.zeros(T, self.router.shape[0], dtype=torch.bfloat16, device=normed.device)
                if self.sh_gu is not None:
                    b["sh_gu_out"] = torch.zeros(T, self.sh_gu.shape[0], dtype=torch.bfloat16, device=normed.device)
            K.gemm(normed, self.router, out=b["logits_bf"])
            b["logits"][:T].copy_(b["logits_bf"])
            K._count()
        else:
            K.gemv(self.router, normed, b["logits"][:T])
        K.call("moe_router", b["logits"], b["logits"].stride(0), T, E, k, int(c.norm_topk_prob), b["idx"], b["w"],
               self.e_lo, self.e_hi)
        K._count()
        if self.w4:
            K.moe_gemv_w4(self.gate_up.wq, self.gate_up.scale, normed, b["inter"], b["idx"], b["xrow"], swiglu=True)
            K.moe_gemv_w4(self.down.wq, self.down.scale, b["inter"], b["y"], b["idx"], b["irow"])
        elif self.i8:
            K.moe_gemv_i8(self.gate_up.wq, self.gate_up.scale, normed, b["inter"], b["idx"], b["xrow"], swiglu=True)
            K.moe_gemv_i8(self.down.wq, self.down.scale, b["inter"], b["y"], b["idx"], b["irow"])
        else:
            K.call("moe_gemv", self.gate_up, normed, b["inter"], T * k, I, H, I, 1, b["idx"], b["xrow"],
                   self.gate_up.stride(0))
            K.call("moe_gemv", self.down, b["inter"], b["y"], T * k, H, I, H, 0, b["idx"], b["irow"], self.down.stride(0))
            K._count(2)
        shared = gate = None
        if self.sh_gu is not None:
            if wide:
                K.gemm(normed, self.sh_gu, out=b["sh_gu_out"])
                K.swiglu(b["sh_gu_out"], out=b["sh_inter"][:T])
                K.gemm(b["sh_inter"][:T], self.sh_down, out=b["sh_out"][:T])
            else:
                K.gemv(self.sh_gu, normed, b["sh_inter"][:T], swiglu=True)
                K.gemv(self.sh_down, b["sh_inter"][:T], b["sh_out"][:T])
            shared, gate = b["sh_out"], b["logits"][:, E:]
        K.call("moe_combine", b["y"], b["w"], shared, gate, b["logits"].stride(0), out, T, H, k,
               tp.cstruct_ref() if tp is not None and push_site >= 0 else None, push_site)
        K._count()

    # ------------------------------------------------------------------ prefill
    def forward_prefill(self, normed: torch.Tensor, res: torch.Tensor, model) -> None:
        """``res += moe(normed)`` for a prefill chunk."""
        res.add_(self.apply(normed, model))

    def apply(self, normed: torch.Tensor, model=None) -> torch.Tensor:
        """``moe(normed)`` for ``T`` rows (a new ``[T, H]`` tensor).  Small row counts reuse the decode
        kernels (every slot streams its expert once); larger ones sort the slots by expert on the
        device and run two grouped tcgen05 GEMMs over the sorted rows.  ``model`` supplies the all-reduce under
        expert parallelism."""
        c = self.cfg
        T = normed.shape[0]
        E, k, H, I = c.num_experts, c.num_experts_per_tok, c.hidden_size, c.moe_intermediate_size
        if T <= (64 if self.w4 else 32):      # few rows: every slot streams its expert once
            b = self._b(T, normed.device)
            b["normed"][:T].copy_(normed)
            out = torch.empty(T, H, dtype=torch.bfloat16, device=normed.device)
            self._experts(b, T, out)
            if self.ep_world > 1:
                out = model._tp_reduce(out)
            return out
        logits = K.gemm(normed, self.router).float()                       # [T, pad8(E+1)]
        idx = torch.empty(T, k, dtype=torch.int32, device=normed.device)
        w = torch.empty(T, k, dtype=torch.float32, device=normed.device)
        K.call("moe_router", logits, logits.stride(0), T, E, k, int(c.norm_topk_prob), idx, w, self.e_lo, self.e_hi)
        K._count()
        n_local = self.e_hi - self.e_lo
        # device-side dispatch (count -> prefix -> scatter), then one grouped tcgen05 GEMM per
        # projection over the expert-sorted rows; nothing is read back to the host
        disp = K.moe_dispatch(idx, n_local)
        from ...engine import debug
        if debug.MOE_CHECK:
            debug.check_moe_dispatch(idx, disp, n_local)
        if debug.MOE_SHAPE:
            storage = "int4" if self.w4 else "int8" if self.i8 else "bf16"
            debug.moe_shape("gate_up", T * k, n_local, 2 * I, H, storage)
            debug.moe_shape("down", T * k, n_local, H, I, storage)
        if not self.i8:
            xs = normed.index_select(0, disp["src_tok"])                  # gathered activations [T*k, H]
        if self.w4 and K.w4_grouped_ok(H) and K.w4_grouped_ok(I):
            # int4 codes straight into the tensor-core GEMM (expanded inside the CTA), SwiGLU in its epilogue
            inter = K.gemm_w4_grouped(xs, self.gate_up.wq, self.gate_up.scale, disp, swiglu=True)
            y = K.gemm_w4_grouped(inter, self.down.wq, self.down.scale, disp)
        elif self.i8:
            # W8A8: the chunk's rows are quantised once per token and gathered as int8; kind::i8 grouped GEMMs
            q, qs = K.quant_rows(normed)
            src = disp["src_tok"]
            gu = K.gemm_i8_grouped(q.index_select(0, src), qs.index_select(0, src), self.gate_up.wq, self.gate_up.scale, disp)
            iq, iscale = K.quant_rows(gu, swiglu=True)
            y = K.gemm_i8_grouped(iq, iscale, self.down.wq, self.down.scale, disp)
        else:
            gu = K.gemm_grouped(xs, self._stack(self.gate_up), disp)
            inter = K.swiglu(gu)
            y = K.gemm_grouped(inter, self._stack(self.down), disp)
        shared = gate = None
        if self.sh_gu is not None:
            sh = K.gemm_swiglu(normed, self.sh_gu)
            shared = K.gemm(sh, self.sh_down)
            gate = logits[:, E:].contiguous()
        out = torch.empty(T, H, dtype=torch.bfloat16, device=normed.device)
        K.call("moe_combine_pos", y, w, disp["pos"], shared, gate, gate.stride(0) if gate is not None else 0, out, T, H, k)
        K._count()
        if self.ep_world > 1:
            out = model._tp_reduce(out)
        return out
