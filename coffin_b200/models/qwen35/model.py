"""Qwen3.5-style hybrid model on one B200 (optionally one tensor-parallel shard).

Execution model
---------------
* Weights are repacked once at load into the shapes the kernels read: per layer one fused
  input projection (``q|k|v|z|b|a`` for a delta-net layer, ``q+gate|k|v`` for an attention
  layer), one fused ``gate|up`` matrix, all ``[N, K]`` bf16 (the checkpoint layout is already
  K-major, which is what both the GEMV and the tcgen05 GEMM want).
* Decode is a CUDA graph per row bucket (1, 2, 4, 8): 5 launches per delta-net layer, 6 per
  attention layer — residual add + RMSNorm are folded into the projections, SwiGLU into the
  gate/up projection, conv + head prep + delta rule + gated norm into one kernel, q/k norm +
  rotary + KV append into the attention kernel (the reference runs ~26 launches per layer,
  ``docs/DECODE-LAUNCH-LEDGER.md:15-23``, and keeps graphs disabled,
  ``backends/corex/__init__.py:2830-2896``).
* Prefill runs one sequence chunk at a time through tcgen05 GEMMs (residual add fused in the
  epilogue), the chunked delta-net scan and paged flash attention.
* Sequence state lives in caller-assigned *slots* (delta-net recurrent state + conv ring) and
  in a paged KV pool addressed through block tables, so the engine's block manager, radix
  cache and scheduler own placement; this class owns no policy.

Structure reference: ``models/qwen35/model.py:81-266`` (init), ``:515-604`` (decode forward),
``:641-858`` (prefill), ``:1093-1349`` (graph capture, row buckets).
"""
from __future__ import annotations

import dataclasses

import torch

from ...config import LINEAR, ModelConfig
from ...ops import kernels as K
from ...oracle import ops as O
from ...weights.init import LM

BUCKETS = (1, 2, 4, 8, 16, 32, 64)
WIDE = 8          # buckets above this run their projections on the tcgen05 GEMM instead of the GEMV


class QW:
    """Device-resident int8 projection: ``wq [N, K]`` int8 + per-row ``scale [N]`` (W8A8)."""

    def __init__(self, wq: torch.Tensor, scale: torch.Tensor) -> None:
        self.wq, self.scale = wq.contiguous(), scale.float().contiguous()

    @property
    def shape(self):
        return self.wq.shape

    def __getitem__(self, sl):
        return QW(self.wq[sl], self.scale[sl])

    def numel(self) -> int:
        return self.wq.numel()

    def element_size(self) -> int:
        return 1

    def data_ptr(self) -> int:
        return self.wq.data_ptr()

    @classmethod
    def quantize(cls, w: torch.Tensor) -> "QW":
        from ...weights.quant import QWeight
        q = QWeight.quantize(w)
        return cls(q.wq, q.scale)


class QW4:
    """Device-resident W4A8 projection: codes ``[N, K/2]`` uint8 + group scales ``[N, K/128]`` fp32
    (``weights.quant.W4A8Weight.to_nk``).  A leading expert axis is allowed."""

    def __init__(self, wq: torch.Tensor, scale: torch.Tensor) -> None:
        self.wq, self.scale = wq.contiguous(), scale.float().contiguous()

    @property
    def shape(self):
        return (*self.wq.shape[:-1], self.wq.shape[-1] * 2)

    def __getitem__(self, sl):
        return QW4(self.wq[sl], self.scale[sl])

    def numel(self) -> int:
        return self.wq.numel()

    def element_size(self) -> int:
        return 1

    def data_ptr(self) -> int:
        return self.wq.data_ptr()

    @classmethod
    def quantize(cls, w: torch.Tensor) -> "QW4":
        from ...weights.quant import W4A8Weight
        return cls(*W4A8Weight.quantize(w).to_nk())

    @classmethod
    def zeros(cls, rows: int, K: int, device) -> "QW4":
        return cls(torch.full((rows, K // 2), 0x88, dtype=torch.uint8, device=device),
                   torch.full((rows, K // 128), 1e-8, dtype=torch.float32, device=device))

    def dequant(self) -> torch.Tensor:
        """bf16 ``[N, K]`` (2-D only)."""
        return K.w4_dequant(self.wq, self.scale)

    def expanded(self) -> torch.Tensor:
        """The bf16 expansion for a tensor-core GEMM, kept after the first call while HBM allows: decode
        streams the int4 codes (bandwidth bound), prefill and wide decode buckets multiply the bf16 copy
        (compute bound) instead of expanding the projection on every call."""
        kept = getattr(self, "_kept", None)
        if kept is not None:
            return kept
        out = self.dequant()
        from .moe import keep_expansion
        if keep_expansion(out):
            self._kept = out
        return out


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


@dataclasses.dataclass
class LayerWeights:
    kind: str
    in_gain: torch.Tensor
    post_gain: torch.Tensor
    w_in: torch.Tensor          # fused input projection [N_in, H]
    w_out: torch.Tensor         # [H, mixer_width]
    w_gu: torch.Tensor | None   # [2I, H]
    w_down: torch.Tensor | None  # [H, I]
    # delta net
    conv_w: torch.Tensor | None = None
    A_log: torch.Tensor | None = None
    dt_bias: torch.Tensor | None = None
    norm_w: torch.Tensor | None = None
    # attention
    qg: torch.Tensor | None = None
    kg: torch.Tensor | None = None
    moe: object | None = None


class Qwen35Model:
    """sm_100a execution of the hybrid model. ``sd`` uses the HF key layout."""

    def __init__(self, cfg: ModelConfig, sd: dict[str, torch.Tensor], device: str | torch.device = "cuda",
                 max_seq: int = 4096, num_slots: int = 2, num_blocks: int | None = None,
                 max_chunk: int = 2048, pdl: bool = True, free_source: bool = False, tp=None,
                 full_cfg: ModelConfig | None = None, quant: str = "none", ep_rank: int = 0, ep_world: int = 1,
                 pp_first: bool = True, pp_last: bool = True, kv_dtype: str = "bf16") -> None:
        """``cfg`` is the geometry this instance computes (a tensor-parallel shard gets its local
        head / channel counts, ``full_cfg`` the unsharded model and ``tp`` the communicator)."""
        self.cfg = cfg
        self.quant = quant
        if kv_dtype not in ("bf16", "int8"):
            raise ValueError(f"kv_dtype {kv_dtype!r}: expected bf16 or int8")
        self.kv_dtype = kv_dtype
        # pipeline stage: a non-first stage starts from a received hidden state instead of the
        # embedding, a non-last stage ends at the residual stream instead of the logits
        self.pp_first, self.pp_last = pp_first, pp_last
        self.lane = 0              # micro-batch lane: decode buffers and graphs are kept per (bucket, lane)
        self.ep_rank, self.ep_world, self.ep_site = ep_rank, ep_world, -1
        self.tp = tp
        # under expert parallelism the communicator spans the ranks but the dense weights are
        # replicated: the model is not tensor-parallel
        self.tp_world = tp.world if (tp is not None and ep_world == 1) else 1
        self.tp_rank = tp.rank if (tp is not None and ep_world == 1) else 0
        self.full_cfg = full_cfg or cfg
        self.device = torch.device(device)
        self.max_seq = int(max_seq)
        self.num_slots = int(num_slots)
        self.max_chunk = int(max_chunk)
        self.max_blocks_per_seq = (self.max_seq + K.BLOCK - 1) // K.BLOCK
        self.num_blocks = int(num_blocks) if num_blocks else self.max_blocks_per_seq * self.num_slots + 1
        self.eps = cfg.rms_norm_eps
        K.status_word(self.device)
        K._lib.set_pdl(pdl)
        dev, bf = self.device, torch.bfloat16
        c = cfg

        from ...weights.quant import QWeight, W4A8Weight

        def w(key: str):
            t = sd.pop(key) if free_source else sd[key]
            if isinstance(t, QWeight):                      # pre-quantised int8 checkpoint
                return QW(t.wq.to(dev), t.scale.to(dev))
            if isinstance(t, W4A8Weight):                   # int4 group-128 storage
                if t.k % t.group_size == 0 and t.group_size == 128:
                    return QW4(*t.to(dev).to_nk())
                t = t.dequant(bf)                           # odd K: computed as bf16
            return t.to(device=dev, dtype=bf)

        def cat(parts):
            """Row-concatenate projections; int8 parts keep their per-row scales."""
            if any(isinstance(p_, QW4) for p_ in parts) or quant == "w4a8":
                def w4(p_):
                    if isinstance(p_, QW4):
                        return p_
                    if not bool(p_.any()):                  # zero padding rows
                        return QW4.zeros(p_.shape[0], p_.shape[1], dev)
                    return QW4.quantize(p_)
                parts = [w4(p_) for p_ in parts]
                return QW4(torch.cat([p_.wq for p_ in parts]), torch.cat([p_.scale for p_ in parts]))
            if any(isinstance(p_, QW) for p_ in parts):
                parts = [p_ if isinstance(p_, QW) else QW.quantize(p_) for p_ in parts]
                return QW(torch.cat([p_.wq for p_ in parts]), torch.cat([p_.scale for p_ in parts]))
            t = torch.cat(parts).contiguous()
            return QW.quantize(t) if quant == "int8" else t

        def one(t):
            if isinstance(t, (QW, QW4)):
                return t
            if quant == "w4a8" and t.shape[1] % 128 == 0:
                return QW4.quantize(t)
            return QW.quantize(t) if quant == "int8" else t.contiguous()

        def gain(key: str, centred: bool = True) -> torch.Tensor:
            t = sd[key].to(device=dev, dtype=torch.float32)
            return (1.0 + t).contiguous() if centred else t.contiguous()

        self.embed = w(LM + "embed_tokens.weight") if LM + "embed_tokens.weight" in sd else None
        if isinstance(self.embed, QW):
            self.embed = (self.embed.wq.float() * self.embed.scale[:, None]).to(bf)
        if isinstance(self.embed, QW4):
            self.embed = self.embed.dequant()
        if self.embed is not None:
            self.embed = self.embed.contiguous()
        self.lm_head = None
        if pp_last:
            self.lm_head = one(w("lm_head.weight")) if "lm_head.weight" in sd else one(self.embed)
        self.vocab_local = c.vocab_size
        if self.tp_world > 1:       # vocabulary-parallel head: this rank scores a contiguous slice
            if c.vocab_size % self.tp_world:
                raise ValueError("vocab_size must divide by the tensor-parallel world")
            self.vocab_local = c.vocab_size // self.tp_world
            self.lm_head = self.lm_head[self.tp_rank * self.vocab_local:(self.tp_rank + 1) * self.vocab_local]
        self.final_gain = gain(LM + "norm.weight")
        self.layers: list[LayerWeights] = []
        for i, kind in enumerate(c.layer_types):
            p = f"{LM}layers.{i}."
            if kind == LINEAR:
                q = p + "linear_attn."
                parts = [w(q + "in_proj_qkv.weight"), w(q + "in_proj_z.weight"),
                         w(q + "in_proj_b.weight"), w(q + "in_proj_a.weight")]
                n = sum(t.shape[0] for t in parts)
                if _pad8(n) != n:
                    parts.append(torch.zeros(_pad8(n) - n, c.hidden_size, dtype=bf, device=dev))
                lw = LayerWeights(
                    kind=kind, in_gain=gain(p + "input_layernorm.weight"),
                    post_gain=gain(p + "post_attention_layernorm.weight"),
                    w_in=cat(parts), w_out=one(w(q + "out_proj.weight")),
                    w_gu=None, w_down=None,
                    conv_w=sd[q + "conv1d.weight"].to(dev, torch.float32).reshape(c.lin_conv_dim, -1).contiguous(),
                    A_log=sd[q + "A_log"].to(dev, torch.float32).contiguous(),
                    dt_bias=sd[q + "dt_bias"].to(dev, torch.float32).contiguous(),
                    norm_w=gain(q + "norm.weight", centred=False))
            else:
                q = p + "self_attn."
                lw = LayerWeights(
                    kind=kind, in_gain=gain(p + "input_layernorm.weight"),
                    post_gain=gain(p + "post_attention_layernorm.weight"),
                    w_in=cat([w(q + "q_proj.weight"), w(q + "k_proj.weight"), w(q + "v_proj.weight")]),
                    w_out=one(w(q + "o_proj.weight")), w_gu=None, w_down=None,
                    qg=gain(q + "q_norm.weight"), kg=gain(q + "k_norm.weight"))
            m = p + "mlp."
            if c.is_moe:
                from .moe import MoEWeights
                lw.moe = MoEWeights.from_state_dict(c, sd, m, dev, ep_rank, ep_world, quant=quant)
            else:
                lw.w_gu = cat([w(m + "gate_proj.weight"), w(m + "up_proj.weight")])
                lw.w_down = one(w(m + "down_proj.weight"))
            self.layers.append(lw)
        # ---- rotary tables -------------------------------------------------------------
        cos, sin = O.rope_tables(c.rotary_dim, c.rope_theta, self.max_seq + 64)
        self.cos, self.sin = cos.to(dev).contiguous(), sin.to(dev).contiguous()
        # ---- sequence state ------------------------------------------------------------
        self.lin_ids = {li: j for j, li in enumerate(c.linear_layers)}
        self.full_ids = {li: j for j, li in enumerate(c.full_layers)}
        nl, nf = len(self.lin_ids), len(self.full_ids)
        self.state = torch.zeros(nl, self.num_slots, c.linear_num_value_heads, c.linear_key_head_dim,
                                 c.linear_value_head_dim, dtype=torch.float32, device=dev)
        self.ring = torch.zeros(nl, self.num_slots, K.RING, c.lin_conv_dim, dtype=bf, device=dev)
        # KV pool: bf16, or int8 with one fp32 scale per (token, kv head) - half the bytes per key read
        # (reference: int8 pools + scales, cache/paged_cache.py:78-141)
        kvt = torch.int8 if kv_dtype == "int8" else bf
        self.kpool = torch.zeros(nf, self.num_blocks * K.BLOCK, c.num_key_value_heads, c.head_dim, dtype=kvt, device=dev)
        self.vpool = torch.zeros_like(self.kpool)
        self.kscale = self.vscale = None
        if kv_dtype == "int8":
            self.kscale = torch.zeros(nf, self.num_blocks * K.BLOCK, c.num_key_value_heads, dtype=torch.float32, device=dev)
            self.vscale = torch.zeros_like(self.kscale)
        # ---- prefill workspace (allocated lazily at the largest chunk seen) ----------------
        self._pf: dict | None = None
        self._pf_rows = 0
        self._rows: dict[int, dict] = {}
        self._graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self.graph_pool = None
        self.input_hidden = None   # when set, a decode step starts from this [M, H] input instead of the token embedding
        self.tp_force = False      # run the push/pull path even with world == 1 (single-GPU test of the protocol)
        self._step_launches: dict[int, int] = {}
        self._w4_part: dict[int, torch.Tensor] = {}
        # persistent decode kernel (one cooperative launch per step), planned on first use
        self.mega = None
        self._mega_planned = False
        self.use_mega = True
        # tensor parallel: whether a decode step must leave the full-vocabulary logits on every rank
        # (sampling with a temperature needs them; greedy decoding only needs the arg-max, which the
        # persistent kernel reduces across ranks itself)
        self.full_logits = True

    @property
    def max_decode_rows(self) -> int:
        """Rows one decode step can carry: the widest bucket, or the narrow-bucket limit when the
        multi-rank exchange of the wide path is not available for this model."""
        multi = self.tp is not None and (self.tp_world > 1 or self.ep_world > 1)
        return BUCKETS[-1] if (not multi or self.wide_parallel_ok()) else WIDE

    def wide_parallel_ok(self) -> bool:
        """Whether buckets above ``WIDE`` rows run under tensor / expert parallelism: the exchange of
        the wide step is the communicator's peer-memory prefill region."""
        if self.tp is None:
            return False
        import torch.distributed as dist
        return self.tp.pf_rows >= BUCKETS[-1] or (dist.is_available() and dist.is_initialized())   # NCCL between kernels otherwise

    def _kvs(self, j: int) -> dict:
        """Scale tensors of attention layer ``j`` for the attention kernels (empty for a bf16 pool)."""
        if self.kscale is None:
            return {}
        return {"kscale": self.kscale[j], "vscale": self.vscale[j]}

    def launches_per_step(self, M: int) -> int:
        """Kernels launched by one decode step of bucket ``M`` (counted while capturing)."""
        return self._step_launches.get(M, 0)

    # ------------------------------------------------------------------ projection dispatch
    def _gemv(self, W, x, out, **kw):
        """Decode projection on whichever storage the weight has (bf16 or int8 W8A8)."""
        if isinstance(W, QW):
            kw.pop("tail", None)
            return K.gemv_i8(W.wq, W.scale, x, out, **kw)
        if isinstance(W, QW4):
            kw.pop("tail", None)
            if kw.get("tp") is not None and kw.get("push_site", -1) >= 0:
                # row-parallel int4 projection under tensor parallelism: fp32 partial rows, then a small
                # kernel stores them into every rank's inbox (the int4 GEMV has no push epilogue)
                M = kw.get("rows") or x.shape[0]
                part = self._w4_part.get(M)
                if part is None:
                    part = self._w4_part[M] = torch.empty(M, self.cfg.hidden_size, dtype=torch.float32, device=self.device)
                K.gemv_w4(W.wq, W.scale, x, part[:, :W.shape[0]])
                K.call("tp_push_rows", kw["tp"].cstruct_ref(), kw["push_site"], part, part.stride(0), M, W.shape[0])
                K._count()
                return None
            norm = kw.get("norm")
            if kw.get("tp") is not None and kw.get("pull_site", -1) >= 0:
                # expert parallel: the sum pushed by the MoE combine is pulled, added and normalised by
                # the one-CTA kernel; the W4 projection then takes plain rows
                res_in, _add, gain, res_out, eps = norm
                x, norm = K._pull_norm_rows(kw["tp"], kw["pull_site"], res_in, gain, res_out, eps), None
            return K.gemv_w4(W.wq, W.scale, x, out, swiglu=kw.get("swiglu", False), norm=norm)
        return K.gemv(W, x, out, **kw)

    def _gemm(self, A, W, out=None, residual=None, swiglu_in: bool = False, push=None, aq=None):
        """Prefill projection.  ``swiglu_in``: ``A`` is a ``[T, 2I]`` gate|up tensor whose SwiGLU
        product is the real input (fused into the activation quantisation on the int8 path).
        ``push``: the tensor-parallel communicator; the epilogue then sends the partial rows to their
        owners instead of writing ``out`` (``_tp_finish`` completes the all-reduce)."""
        if isinstance(W, QW):
            q, sc = aq if aq is not None else K.quant_rows(A, swiglu=swiglu_in)     # aq: rows quantised by the producing kernel
            return K.gemm_i8(q, sc, W.wq, W.scale, out=out, residual=residual, push=push)
        if isinstance(W, QW4):
            W = W.expanded()                # bf16 copy (kept while HBM allows); the tcgen05 GEMM does the rest
        if swiglu_in:
            A = K.swiglu(A)
        return K.gemm(A, W, out=out, residual=residual, push=push)

    def _gemm_gu(self, A, W, gu: torch.Tensor, aq=None):
        """Gate|up projection of a prefill chunk into ``gu [T, 2I]``.  bf16 weights and more rows than one
        CTA-pair tile: the SwiGLU product comes out of the GEMM epilogue and the ``[T, I]`` view holding it
        is returned; otherwise ``gu`` is filled with both halves and None is returned."""
        if isinstance(W, QW4):
            W = W.expanded()
        if K.PAIR_GEMM and gu.shape[0] >= K.PAIR_MIN_ROWS and W.shape[0] >= 256:
            if isinstance(W, QW):
                q, sc = aq if aq is not None else K.quant_rows(A)
                return K.gemm_i8_swiglu(q, sc, W.wq, W.scale, out=gu[:, :W.shape[0] // 2])
            return K.gemm_swiglu(A, W, out=gu[:, :W.shape[0] // 2])
        self._gemm(A, W, out=gu, aq=aq)
        return None

    def _row_parallel(self, A, W, scratch: torch.Tensor, swiglu_in: bool = False) -> torch.Tensor:
        """Row-parallel projection + all-reduce.  With a peer-memory region the all-reduce is a
        reduce-scatter + all-gather over NVLink: for a prefill chunk the tcgen05 GEMM epilogue leaves its
        partial rows in this rank's peer-visible buffer and publishes a sequence number; for the few
        rows of a decode bucket the K-split GEMM (one wave of CTAs, which a 128-row tile per CTA would
        not fill) writes the partial rows and a small kernel copies them there.  A reduce/gather kernel
        on every rank then pulls the rows it owns from all ranks, adds them and stores the sums to every rank.  Without the region the partial result is all-reduced by NCCL."""
        if self.tp is not None and self.tp.pf_rows:
            if A.shape[0] <= 128 and K.SPLITK_GEMM:
                self._gemm(A, W, out=scratch, swiglu_in=swiglu_in)
                self.tp.scatter(scratch)
            else:
                self._gemm(A, W, swiglu_in=swiglu_in, push=self.tp)
            return self.tp.finish_reduce()
        return self._tp_reduce(self._gemm(A, W, out=scratch, swiglu_in=swiglu_in))

    # ------------------------------------------------------------------ sizes
    @property
    def in_width(self) -> int:
        return max(l.w_in.shape[0] for l in self.layers)

    @property
    def mix_width(self) -> int:
        c = self.cfg
        return max(c.lin_vdim, c.num_attention_heads * c.head_dim)

    def weight_bytes(self) -> int:
        """Bytes of weights one decode step streams on this rank: every projection and the (local
        slice of the) lm_head.  The embedding table is not counted (a step gathers one row of it)."""
        seen, total = set(), 0
        tensors = [t for t in (self.lm_head,) if t is not None]
        for l in self.layers:
            tensors += [l.w_in, l.w_out] + ([l.w_gu, l.w_down] if l.w_gu is not None else [])
            if l.moe is not None:
                tensors += l.moe.tensors()
        for t in tensors:
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    # ------------------------------------------------------------------ sequence state
    def zero_state(self, slot: int) -> None:
        self.state[:, slot].zero_()
        self.ring[:, slot].zero_()

    def snapshot_state(self, slot: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Clone of the slot's delta-net state (recurrent matrices + conv ring)."""
        return self.state[:, slot].clone(), self.ring[:, slot].clone()

    def restore_state(self, slot: int, snap: tuple[torch.Tensor, torch.Tensor]) -> None:
        self.state[:, slot].copy_(snap[0])
        self.ring[:, slot].copy_(snap[1])

    def copy_block(self, src: int, dst: int) -> None:
        """Copy one KV block in every attention layer (copy-on-write of a shared tail block)."""
        s, d = src * K.BLOCK, dst * K.BLOCK
        self.kpool[:, d:d + K.BLOCK].copy_(self.kpool[:, s:s + K.BLOCK])
        self.vpool[:, d:d + K.BLOCK].copy_(self.vpool[:, s:s + K.BLOCK])
        if self.kscale is not None:
            self.kscale[:, d:d + K.BLOCK].copy_(self.kscale[:, s:s + K.BLOCK])
            self.vscale[:, d:d + K.BLOCK].copy_(self.vscale[:, s:s + K.BLOCK])

    # ------------------------------------------------------------------ prefill
    def _prefill_ws(self, T: int) -> dict:
        if self._pf is None or self._pf_rows < T:
            c, dev, bf = self.cfg, self.device, torch.bfloat16
            rows = max(T, min(self.max_chunk, 256))
            H = c.hidden_size
            ws = {
                "res": torch.empty(rows, H, dtype=bf, device=dev),
                "normed": torch.empty(rows, H, dtype=bf, device=dev),
                "proj": torch.empty(rows, self.in_width, dtype=bf, device=dev),
                "act": torch.empty(rows, self.mix_width, dtype=bf, device=dev),
                "q": torch.empty(rows, c.num_attention_heads, c.head_dim, dtype=bf, device=dev),
                "slots": torch.empty(rows, dtype=torch.int32, device=dev),
                "ridx": torch.empty(rows, dtype=torch.int32, device=dev),
            }
            if self.tp is not None:
                ws["part"] = torch.empty(rows, H, dtype=bf, device=dev)
            if any(isinstance(lw.w_in, QW) for lw in self.layers):
                ws["q8"] = torch.empty(rows, H, dtype=torch.int8, device=dev)
                ws["s8"] = torch.empty(rows, dtype=torch.float32, device=dev)
            if not c.is_moe:
                ws["gu"] = torch.empty(rows, 2 * c.intermediate_size, dtype=bf, device=dev)
                ws["inter"] = torch.empty(rows, c.intermediate_size, dtype=bf, device=dev)
            if self.lin_ids:
                n = K.gdn_prefill_scratch_floats(rows, c.linear_num_key_heads, c.linear_num_value_heads,
                                                 c.linear_key_head_dim, c.linear_value_head_dim)
                ws["gdn"] = torch.empty(n, dtype=torch.float32, device=dev)
            self._pf, self._pf_rows = ws, rows
        return self._pf

    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor, pos0: int, slot: int, block_table: torch.Tensor,
                embeds: torch.Tensor | None = None, cos_sin: tuple[torch.Tensor, torch.Tensor] | None = None,
                want_logits: bool = True, want_hidden: bool = False):
        """Run ``tokens`` (int64 ``[T]`` on the device) of one sequence at positions
        ``pos0..pos0+T-1``.

        ``block_table`` (int32 on the device) lists the sequence's pool blocks from position 0.
        ``embeds [T, H]`` overrides the token embeddings (image rows scattered in);
        ``cos_sin`` gives per-token rotary rows ``[T, rot]`` (mRoPE) instead of the 1-D table.
        Returns fp32 logits ``[vocab]`` of the last token (or ``None``).
        """
        out = self.prefill_group([(tokens, pos0, slot, block_table)], embeds=embeds, cos_sin=cos_sin,
                                 want_logits=[want_logits], want_hidden=want_hidden)
        return out[0]

    @torch.no_grad()
    def prefill_group(self, items: list[tuple], embeds: torch.Tensor | None = None,
                      cos_sin: tuple[torch.Tensor, torch.Tensor] | None = None, want_logits: list[bool] | None = None,
                      want_hidden: bool = False) -> list:
        """Chunks of several sequences in ONE forward: ``items[i] = (tokens [T_i], pos0, slot,
        block_table)``.  The rows of all chunks are stacked, so every projection is one GEMM over
        ``sum(T_i)`` rows (short prompts share weight tiles instead of each streaming the weights); the
        delta-net scan and the attention, which are per sequence, run per chunk on its row range.
        ``embeds`` / ``cos_sin`` cover the stacked rows (only used with a single item by the engine).
        Returns, per item, the fp32 logits ``[vocab]`` of its last token or ``None``
        (reference: ``models/qwen35/model.py:861`` ``prefill_group``)."""
        c = self.cfg
        lens = [int(it[0].numel()) for it in items]
        T = sum(lens)
        assert all(n > 0 for n in lens) and T <= self.max_chunk, f"group of {T} tokens exceeds max_chunk {self.max_chunk}"
        want_logits = list(want_logits) if want_logits is not None else [True] * len(items)
        for (toks, pos0, slot, bt), n in zip(items, lens):
            self._check_row(pos0, n, int(bt.numel()), 0, slot)
        ws = self._prefill_ws(T)
        res, normed = ws["res"][:T], ws["normed"][:T]
        tokens = items[0][0] if len(items) == 1 else torch.cat([it[0] for it in items])
        if embeds is None:
            K.embed_gather(self.embed, tokens, res)
        else:
            res.copy_(embeds)
        offs = [0]
        for n in lens:
            offs.append(offs[-1] + n)
        slots = ws["slots"][:T]
        ridx = ws["ridx"][:T] if cos_sin is None else None
        for i, (it, n) in enumerate(zip(items, lens)):          # pool slots (and 1-D rotary rows): one small kernel per chunk
            bt = it[3] if it[3].dtype == torch.int32 and it[3].is_contiguous() else it[3].to(torch.int32).contiguous()
            K.call("prefill_index", bt, it[1], n, K.BLOCK, slots[offs[i]:offs[i + 1]],
                   ridx[offs[i]:offs[i + 1]] if ridx is not None else None)
            K._count()
        if cos_sin is None:
            cos, sin = self.cos, self.sin
        else:
            cos, sin = cos_sin[0].float().contiguous(), cos_sin[1].float().contiguous()
            ridx = None
        q8 = (ws["q8"][:T], ws["s8"][:T]) if "q8" in ws else None
        for li, lw in enumerate(self.layers):
            # an int8 projection takes its int8 rows straight from the norm kernel (no bf16 copy, no quantise launch)
            aq = q8 if isinstance(lw.w_in, QW) else None
            K.rmsnorm(res, lw.in_gain, self.eps, out=None if aq else normed, quant=aq)
            n_in = lw.w_in.shape[0]
            proj = ws["proj"][:T, :n_in]
            self._gemm(normed, lw.w_in, out=proj, aq=aq)
            if lw.kind == LINEAR:
                j = self.lin_ids[li]
                act = ws["act"][:T, :c.lin_vdim]
                for i, (it, n) in enumerate(zip(items, lens)):
                    sl = slice(offs[i], offs[i + 1])
                    K.gdn_prefill(proj[sl], lw.conv_w, lw.A_log, lw.dt_bias, lw.norm_w, self.ring[j, it[2]],
                                  self.state[j, it[2]], ws["gdn"], act[sl], pos0=it[1], nk=c.linear_num_key_heads,
                                  nv=c.linear_num_value_heads, dk=c.linear_key_head_dim, dv=c.linear_value_head_dim,
                                  eps=self.eps)
            else:
                j = self.full_ids[li]
                act = ws["act"][:T, :c.num_attention_heads * c.head_dim]
                q = ws["q"][:T]
                K.attn_prep(proj, lw.qg, lw.kg, cos, sin, ridx, slots, q, self.kpool[j], self.vpool[j],
                            nh=c.num_attention_heads, nkv=c.num_key_value_heads, hd=c.head_dim,
                            rot=c.rotary_dim, eps=self.eps, **self._kvs(j))
                for i, (it, n) in enumerate(zip(items, lens)):
                    sl = slice(offs[i], offs[i + 1])
                    K.attn_prefill(q[sl], proj[sl], self.kpool[j], self.vpool[j], it[3], act[sl], q_pos0=it[1],
                                   nh=c.num_attention_heads, nkv=c.num_key_value_heads, hd=c.head_dim, **self._kvs(j))
            aq = q8 if lw.moe is None and isinstance(lw.w_gu, QW) else None
            if self.tp_world > 1 or (self.tp_force and not c.is_moe):
                part = self._row_parallel(act, lw.w_out, ws["part"][:T])
                K.rmsnorm(res, lw.post_gain, self.eps, out=None if aq else normed, add=part, res_out=res, quant=aq)
            else:
                self._gemm(act, lw.w_out, out=res, residual=res)
                K.rmsnorm(res, lw.post_gain, self.eps, out=None if aq else normed, quant=aq)
            if lw.moe is not None:
                lw.moe.forward_prefill(normed, res, self)
            else:
                gu = ws["gu"][:T]
                fused = self._gemm_gu(normed, lw.w_gu, gu, aq=aq)       # SwiGLU taken in the epilogue: gu[:, :I] is the product
                if fused is not None:
                    gu = fused
                if self.tp_world > 1 or self.tp_force:
                    res.add_(self._row_parallel(gu, lw.w_down, ws["part"][:T], swiglu_in=fused is None))
                else:
                    self._gemm(gu, lw.w_down, out=res, residual=res, swiglu_in=fused is None)
        self.last_hidden = None
        self.last_prenorm = res            # last-layer residual stream of the group (view of the workspace)
        out: list = [None] * len(items)
        if not self.pp_last:
            return out
        if want_hidden:
            self.last_hidden = K.rmsnorm(res, self.final_gain, self.eps)
        for i in range(len(items)):
            if want_logits[i]:
                last = offs[i + 1] - 1
                local = torch.empty(1, self.vocab_local, dtype=torch.float32, device=self.device)
                self._gemv(self.lm_head, None, local, norm=(res[last:last + 1].contiguous(), None, self.final_gain, None, self.eps))
                out[i] = self._gather_logits(local, 1)[0]
        return out

    # ------------------------------------------------------------------ tensor-parallel helpers
    def _tp_reduce(self, t: torch.Tensor) -> torch.Tensor:
        """All-reduce of a ``[T, hidden]`` prefill tensor whose producer is not a GEMM (the MoE
        combine under expert parallelism): scatter + reduce/gather over peer memory when the
        communicator has a prefill region, NCCL otherwise.  Returns the reduced rows (``t`` itself
        with NCCL, a view of the communicator's result buffer otherwise)."""
        if self.tp is not None and self.tp.pf_rows and t.shape[0] <= self.tp.pf_rows:
            from ...engine import debug
            from ...parallel.tp import OS_ROWS
            end = debug.ep_span()
            if t.shape[0] <= OS_ROWS:           # a decode bucket: one NVLink crossing, two launches
                out = torch.empty_like(t)
                self.tp.oneshot(t, res_out=out)
            else:
                self.tp.scatter(t)
                out = self.tp.finish_reduce()
            if end is not None:
                end.record()
            return out
        if self.tp_world == 1 and self.ep_world == 1:
            return t
        import torch.distributed as dist
        dist.all_reduce(t)
        K._count()
        return t

    def _gather_logits(self, local: torch.Tensor, M: int) -> torch.Tensor:
        """``[M, vocab/world]`` per rank -> ``[M, vocab]`` on every rank."""
        if self.tp_world == 1:
            return local
        import torch.distributed as dist
        buf = torch.empty(self.tp_world, M, self.vocab_local, dtype=local.dtype, device=self.device)
        dist.all_gather_into_tensor(buf, local.contiguous())
        K._count()
        if M == 1:
            return buf.reshape(1, -1)
        return buf.permute(1, 0, 2).reshape(M, -1)

    # ------------------------------------------------------------------ decode
    def _row_buffers(self, M: int) -> dict:
        key = M if self.lane == 0 else (M, self.lane)
        b = self._rows.get(key)
        if b is None:
            c, dev, bf = self.cfg, self.device, torch.bfloat16
            H = c.hidden_size
            nsplit = K.decode_splits(c.num_key_value_heads, M)
            b = {
                "tokens": torch.zeros(M, dtype=torch.int64, device=dev),
                "positions": torch.full((M,), -1, dtype=torch.int32, device=dev),
                "rope_pos": torch.zeros(M, dtype=torch.int32, device=dev),
                "slots": torch.full((M,), -1, dtype=torch.int32, device=dev),
                "block_table": torch.zeros(M, self.max_blocks_per_seq, dtype=torch.int32, device=dev),
                "res": [torch.zeros(M, H, dtype=bf, device=dev) for _ in range(2)],
                "h": torch.zeros(M, H, dtype=bf, device=dev),
                "h2": torch.zeros(M, H, dtype=bf, device=dev),
                "proj": torch.zeros(M, self.in_width, dtype=bf, device=dev),
                "act_lin": torch.zeros(M, c.lin_vdim, dtype=bf, device=dev),
                "act_full": torch.zeros(M, c.num_attention_heads * c.head_dim, dtype=bf, device=dev),
                "inter": torch.zeros(M, max(1, c.intermediate_size), dtype=bf, device=dev),
                "logits": torch.zeros(M, c.vocab_size, dtype=torch.float32, device=dev),
                "logits_local": None,
                "next": torch.zeros(M, dtype=torch.int64, device=dev),
                "next_local": torch.zeros(M, dtype=torch.int64, device=dev),
                "hidden": torch.zeros(M, H, dtype=bf, device=dev),
                "nsplit": nsplit,
                "part_o": torch.zeros(M, c.num_attention_heads, nsplit, c.head_dim, dtype=torch.float32, device=dev),
                "part_ml": torch.zeros(M, c.num_attention_heads, nsplit, 2, dtype=torch.float32, device=dev),
                "tickets": torch.zeros(M, c.num_key_value_heads, dtype=torch.int32, device=dev),
                # host staging (pinned) so that set_rows is one async copy per array
                "h_tokens": torch.zeros(M, dtype=torch.int64).pin_memory(),
                "h_meta": torch.zeros(3, M, dtype=torch.int32).pin_memory(),
                "h_bt": torch.zeros(M, self.max_blocks_per_seq, dtype=torch.int32).pin_memory(),
            }
            b["logits_local"] = (b["logits"] if self.tp_world == 1 else
                                 torch.zeros(M, self.vocab_local, dtype=torch.float32, device=dev))
            if M > WIDE:
                b["normed"] = torch.zeros(M, H, dtype=bf, device=dev)
                if not c.is_moe:
                    b["gu"] = torch.zeros(M, 2 * c.intermediate_size, dtype=bf, device=dev)
                b["logits_bf"] = torch.zeros(M, self.vocab_local, dtype=bf, device=dev)
                if self.tp is not None:
                    b["part"] = torch.zeros(M, H, dtype=bf, device=dev)
            self._rows[key] = b
        return b

    def _decode_body(self, M: int) -> None:
        """One decode step for the ``M`` rows staged in the bucket's buffers (graph-capturable).

        Tensor parallel: the two row-parallel projections of a layer push their partial sums to all
        ranks (sites ``2*layer`` and ``2*layer + 1``); a one-CTA kernel per row pulls the sum, adds the
        residual and normalises, and the following projection copies the result - no collective call."""
        if M > WIDE:
            return self._decode_body_wide(M)
        c, b = self.cfg, self._row_buffers(M)
        if self._mega_for(M) is not None:
            # the whole step is one cooperative launch: projections, mixers, all-reduces and arg-max
            self.mega.launch(M, advance=self._advance)
            b["final_res"] = b["res"][1]
            if self.tp_world > 1 and self.full_logits:
                b["logits"].copy_(self._gather_logits(b["logits_local"], M))
            return
        comm = self.tp if (self.tp is not None and (self.tp_world > 1 or self.ep_world > 1 or self.tp_force)) else None
        tp = comm if (self.ep_world == 1 and not self.cfg.is_moe) else None     # dense row-parallel push/pull
        cur, nxt = b["res"]
        if comm is not None:
            comm.epoch_bump()
        if self.input_hidden is not None:
            cur.copy_(self.input_hidden)
        else:
            K.embed_gather(self.embed, b["tokens"], cur)
        carry, pull = None, -1
        for li, lw in enumerate(self.layers):
            n_in = lw.w_in.shape[0]
            proj = b["proj"][:, :n_in]
            have = carry is not None or pull >= 0
            self._gemv(lw.w_in, None, proj, norm=(cur, carry, lw.in_gain, nxt if have else None, self.eps),
                       tp=comm, pull_site=pull)
            if have:
                cur, nxt = nxt, cur
            if lw.kind == LINEAR:
                j = self.lin_ids[li]
                act = b["act_lin"]
                K.gdn_decode(proj, lw.conv_w, lw.A_log, lw.dt_bias, lw.norm_w, self.ring[j], self.state[j],
                             b["slots"], b["positions"], act, nk=c.linear_num_key_heads,
                             nv=c.linear_num_value_heads, dk=c.linear_key_head_dim, dv=c.linear_value_head_dim,
                             eps=self.eps)
            else:
                j = self.full_ids[li]
                act = b["act_full"]
                K.attn_decode(proj, lw.qg, lw.kg, self.cos, self.sin, b["positions"], b["rope_pos"],
                              b["block_table"], self.kpool[j], self.vpool[j], b["part_o"], b["part_ml"], b["tickets"], act,
                              nh=c.num_attention_heads, nkv=c.num_key_value_heads, hd=c.head_dim,
                              rot=c.rotary_dim, nsplit=b["nsplit"], eps=self.eps, **self._kvs(j))
            if tp is not None:
                # the pushing kernel's last CTA also pulls the ranks' sums, adds the residual and applies the
                # post-attention norm, so the gate|up projection below starts from finished rows
                self._gemv(lw.w_out, act, None, tp=tp, push_site=2 * li, rows=M,
                           tail=(cur, lw.post_gain if lw.moe is None else None, nxt, self.eps))
            else:
                self._gemv(lw.w_out, act, b["h"])
            if lw.moe is not None:
                # expert parallel: the combine kernel pushes this rank's partial sum to every rank and
                # the next projection pulls the total (site 2 * layer + 1)
                ep = self.tp is not None and (self.ep_world > 1 or self.tp_force)
                self.ep_site = 2 * li + 1
                lw.moe.forward_decode(cur, b["h"], nxt, lw.post_gain, b["h2"], self, M)
                cur, nxt = nxt, cur
                carry, pull = (None, 2 * li + 1) if ep else (b["h2"], -1)
                continue
            self._gemv(lw.w_gu, None, b["inter"], swiglu=True,
                   norm=(cur, None if tp is not None else b["h"], lw.post_gain, nxt, self.eps),
                   tp=tp, pull_site=2 * li if tp is not None else -1)
            cur, nxt = nxt, cur
            if tp is not None:
                nxt_gain = self.layers[li + 1].in_gain if li + 1 < len(self.layers) else (self.final_gain if self.pp_last else None)
                self._gemv(lw.w_down, b["inter"], None, tp=tp, push_site=2 * li + 1, rows=M,
                           tail=(cur, nxt_gain, nxt, self.eps))
                carry, pull = None, 2 * li + 1
            else:
                self._gemv(lw.w_down, b["inter"], b["h2"])
                carry, pull = b["h2"], -1
        if not self.pp_last:
            # pipeline hand-off: the residual stream that the next stage starts from
            if carry is not None:
                torch.add(cur, carry, out=b["hidden"])
            else:
                b["hidden"].copy_(cur)
            K._count()
            return
        self._gemv(self.lm_head, None, b["logits_local"], norm=(cur, carry, self.final_gain, nxt, self.eps),
                   tp=comm, pull_site=pull)
        if self.tp_world > 1 and not self.full_logits and self.tp.n_sites > 2 * len(self.layers):
            # greedy rows only need the arg-max: each rank's best {value, index} goes through the inbox
            # (site after the layers' sites) instead of an all-gather of the logits
            K.argmax(b["logits_local"], b["next_local"])
            K.call("tp_argmax", self.tp.cstruct_ref(), 2 * len(self.layers), b["logits_local"], b["logits_local"].stride(0),
                   b["next_local"], self.tp_rank * self.vocab_local, b["next"], M)
            K._count()
        else:
            if self.tp_world > 1:
                b["logits"].copy_(self._gather_logits(b["logits_local"], M))
            K.argmax(b["logits"], b["next"])
        b["final_res"] = nxt
        if self._advance:
            self.advance_rows(M)

    def _mega_for(self, M: int):
        """The persistent-kernel launcher when bucket ``M`` of this model runs on it, else ``None``."""
        if not self._mega_planned:
            self._mega_planned = True
            from .mega import MegaDecode
            self.mega = MegaDecode.plan(self)
        if self.mega is None or not self.use_mega or self.input_hidden is not None or not self.mega.rows_ok(M):
            return None
        return self.mega

    def _decode_body_wide(self, M: int) -> None:
        """One decode step for a wide bucket (16..64 rows): every row still advances by one token
        through the per-row state kernels (delta-net step, split-KV attention with the fused KV
        append), but the projections run on the tcgen05 GEMM - at these row counts one 128-row tile
        streams each weight once, which is what the GEMV would do eight rows at a time.

        Tensor parallel: the row-parallel projections all-reduce in one kernel per site (peer stores paired
        with sequence numbers), or through the prefill path's reduce/gather exchange (partial rows left in a
        peer-visible buffer, owners pull them;
        its sequence numbers live on the device, so the step is captured in a CUDA graph like any
        other).  Expert parallel: the routed-expert output goes through the same exchange."""
        multi = self.tp is not None and (self.tp_world > 1 or self.ep_world > 1)
        if multi and not self.wide_parallel_ok():
            raise NotImplementedError("wide decode buckets need the peer-memory prefill region of the communicator")
        c, b = self.cfg, self._row_buffers(M)
        tpw = self.tp_world > 1
        res, normed = b["res"][0], b["normed"]
        if self.input_hidden is not None:
            res.copy_(self.input_hidden)
        else:
            K.embed_gather(self.embed, b["tokens"], res)
        # int8 projections take their activation rows already quantised from the norm (or all-reduce + norm)
        # kernel that produced them: no quantisation launch between the two
        i8 = isinstance(self.layers[0].w_in, QW)
        if i8 and "aq" not in b:
            b["aq"] = (torch.empty(M, c.hidden_size, dtype=torch.int8, device=self.device),
                       torch.empty(M, dtype=torch.float32, device=self.device))
        aq = b["aq"] if i8 else None
        for li, lw in enumerate(self.layers):
            if aq is not None and isinstance(lw.w_in, QW):
                K.rmsnorm(res, lw.in_gain, self.eps, quant=aq)
            else:
                K.rmsnorm(res, lw.in_gain, self.eps, out=normed)
            proj = b["proj"][:, :lw.w_in.shape[0]]
            self._gemm(normed, lw.w_in, out=proj, aq=aq if isinstance(lw.w_in, QW) else None)
            if lw.kind == LINEAR:
                j = self.lin_ids[li]
                act = b["act_lin"]
                K.gdn_decode(proj, lw.conv_w, lw.A_log, lw.dt_bias, lw.norm_w, self.ring[j], self.state[j],
                             b["slots"], b["positions"], act, nk=c.linear_num_key_heads,
                             nv=c.linear_num_value_heads, dk=c.linear_key_head_dim, dv=c.linear_value_head_dim,
                             eps=self.eps)
            else:
                j = self.full_ids[li]
                act = b["act_full"]
                K.attn_decode(proj, lw.qg, lw.kg, self.cos, self.sin, b["positions"], b["rope_pos"],
                              b["block_table"], self.kpool[j], self.vpool[j], b["part_o"], b["part_ml"], b["tickets"], act,
                              nh=c.num_attention_heads, nkv=c.num_key_value_heads, hd=c.head_dim,
                              rot=c.rotary_dim, nsplit=b["nsplit"], eps=self.eps, **self._kvs(j))
            if tpw and self.tp.pf_rows:
                # K-split GEMM, then the one-shot all-reduce whose second kernel also adds the residual and
                # applies the post-attention norm
                self._gemm(act, lw.w_out, out=b["part"])
                gq = aq if (lw.moe is None and isinstance(lw.w_gu, QW)) else None
                self.tp.oneshot(b["part"], residual=res, gain=lw.post_gain, res_out=res, normed=None if gq else normed,
                                eps=self.eps, quant=gq)
            elif tpw:
                gq = None
                part = self._row_parallel(act, lw.w_out, b["part"])
                K.rmsnorm(res, lw.post_gain, self.eps, out=normed, add=part, res_out=res)
            else:
                gq = aq if (lw.moe is None and isinstance(lw.w_gu, QW)) else None
                self._gemm(act, lw.w_out, out=res, residual=res)
                if gq is not None:
                    K.rmsnorm(res, lw.post_gain, self.eps, quant=gq)
                else:
                    K.rmsnorm(res, lw.post_gain, self.eps, out=normed)
            if lw.moe is not None:
                res.add_(lw.moe.apply(normed, self))
                K._count()
            else:
                self._gemm(normed, lw.w_gu, out=b["gu"], aq=gq)
                if tpw and self.tp.pf_rows:
                    self._gemm(b["gu"], lw.w_down, out=b["part"], swiglu_in=True)
                    self.tp.oneshot(b["part"], residual=res, res_out=res)
                elif tpw:
                    res.add_(self._row_parallel(b["gu"], lw.w_down, b["part"], swiglu_in=True))
                    K._count()
                else:
                    self._gemm(b["gu"], lw.w_down, out=res, residual=res, swiglu_in=True)
        if not self.pp_last:
            b["hidden"].copy_(res)
            K._count()
            return
        hq = aq if isinstance(self.lm_head, QW) else None
        if hq is not None:
            K.rmsnorm(res, self.final_gain, self.eps, quant=hq)
        else:
            K.rmsnorm(res, self.final_gain, self.eps, out=normed)
        self._gemm(normed, self.lm_head, out=b["logits_bf"], aq=hq)
        if tpw:
            # vocabulary-parallel head: every rank needs the arg-max over the whole vocabulary
            b["logits_local"].copy_(b["logits_bf"])
            K._count()
            if not self.full_logits and self.tp.n_sites > 2 * len(self.layers):
                # greedy rows: each rank's best {value, index} per row through the inbox, no logits gather
                self.tp.epoch_bump()
                K.argmax(b["logits_local"], b["next_local"])
                K.call("tp_argmax", self.tp.cstruct_ref(), 2 * len(self.layers), b["logits_local"],
                       b["logits_local"].stride(0), b["next_local"], self.tp_rank * self.vocab_local, b["next"], M)
                K._count()
            else:
                b["logits"].copy_(self._gather_logits(b["logits_local"], M))
                K.argmax(b["logits"], b["next"])
        else:
            b["logits"].copy_(b["logits_bf"])
            K._count()
            K.argmax(b["logits"], b["next"])
        b["final_res"] = res
        if self._advance:
            self.advance_rows(M)

    def set_rows(self, M: int, tokens, positions, slots, block_tables, rope_deltas=None) -> None:
        """Stage up to ``M`` rows (lists of per-row values); missing rows are padding."""
        b = self._row_buffers(M)
        n = len(tokens)
        if n > M:
            raise ValueError(f"{n} rows do not fit bucket {M}")
        for r in range(n):
            self._check_row(positions[r], 1, len(block_tables[r]), rope_deltas[r] if rope_deltas else 0, slots[r])
        ht, hm, hb = b["h_tokens"], b["h_meta"], b["h_bt"]
        # the pinned staging arrays are reused: wait until the copies of the previous call have left them
        # (a caller that queues steps without synchronising would otherwise overwrite rows in flight)
        ev = b.get("h_event")
        if ev is None:
            ev = b["h_event"] = torch.cuda.Event()
        else:
            ev.synchronize()
        ht.zero_()
        hm[0].fill_(-1)
        hm[1].zero_()
        hm[2].fill_(-1)
        for r in range(n):
            ht[r] = tokens[r]
            hm[0, r] = positions[r]
            hm[1, r] = positions[r] + (rope_deltas[r] if rope_deltas else 0)
            hm[2, r] = slots[r]
            bt = block_tables[r]
            hb[r, :len(bt)] = torch.as_tensor(bt, dtype=torch.int32)
        b["tokens"].copy_(ht, non_blocking=True)
        b["positions"].copy_(hm[0], non_blocking=True)
        b["rope_pos"].copy_(hm[1], non_blocking=True)
        b["slots"].copy_(hm[2], non_blocking=True)
        b["block_table"].copy_(hb, non_blocking=True)
        ev.record()

    def _check_row(self, pos0: int, n: int, table_len: int, rope_delta: int = 0, slot: int = 0) -> None:
        """Host-side guard of everything a kernel indexes with a position: ``n`` tokens from ``pos0``
        must lie inside the row's block table, the rotary table and the window; the slot must exist.
        The kernels trust these values (they index the block table, the cos/sin tables and the KV pool
        with them), so a bad request must stop here, not on the device."""
        end = pos0 + n
        if pos0 < 0 or end > self.max_seq or end > table_len * K.BLOCK or table_len > self.max_blocks_per_seq:
            raise ValueError(f"positions {pos0}..{end - 1} outside the block table ({table_len} blocks) "
                             f"or the {self.max_seq}-token window")
        if not (0 <= pos0 + rope_delta and end + rope_delta <= self.cos.shape[0]):
            raise ValueError(f"rotary positions {pos0 + rope_delta}..{end + rope_delta - 1} outside the table")
        if not (0 <= slot < self.num_slots):
            raise ValueError(f"state slot {slot} outside 0..{self.num_slots - 1}")

    _advance = False

    def _gkey(self, M: int, advance: bool):
        return (M, self.lane, bool(advance), bool(self.full_logits) if self.tp_world > 1 else True, bool(self.use_mega))

    def capture(self, M: int, warmup: int = 2, advance: bool = False) -> None:
        """Capture the decode step of bucket ``M`` into a CUDA graph. Warm-up runs use padded
        rows (slot -1 / position -1) so that no sequence state is touched.  ``advance``: the step
        also feeds the sampled tokens back and advances the positions (a graph of its own)."""
        gkey = self._gkey(M, advance)
        if gkey in self._graphs:
            return
        self._advance = bool(advance)
        b = self._row_buffers(M)
        saved = (b["positions"].clone(), b["slots"].clone(), b["tokens"].clone(), b["rope_pos"].clone())
        b["positions"].fill_(-1)
        b["slots"].fill_(-1)
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(warmup):
                self._decode_body(M)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        if self.graph_pool is None:
            self.graph_pool = torch.cuda.graph_pool_handle()
        l0 = K.LAUNCHES
        with K.capture_graph(g, pool=self.graph_pool):
            self._decode_body(M)
        self._step_launches[M] = K.LAUNCHES - l0
        self._graphs[gkey] = g
        self._advance = False
        b["positions"].copy_(saved[0])
        b["slots"].copy_(saved[1])
        b["tokens"].copy_(saved[2])
        b["rope_pos"].copy_(saved[3])

    @torch.no_grad()
    def decode(self, M: int, graph: bool = True, advance: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
        """Run one decode step on the staged rows. Returns ``(next_tokens [M], logits [M, V])``
        device tensors owned by the bucket (overwritten by the next step).  ``advance``: the step
        ends by feeding the sampled tokens back and advancing the positions, so that a caller can
        run greedy steps back to back without touching the rows.  Under tensor parallelism the
        logits hold the full vocabulary only while ``full_logits`` is set."""
        b = self._row_buffers(M)
        if graph:
            gkey = self._gkey(M, advance)
            if gkey not in self._graphs:
                self.capture(M, advance=advance)
            self._graphs[gkey].replay()
        else:
            self._advance = bool(advance)
            try:
                self._decode_body(M)
            finally:
                self._advance = False
        return b["next"], b["logits"]

    def stage_hidden(self, M: int) -> torch.Tensor:
        """Residual stream after this pipeline stage's layers for the rows of the last decode step."""
        return self._row_buffers(M)["hidden"]

    def final_hidden(self, M: int, normed: bool = True) -> torch.Tensor:
        """Last-layer residual stream of the previous decode step (``normed``: after the final norm)."""
        res = self._row_buffers(M)["final_res"]
        return K.rmsnorm(res, self.final_gain, self.eps) if normed else res

    def advance_rows(self, M: int) -> None:
        """Feed the sampled tokens back and advance positions by one (one small kernel, no host sync):
        lets a caller run many greedy steps back to back."""
        b = self._row_buffers(M)
        K.call("advance_rows", b["tokens"], b["next"], b["positions"], b["rope_pos"], M)
        K._count()

    # ------------------------------------------------------------------ speculative verification
    VERIFY_WIDTHS = (2, 4, 8)

    def _verify_buffers(self, R: int, C: int) -> dict:
        """Buffers of a verify pass over ``R`` sequences x ``C`` tokens (``R`` a power of two)."""
        key = ("verify", R, C)
        b = self._rows.get(key)
        if b is None:
            c, dev, bf = self.cfg, self.device, torch.bfloat16
            H, N = c.hidden_size, R * C
            b = {
                "tokens": torch.zeros(N, dtype=torch.int64, device=dev),
                "res": [torch.zeros(N, H, dtype=bf, device=dev) for _ in range(2)],
                "h": torch.zeros(N, H, dtype=bf, device=dev), "h2": torch.zeros(N, H, dtype=bf, device=dev),
                "normed": torch.zeros(N, H, dtype=bf, device=dev),
                "proj": torch.zeros(N, self.in_width, dtype=bf, device=dev),
                "act_lin": torch.zeros(N, c.lin_vdim, dtype=bf, device=dev),
                "act_full": torch.zeros(N, c.num_attention_heads * c.head_dim, dtype=bf, device=dev),
                "q": torch.zeros(N, c.num_attention_heads, c.head_dim, dtype=bf, device=dev),
                "inter": torch.zeros(N, max(1, c.intermediate_size), dtype=bf, device=dev),
                "gu": torch.zeros(N, max(1, 2 * c.intermediate_size), dtype=bf, device=dev) if N > WIDE else None,
                "logits": torch.zeros(N, c.vocab_size, dtype=torch.float32, device=dev),
                "logits_bf": torch.zeros(N, self.vocab_local, dtype=bf, device=dev) if N > WIDE else None,
                "slot": torch.full((R,), -1, dtype=torch.int32, device=dev),
                "pos": torch.zeros(R, dtype=torch.int32, device=dev),
                "kv_slots": torch.full((N,), -1, dtype=torch.int32, device=dev),
                "ridx": torch.zeros(N, dtype=torch.int32, device=dev),
                "record": torch.zeros(len(self.lin_ids), R, C, c.linear_num_value_heads,
                                      c.linear_key_head_dim + c.linear_value_head_dim + 1,
                                      dtype=torch.float32, device=dev),
                "steps": torch.zeros(R, dtype=torch.int32, device=dev),
            }
            self._rows[key] = b
        return b

    @torch.no_grad()
    def verify_batch(self, rows: list[tuple]) -> torch.Tensor:
        """Score ``C`` consecutive tokens (the last sampled token followed by drafts) of each of ``R``
        sequences in one pass over the weights.  ``rows[i] = (tokens[C], pos0, slot, block_table,
        rope_delta)`` with the same ``C`` in (2, 4, 8) for every row and ``R * C <= 64``; returns
        logits ``[R, C, vocab]``.  KV rows of all positions are written (rejected ones are overwritten
        later); the delta-net states are left untouched and the per-token rank-one updates are
        recorded, so that ``commit_batch`` can apply each row's accepted prefix.  Up to 8 token rows
        run on the decode projections, more on the tcgen05 GEMM (reference: batched speculative step,
        ``models/qwen35/model.py:1351-1759``)."""
        c = self.cfg
        n = len(rows)
        C = len(rows[0][0])
        assert C in self.VERIFY_WIDTHS and all(len(r[0]) == C for r in rows), "verify width must be 2, 4 or 8 for every row"
        R = 1
        while R < n:
            R *= 2
        N = R * C
        if N > BUCKETS[-1]:
            raise ValueError(f"{n} rows x {C} tokens exceed the {BUCKETS[-1]} token rows of one verify pass")
        if N > WIDE and self.tp is not None and (self.tp_world > 1 or self.ep_world > 1):
            raise NotImplementedError("a verify pass of more than 8 token rows is single-GPU")
        tables = []
        for toks, pos0, slot, table, delta in rows:
            tl = table.tolist() if isinstance(table, torch.Tensor) else list(table)
            self._check_row(pos0, C, len(tl), delta, slot)
            tables.append(tl)
        b = self._verify_buffers(R, C)
        h_tok = torch.zeros(N, dtype=torch.int64)
        h_slot = torch.full((R,), -1, dtype=torch.int32)
        h_pos = torch.zeros(R, dtype=torch.int32)
        h_kv = torch.full((N,), -1, dtype=torch.int32)
        h_ridx = torch.zeros(N, dtype=torch.int32)
        for i, (toks, pos0, slot, _t, delta) in enumerate(rows):
            h_tok[i * C:(i + 1) * C] = torch.as_tensor(list(toks), dtype=torch.int64)
            h_slot[i], h_pos[i] = slot, pos0
            for j in range(C):
                p = pos0 + j
                h_kv[i * C + j] = tables[i][p // K.BLOCK] * K.BLOCK + p % K.BLOCK
                h_ridx[i * C + j] = p + delta
        b["tokens"].copy_(h_tok)
        b["slot"].copy_(h_slot)
        b["pos"].copy_(h_pos)
        b["kv_slots"].copy_(h_kv)
        b["ridx"].copy_(h_ridx)
        dev_tables = [torch.tensor(t, dtype=torch.int32, device=self.device) for t in tables]
        wide = N > WIDE
        cur, nxt = b["res"]
        K.embed_gather(self.embed, b["tokens"], cur)
        carry = None
        for li, lw in enumerate(self.layers):
            proj = b["proj"][:, :lw.w_in.shape[0]]
            if wide:
                K.rmsnorm(cur, lw.in_gain, self.eps, out=b["normed"])
                self._gemm(b["normed"], lw.w_in, out=proj)
            else:
                self._gemv(lw.w_in, None, proj, norm=(cur, carry, lw.in_gain, nxt if carry is not None else None, self.eps))
                if carry is not None:
                    cur, nxt = nxt, cur
            if lw.kind == LINEAR:
                j = self.lin_ids[li]
                act = b["act_lin"]
                K.gdn_decode(proj, lw.conv_w, lw.A_log, lw.dt_bias, lw.norm_w, self.ring[j], self.state[j], b["slot"],
                             b["pos"], act, nk=c.linear_num_key_heads, nv=c.linear_num_value_heads,
                             dk=c.linear_key_head_dim, dv=c.linear_value_head_dim, eps=self.eps, ntok=C,
                             record=b["record"][j], write_state=False)
            else:
                j = self.full_ids[li]
                act = b["act_full"]
                K.attn_prep(proj, lw.qg, lw.kg, self.cos, self.sin, b["ridx"], b["kv_slots"], b["q"], self.kpool[j],
                            self.vpool[j], nh=c.num_attention_heads, nkv=c.num_key_value_heads, hd=c.head_dim,
                            rot=c.rotary_dim, eps=self.eps, **self._kvs(j))
                for i, (_tk, pos0, _s, _t, _d) in enumerate(rows):
                    sl = slice(i * C, (i + 1) * C)
                    K.attn_prefill(b["q"][sl], proj[sl], self.kpool[j], self.vpool[j], dev_tables[i], act[sl], q_pos0=pos0,
                                   nh=c.num_attention_heads, nkv=c.num_key_value_heads, hd=c.head_dim, **self._kvs(j))
            if wide:
                self._gemm(act, lw.w_out, out=cur, residual=cur)
                K.rmsnorm(cur, lw.post_gain, self.eps, out=b["normed"])
                if lw.moe is not None:
                    cur.add_(lw.moe.apply(b["normed"], self))
                    K._count()
                else:
                    self._gemm(b["normed"], lw.w_gu, out=b["gu"])
                    self._gemm(b["gu"], lw.w_down, out=cur, residual=cur, swiglu_in=True)
                continue
            self._gemv(lw.w_out, act, b["h"])
            if lw.moe is not None:
                lw.moe.forward_decode(cur, b["h"], nxt, lw.post_gain, b["h2"], self, N)
                cur, nxt = nxt, cur
            else:
                self._gemv(lw.w_gu, None, b["inter"], swiglu=True, norm=(cur, b["h"], lw.post_gain, nxt, self.eps))
                cur, nxt = nxt, cur
                self._gemv(lw.w_down, b["inter"], b["h2"])
            carry = b["h2"]
        if wide:
            K.rmsnorm(cur, self.final_gain, self.eps, out=b["normed"])
            self._gemm(b["normed"], self.lm_head, out=b["logits_bf"])
            b["logits"].copy_(b["logits_bf"])
            K._count()
            b["final_res"] = cur
        else:
            self._gemv(self.lm_head, None, b["logits"], norm=(cur, carry, self.final_gain, nxt, self.eps))
            b["final_res"] = nxt
        self._verify_shape = (R, C, n)
        return b["logits"].view(R, C, -1)[:n]

    def commit_batch(self, slots: list[int], steps: list[int]) -> None:
        """Apply, for row ``i`` of the last ``verify_batch`` call, its first ``steps[i]`` recorded
        delta-net updates to the state of ``slots[i]``."""
        c = self.cfg
        R, C, n = self._verify_shape
        assert len(slots) == len(steps) == n
        b = self._verify_buffers(R, C)
        h_steps = torch.zeros(R, dtype=torch.int32)
        h_slot = torch.full((R,), -1, dtype=torch.int32)
        h_steps[:n] = torch.as_tensor(steps, dtype=torch.int32)
        h_slot[:n] = torch.as_tensor(slots, dtype=torch.int32)
        b["steps"].copy_(h_steps)
        b["slot"].copy_(h_slot)
        for li, j in self.lin_ids.items():
            K.gdn_commit(self.state[j], b["record"][j], b["slot"], b["steps"], nv=c.linear_num_value_heads,
                         dk=c.linear_key_head_dim, dv=c.linear_value_head_dim)

    def verify(self, tokens: list[int], pos0: int, slot: int, block_table: torch.Tensor, rope_delta: int = 0) -> torch.Tensor:
        """One sequence: logits ``[C, vocab]`` of ``C`` (2, 4 or 8) consecutive tokens
        (``models/qwen35/model.py:1761-1911`` in the reference)."""
        return self.verify_batch([(tokens, pos0, slot, block_table, rope_delta)])[0]

    def verify_hidden(self) -> torch.Tensor:
        """Last-layer residual stream ``[rows * C, H]`` (before the final norm) of the token rows of the
        last verify pass - what the MTP head pairs with the following token."""
        R, C, _ = self._verify_shape
        return self._verify_buffers(R, C)["final_res"]

    def commit(self, slot: int, n_accept: int) -> None:
        """Apply the first ``n_accept`` recorded delta-net updates of the last one-sequence ``verify``."""
        self.commit_batch([slot], [n_accept])

    # ------------------------------------------------------------------ runner hooks
    def poll_status(self) -> None:
        """Queue the read-back of the device status words behind the kernels launched so far."""
        K.poll_status()

    def check_status(self) -> None:
        """After a synchronisation that followed ``poll_status``: raise if a bounded device-side wait
        ran out during the step (a stalled peer, a stuck pipeline), so that wrong tokens never leave."""
        K.raise_on_status()

    def embed_tokens(self, tokens: torch.Tensor) -> torch.Tensor:
        return K.embed_gather(self.embed, tokens)

    def mrope_rows(self, positions3: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """Per-token rotary rows ``[T, rot]`` for 3-axis (t, h, w) positions ``[3, T]``."""
        c = self.cfg
        cos, sin = O.mrope_cos_sin(positions3.cpu(), c.rotary_dim, c.rope_theta, c.mrope_section)
        return cos.to(self.device), sin.to(self.device)

    def sample(self, logits: torch.Tensor, temps, us) -> torch.Tensor:
        """Greedy (``temps`` None) or per-row temperature sampling with host uniforms ``us``."""
        if temps is None:
            return K.argmax(logits.contiguous())
        t = torch.tensor(temps, dtype=torch.float32, device=self.device)
        u = torch.tensor(us, dtype=torch.float32, device=self.device)
        return K.sample(logits.contiguous(), t, u)

    @staticmethod
    def bucket_for(n: int) -> int:
        for m in BUCKETS:
            if n <= m:
                return m
        raise ValueError(f"{n} rows exceed the largest decode bucket {BUCKETS[-1]}")
