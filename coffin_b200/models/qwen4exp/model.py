"""Qwen4-exp on one B200: hyper-connected residual lanes, delta-net and block-sparse (QSA)
attention mixers, a routed MoE in every layer, optional n-gram (PLE) injection.

Execution model (prefill eager; the decode step replays as a CUDA graph per row count when the model has no
n-gram layer and no rotary-row cache - the family's reference runs everything eagerly,
``models/qwen4exp/engine.py:12-24``):

* The residual stream is ``[rows, hc * H]`` bf16.  A mixer's output is not written back when it is
  produced: the next hyper-connection read applies ``stream += out (x) inject`` inside its norm
  kernel (``hyper_norm``), so a layer touches the wide stream twice, not four times.
* Hyper-connection read: ``hyper_norm`` -> low-rank down GEMV -> ``hyper_up`` (read gate, lane mix,
  write gates) for up to 8 rows; prefill chunks run the same algebra on tcgen05 GEMMs.
* Delta-net layers reuse the Qwen3.5 kernels (fused decode step, chunked prefill scan); the MoE is
  the Qwen3.5 module (router kernel, grouped tensor-core GEMVs / per-expert GEMMs, combine).
* QSA layers keep three paged pools per layer - K, V and the raw index keys - plus a pool of
  *block keys*: the key of a block of ``ratio`` tokens never changes once the block is complete, so
  it is computed once (``qsa_block_keys``) instead of for every query as in the reference
  (``models/qwen4exp/qsa.py:496-528, 800-860``).  Decode scores the cached block keys, selects by
  an exact radix top-k and runs split-KV attention over the kept tokens only; prefill passes a
  per-query block mask to the flash kernel.
* PLE (one layer in the real model) runs as torch ops on the device; its table lives in HBM when it
  fits and in pinned host memory with an asynchronous gather otherwise (``ngram.NGramTable``).

The class offers the model interface the engine drives (``prefill`` / ``set_rows`` / ``decode`` /
state snapshots / ``copy_block``), so the block manager, radix cache and scheduler are shared with
the Qwen3.5 family.  Speculative decoding: ``verify_batch`` / ``commit_batch`` (what the engine's drafter
path drives) and the family's own draft head (``mtp_run``, ``spec_generate``).
Structure reference: ``models/qwen4exp/blocks.py:52-238``, ``model.py:250-470``, ``engine.py:360-897``.
"""
from __future__ import annotations

import math

import torch

from ...ops import kernels as K
from ...oracle import ops as O
from ..qwen35.model import QW, QW4
from ..qwen35.moe import MoEWeights
from .config import INDEXED, LINEAR, Qwen4Config
from .ngram import NGramHasher, NGramTable, ShardedNGramTable

LM = "model.language_model."
BUCKETS = (1, 2, 4, 8)
GRAPH_DECODE = __import__("os").environ.get("COFFIN_QWEN4_GRAPH", "1") != "0"   # decode steps as CUDA graphs where the model allows


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


class _Hyper:
    """Weights of one hyper-connection."""

    def __init__(self, sd, prefix: str, dev, write_gate: bool = True) -> None:
        bf = torch.bfloat16
        self.gain = (1.0 + sd[prefix + "hc_norm.weight"].float()).to(dev).contiguous()
        self.Wd = sd[prefix + "input_mix_weight_down.weight"].to(dev, bf).contiguous()      # [R, hc*H]
        self.Wu = sd[prefix + "input_mix_weight_up.weight"].to(dev, bf).contiguous()        # [hc*H, R]
        self.Wi = self.Wi8 = None
        if write_gate:
            wi = sd[prefix + "block_inject_weight.weight"].to(dev, bf)
            self.Wi = wi.contiguous()                                                       # [hc, hc*H]
            self.Wi8 = torch.zeros(_pad8(max(wi.shape[0], 8)), wi.shape[1], dtype=bf, device=dev)
            self.Wi8[:wi.shape[0]] = wi                                                     # GEMM needs >= 8 output rows

    def tensors(self):
        return [t for t in (self.Wd, self.Wu, self.Wi) if t is not None]


class _Layer:
    pass


class QuantEmbedding:
    """Embedding table stored as int8 rows + one fp32 scale per row (a quarter of the bf16 table once
    the scales are counted): gathered rows are dequantised to bf16 on the device.  Reference:
    ``models/qwen4exp/proj.py:724-841`` (``QuantizedEmbedding``)."""

    def __init__(self, wq: torch.Tensor, scale: torch.Tensor) -> None:
        self.wq, self.scale = wq.contiguous(), scale.float().contiguous()
        self.shape = self.wq.shape

    def gather(self, tokens: torch.Tensor) -> torch.Tensor:
        rows = self.wq.index_select(0, tokens)
        return (rows.float() * self.scale.index_select(0, tokens)[:, None]).to(torch.bfloat16)

    def dequant(self) -> torch.Tensor:
        return (self.wq.float() * self.scale[:, None]).to(torch.bfloat16)

    def numel(self) -> int:
        return self.wq.numel()

    def element_size(self) -> int:
        return 1

    def data_ptr(self) -> int:
        return self.wq.data_ptr()


class Qwen4ExpModel:
    def __init__(self, cfg: Qwen4Config, sd: dict[str, torch.Tensor], device: str | torch.device = "cuda",
                 max_seq: int = 4096, num_slots: int = 2, num_blocks: int | None = None, max_chunk: int = 2048,
                 pdl: bool = True, ngram_device_budget: int = 120 << 30, quant: str = "none", tp=None,
                 ep_rank: int = 0, ep_world: int = 1, with_mtp: bool = False, mrope_cache: bool = False,
                 **_unused) -> None:
        """``quant``: ``int8`` / ``w4a8`` storage of the mixer projections, the experts and the head (a
        pre-quantised state dict brings its own containers).  ``ep_world`` > 1: the routed experts are split
        by range over the ranks of the communicator ``tp``; everything else is replicated."""
        self.cfg = c = cfg
        self.quant = quant
        self.tp, self.ep_rank, self.ep_world = tp, ep_rank, ep_world
        self.tp_world, self.tp_rank, self.tp_force = 1, 0, False
        if 64 % c.indexer_compress_ratio or c.indexer_compress_ratio < 2:
            raise ValueError("indexer_compress_ratio must be a power of two between 2 and 64")
        if c.indexer_n_heads > 8 or c.indexer_head_dim > 256:
            raise ValueError("indexer geometry outside the kernels' range (heads <= 8, head_dim <= 256)")
        self.device = dev = torch.device(device)
        self.max_seq, self.num_slots, self.max_chunk = int(max_seq), int(num_slots), int(max_chunk)
        self.max_blocks_per_seq = (self.max_seq + K.BLOCK - 1) // K.BLOCK
        self.num_blocks = int(num_blocks) if num_blocks else self.max_blocks_per_seq * self.num_slots + 1
        self.eps = c.rms_norm_eps
        self.gate_sigmoid = c.output_gate_type == "sigmoid"
        K.status_word(dev)
        K._lib.set_pdl(pdl)
        bf = torch.bfloat16

        from ...weights.quant import QWeight, W4A8Weight

        def w(key):
            """A projection in the storage the checkpoint (or ``quant``) gives it: bf16, int8 rows with
            per-row scales, or int4 codes with group scales (``Proj`` of the reference, ``proj.py:524-722``)."""
            t = sd[key]
            if isinstance(t, QWeight):
                return QW(t.wq.to(dev), t.scale.to(dev))
            if isinstance(t, W4A8Weight):
                if t.k % t.group_size == 0 and t.group_size == 128:
                    return QW4(*t.to(dev).to_nk())
                t = t.dequant(bf)
            return t.to(dev, bf)

        def dense(key):
            t = sd[key]
            return (t.dequant(bf) if isinstance(t, (QWeight, W4A8Weight)) else t).to(dev, bf)

        def quantise(t):
            """Apply ``quant`` to a dense projection (containers pass through)."""
            if isinstance(t, (QW, QW4)):
                return t
            if quant == "w4a8" and t.shape[1] % 128 == 0:
                return QW4.quantize(t)
            return QW.quantize(t) if quant == "int8" else t.contiguous()

        def cat(parts):
            """Row-concatenate projections that share an input; quantised parts keep their scales."""
            if any(isinstance(p_, QW4) for p_ in parts) or quant == "w4a8":
                conv = [p_ if isinstance(p_, QW4) else (QW4.zeros(p_.shape[0], p_.shape[1], dev) if not bool(p_.any())
                                                         else QW4.quantize(p_)) for p_ in parts]
                return QW4(torch.cat([p_.wq for p_ in conv]), torch.cat([p_.scale for p_ in conv]))
            if any(isinstance(p_, QW) for p_ in parts) or quant == "int8":
                conv = [p_ if isinstance(p_, QW) else QW.quantize(p_) for p_ in parts]
                return QW(torch.cat([p_.wq for p_ in conv]), torch.cat([p_.scale for p_ in conv]))
            return torch.cat(parts).contiguous()

        def gain(key):
            return (1.0 + sd[key].float()).to(dev).contiguous()

        e = sd[LM + "embed_tokens.weight"]
        if isinstance(e, QWeight):
            self.embed = QuantEmbedding(e.wq.to(dev), e.scale.to(dev))
        else:
            self.embed = dense(LM + "embed_tokens.weight").contiguous()
        if "lm_head.weight" in sd:
            self.lm_head = quantise(w("lm_head.weight"))
        else:
            self.lm_head = quantise(self.embed.dequant() if isinstance(self.embed, QuantEmbedding) else self.embed)
        self.final = _Hyper(sd, LM + "hyper_connection_mixer.", dev, write_gate=False)
        self.layers: list[_Layer] = []
        self.lin_ids = {li: j for j, li in enumerate(c.linear_layers)}
        self.full_ids = {li: j for j, li in enumerate(c.full_layers)}
        self.ple_ids: dict[int, int] = {}
        def make_layer(p: str, kind: str, ple_j):
            L = _Layer()
            L.kind = kind
            L.h_attn = _Hyper(sd, p + "attn_hyper_connection.", dev)
            L.h_mlp = _Hyper(sd, p + "mlp_hyper_connection.", dev)
            if kind == LINEAR:
                q = p + "linear_attn."
                parts = [w(q + "in_proj_qkv.weight"), w(q + "in_proj_z.weight"), w(q + "in_proj_b.weight"),
                         w(q + "in_proj_a.weight")]
                n = sum(t.shape[0] for t in parts)
                if _pad8(n) != n:
                    parts.append(torch.zeros(_pad8(n) - n, c.hidden_size, dtype=bf, device=dev))
                L.w_in = cat(parts)
                L.w_out = quantise(w(q + "out_proj.weight"))
                L.conv_w = sd[q + "conv1d.weight"].to(dev, torch.float32).reshape(c.lin_conv_dim, -1).contiguous()
                L.A_log = sd[q + "A_log"].to(dev, torch.float32).contiguous()
                L.dt_bias = sd[q + "dt_bias"].to(dev, torch.float32).contiguous()
                L.norm_w = sd[q + "norm.weight"].to(dev, torch.float32).contiguous()
            else:
                q = p + "self_attn."
                parts = [w(q + "q_proj.weight"), w(q + "k_proj.weight"), w(q + "v_proj.weight"),
                         w(q + "indexer.index_qk_proj.weight")]
                n = sum(t.shape[0] for t in parts)
                L.idx_col = n - parts[3].shape[0]
                if _pad8(n) != n:
                    parts.append(torch.zeros(_pad8(n) - n, c.hidden_size, dtype=bf, device=dev))
                L.w_in = cat(parts)
                L.w_out = quantise(w(q + "o_proj.weight"))
                L.qg, L.kg = gain(q + "q_norm.weight"), gain(q + "k_norm.weight")
                L.iqg, L.ikg = gain(q + "indexer.q_layernorm.weight"), gain(q + "indexer.k_layernorm.weight")
            L.moe = MoEWeights.from_state_dict(c, sd, p + "mlp.", dev, ep_rank, ep_world, quant=quant)
            L.ple = None
            j = ple_j
            if j is not None:
                q = p + "ple."
                P = _Layer()
                P.hasher = NGramHasher(c, j)
                tw = sd[q + "ple_embedding.ngram_embedding.weight"]
                if isinstance(tw, list):                # the checkpoint's row shards as mapped host views
                    P.table = ShardedNGramTable(list(tw), dev, ngram_device_budget, keep=getattr(tw, "keep", None))
                else:
                    P.table = NGramTable(tw.to(bf), dev, ngram_device_budget)
                P.key_w = w(q + "key_proj.weight").float()
                P.val_w = w(q + "value_proj.weight").float()
                P.g_key, P.g_query, P.g_conv = gain(q + "norm_key.weight"), gain(q + "norm_query.weight"), gain(q + "norm_conv.weight")
                P.conv_w = sd[q + "conv1d.weight"].to(dev, torch.float32).reshape(c.hc_hidden, -1).contiguous()
                L.ple = P
            return L

        for li, kind in enumerate(c.layer_types):
            L = make_layer(f"{LM}layers.{li}.", kind, c.ple_index(li))
            if L.ple is not None:
                self.ple_ids[li] = len(self.ple_ids)
            self.layers.append(L)
        # ---- draft head (MTP): one QSA + MoE layer of its own, two [H, H] projections, a final mixer
        self.mtp = None
        if with_mtp:
            if not c.mtp_num_hidden_layers or "mtp.fc_embedding.weight" not in sd:
                raise ValueError("with_mtp needs a checkpoint that carries the draft head (mtp_num_hidden_layers = 1)")
            D = _Layer()
            D.layer = make_layer("mtp.layers.0.", INDEXED, None)
            D.fc_e, D.fc_h = quantise(w("mtp.fc_embedding.weight")), quantise(w("mtp.fc_hidden.weight"))
            D.g_e, D.g_h = gain("mtp.pre_fc_norm_embedding.weight"), gain("mtp.pre_fc_norm_hidden.weight")
            D.final = _Hyper(sd, "mtp.hyper_connection_mixer.", dev, write_gate=False)
            self.mtp = D
        cos, sin = O.rope_tables(c.rotary_dim, c.rope_theta, self.max_seq + 64)
        self.cos, self.sin = cos.to(dev).contiguous(), sin.to(dev).contiguous()
        # Multimodal sequences rotate with 3-axis positions (image tokens) and a position offset after the
        # image, so "the rotary row of position p" is a property of the sequence, not of p.  Query, key and
        # index-query rows get it when they are computed; the key of a BLOCK is rotated with the row of the
        # block's first token when the block completes, possibly in a later pass - that row is looked up in
        # a per-slot cache of the rows every position was rotated with.  Text-only models skip the cache.
        self.rc_cos = self.rc_sin = None
        if mrope_cache:
            self.rc_cos = torch.zeros(self.num_slots, self.max_seq + 64, c.rotary_dim, dtype=torch.float32, device=dev)
            self.rc_sin = torch.zeros_like(self.rc_cos)
        self.vision = None
        # ---- sequence state --------------------------------------------------------------------
        nl, nf, npl = len(self.lin_ids), len(self.full_ids), len(self.ple_ids)
        self.state = torch.zeros(nl, self.num_slots, c.linear_num_value_heads, c.linear_key_head_dim,
                                 c.linear_value_head_dim, dtype=torch.float32, device=dev)
        self.ring = torch.zeros(nl, self.num_slots, K.RING, c.lin_conv_dim, dtype=bf, device=dev)
        rows = self.num_blocks * K.BLOCK
        npool = nf + (1 if self.mtp is not None else 0)       # the draft head pages its own K / V / index keys (last pool)
        self.mtp_pool = nf
        self.kpool = torch.zeros(npool, rows, c.num_key_value_heads, c.head_dim, dtype=bf, device=dev)
        self.vpool = torch.zeros_like(self.kpool)
        self.ipool = torch.zeros(npool, rows, c.indexer_head_dim, dtype=bf, device=dev)
        self.per_page = K.BLOCK // c.indexer_compress_ratio
        self.bkpool = torch.zeros(npool, self.num_blocks * self.per_page, c.indexer_head_dim, dtype=torch.float32, device=dev)
        self.ple_hist = torch.zeros(max(npl, 1), self.num_slots, c.ple_conv_state_len, c.hc_hidden, dtype=torch.float32, device=dev)
        self.ple_ctx: list[list[list[int]]] = [[self._fresh_ctx() for _ in range(self.num_slots)] for _ in range(max(npl, 1))]
        self.max_sel_blocks = (self.max_seq + c.indexer_compress_ratio - 1) // c.indexer_compress_ratio
        self._ws: dict = {}
        self._rows: dict = {}
        self._staged: dict | None = None
        self._rowbuf: dict = {}
        self._graphs: dict = {}
        self.graph_pool = None
        self.last_prenorm = None
        self.last_hidden = None
        self.last_lanes = None
        self._verify: dict | None = None
        self.layer_hook = None            # debugging: called as hook(layer index, residual lanes) before every layer

    # ------------------------------------------------------------------ sizes / bookkeeping
    def _fresh_ctx(self) -> list[int]:
        return [self.cfg.eos_token_id] * self.cfg.ple_context_len

    def poll_status(self) -> None:
        K.poll_status()

    def check_status(self) -> None:
        K.raise_on_status()

    def weight_bytes(self) -> int:
        tensors = [self.embed, self.lm_head] + self.final.tensors()
        for L in self.layers:
            tensors += [L.w_in, L.w_out] + L.h_attn.tensors() + L.h_mlp.tensors() + L.moe.tensors()
        seen, total = set(), 0
        for t in tensors:
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    def launches_per_step(self, M: int) -> int:
        return 0

    @staticmethod
    def bucket_for(n: int) -> int:
        for m in BUCKETS:
            if n <= m:
                return m
        raise ValueError(f"{n} rows exceed the largest decode bucket {BUCKETS[-1]}")

    # ------------------------------------------------------------------ sequence state hooks
    def zero_state(self, slot: int) -> None:
        self.state[:, slot].zero_()
        self.ring[:, slot].zero_()
        self.ple_hist[:, slot].zero_()
        for ctx in self.ple_ctx:
            ctx[slot] = self._fresh_ctx()

    def snapshot_state(self, slot: int):
        return (self.state[:, slot].clone(), self.ring[:, slot].clone(), self.ple_hist[:, slot].clone(),
                [list(ctx[slot]) for ctx in self.ple_ctx])

    def restore_state(self, slot: int, snap) -> None:
        self.state[:, slot].copy_(snap[0])
        self.ring[:, slot].copy_(snap[1])
        self.ple_hist[:, slot].copy_(snap[2])
        for ctx, saved in zip(self.ple_ctx, snap[3]):
            ctx[slot] = list(saved)

    def copy_block(self, src: int, dst: int) -> None:
        """Copy one page of every paged pool (K, V, raw index keys, block keys)."""
        s, d = src * K.BLOCK, dst * K.BLOCK
        for pool in (self.kpool, self.vpool, self.ipool):
            pool[:, d:d + K.BLOCK].copy_(pool[:, s:s + K.BLOCK])
        pp = self.per_page
        self.bkpool[:, dst * pp:(dst + 1) * pp].copy_(self.bkpool[:, src * pp:(src + 1) * pp])

    def embed_tokens(self, tokens: torch.Tensor) -> torch.Tensor:
        return K.embed_gather(self.embed, tokens)

    def sample(self, logits: torch.Tensor, temps, us) -> torch.Tensor:
        if temps is None:
            return K.argmax(logits.contiguous())
        t = torch.tensor(temps, dtype=torch.float32, device=self.device)
        u = torch.tensor(us, dtype=torch.float32, device=self.device)
        return K.sample(logits.contiguous(), t, u)

    # ------------------------------------------------------------------ workspaces
    def _work(self, T: int, tag: str = "") -> dict:
        """Buffers for a pass over ``T`` rows (kept per size; a prefill chunk and a decode bucket
        never share them; ``tag`` separates the draft head's buffers from the main model's)."""
        key = (T, tag)
        ws = self._ws.get(key)
        if ws is None:
            c, dev, bf = self.cfg, self.device, torch.bfloat16
            H, W = c.hidden_size, c.hc_hidden
            in_w = max(L.w_in.shape[0] for L in self.layers)
            mix_w = max(c.lin_vdim, c.num_attention_heads * c.head_dim)
            nsplit = K.decode_splits(c.num_key_value_heads, T) if T <= 8 else 1
            ws = {
                "stream": torch.empty(T, W, dtype=bf, device=dev),
                "normed": torch.empty(T, W, dtype=bf, device=dev),
                "low": torch.empty(T, c.hc_lowrank, dtype=torch.float32, device=dev),
                "mixed": torch.empty(T, H, dtype=bf, device=dev),
                "inject": [torch.empty(T, c.hc_count, dtype=torch.float32, device=dev) for _ in range(2)],
                "proj": torch.empty(T, in_w, dtype=bf, device=dev),
                "act": torch.empty(T, mix_w, dtype=bf, device=dev),
                "out": [torch.empty(T, H, dtype=bf, device=dev) for _ in range(2)],
                "q": torch.empty(T, c.num_attention_heads, c.head_dim, dtype=bf, device=dev),
                "iq": torch.empty(T, c.indexer_n_heads, c.indexer_head_dim, dtype=torch.float32, device=dev),
                "kv_slot": torch.empty(T, dtype=torch.int32, device=dev),
                "pos": torch.empty(T, dtype=torch.int32, device=dev),
                "scores": torch.empty(T, self.max_sel_blocks, dtype=torch.float32, device=dev),
                "sel": torch.zeros(T, c.block_topk, dtype=torch.int32, device=dev),
                "nsel": torch.zeros(T, dtype=torch.int32, device=dev),
                "mask": torch.zeros(T, (self.max_sel_blocks + 31) // 32, dtype=torch.int32, device=dev),
                "nsplit": nsplit,
            }
            if T <= 8:
                ws["part_o"] = torch.zeros(T, c.num_attention_heads, nsplit, c.head_dim, dtype=torch.float32, device=dev)
                ws["part_ml"] = torch.zeros(T, c.num_attention_heads, nsplit, 2, dtype=torch.float32, device=dev)
                ws["tickets"] = torch.zeros(T, c.num_key_value_heads, dtype=torch.int32, device=dev)
            if self.lin_ids and T > 8:
                n = K.gdn_prefill_scratch_floats(T, c.linear_num_key_heads, c.linear_num_value_heads,
                                                 c.linear_key_head_dim, c.linear_value_head_dim)
                ws["gdn"] = torch.empty(n, dtype=torch.float32, device=dev)
            if T <= 8 and self.lin_ids and not tag:
                # verify pass: per-token rank-one updates of every delta-net layer, n-gram conv windows
                ws["record"] = torch.zeros(len(self.lin_ids), 1, T, c.linear_num_value_heads,
                                           c.linear_key_head_dim + c.linear_value_head_dim + 1, dtype=torch.float32, device=dev)
                ws["one_slot"] = torch.zeros(1, dtype=torch.int32, device=dev)
                ws["one_pos"] = torch.zeros(1, dtype=torch.int32, device=dev)
                ws["steps"] = torch.zeros(1, dtype=torch.int32, device=dev)
            ws["ones"] = torch.ones(T, c.hc_count, dtype=torch.float32, device=dev)
            if T > 8:                   # keep at most two chunk-sized workspaces per tag
                big = [k for k in self._ws if k[0] > 8 and k[1] == tag]
                for k in big[:-1]:
                    del self._ws[k]
            self._ws[key] = ws
        return ws

    def _linear(self, W, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """``out = x @ W^T`` on whichever storage ``W`` has: up to 8 rows through the decode projections
        (bf16 tensor-core GEMV, int8 W8A8, int4 W4A8), more through the tcgen05 GEMM (bf16, int8
        ``kind::i8``, int4 expanded to bf16 for the call)."""
        T, Kd = x.shape
        small = T <= 8 and T * Kd * 2 <= 64 * 1024
        if isinstance(W, QW):
            if small:
                return K.gemv_i8(W.wq, W.scale, x, out)
            qx, sc = K.quant_rows(x)
            if out.dtype == torch.bfloat16:
                return K.gemm_i8(qx, sc, W.wq, W.scale, out=out)
            out.copy_(K.gemm_i8(qx, sc, W.wq, W.scale))
            return out
        if isinstance(W, QW4):
            if small:
                return K.gemv_w4(W.wq, W.scale, x, out)
            W = W.expanded()
        if small:
            return K.gemv(W, x, out)
        if out.dtype == torch.bfloat16:
            return K.gemm(x, W, out=out)
        out.copy_(K.gemm(x, W))
        return out

    def _embed(self, tokens: torch.Tensor) -> torch.Tensor:
        if isinstance(self.embed, QuantEmbedding):
            return self.embed.gather(tokens)
        return K.embed_gather(self.embed, tokens)

    def mrope_rows(self, positions3: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """Per-token rotary rows ``[T, rot]`` for 3-axis (t, h, w) positions ``[3, T]``."""
        c = self.cfg
        if not c.mrope_section:
            raise ValueError("this checkpoint has no multi-axis rotary sections")
        cos, sin = O.mrope_cos_sin(positions3.cpu(), c.rotary_dim, c.rope_theta, c.mrope_section)
        return cos.to(self.device), sin.to(self.device)

    def _set_rope(self, ws: dict, *, rows=None, ridx=None, slots=None, positions=None) -> None:
        """Rotary rows of the pass staged in ``ws``: explicit per-row tables ``rows = (cos, sin)`` or the
        1-D table indexed by ``ridx`` (int32, on the device).  With the row cache, the rows are also
        recorded at (``slots[r]``, ``positions[r]``) (host lists; padding rows have slot < 0)."""
        if rows is not None:
            cos, sin = rows[0].float().contiguous(), rows[1].float().contiguous()
            ws["rope"] = (cos, sin, None)
        else:
            ws["rope"] = (self.cos, self.sin, ridx)
        if self.rc_cos is not None:
            keep = [r for r, s_ in enumerate(slots) if s_ >= 0]
            if keep:
                sl = torch.tensor([slots[r] for r in keep], dtype=torch.int64, device=self.device)
                ps = torch.tensor([positions[r] for r in keep], dtype=torch.int64, device=self.device)
                kr = torch.tensor(keep, dtype=torch.int64, device=self.device)
                if rows is not None:
                    rc, rs = ws["rope"][0][kr], ws["rope"][1][kr]
                else:
                    ix = ridx.to(torch.int64)[kr]
                    rc, rs = self.cos[ix], self.sin[ix]
                self.rc_cos[sl, ps] = rc
                self.rc_sin[sl, ps] = rs
                K._count(2)

    def _tp_reduce(self, t: torch.Tensor) -> torch.Tensor:
        """Sum of the ranks' routed-expert outputs ``[T, hidden]`` (expert parallel): scatter + reduce/gather
        over peer memory when the communicator has the region, NCCL otherwise (the reference combines
        through a shared-memory board, ``models/qwen4exp/parallel.py:245-565``)."""
        if self.ep_world == 1:
            return t
        if self.tp is not None and self.tp.pf_rows and t.shape[0] <= self.tp.pf_rows:
            from ...parallel.tp import OS_ROWS
            t = t.contiguous()
            if t.shape[0] <= OS_ROWS:
                out = torch.empty_like(t)
                self.tp.oneshot(t, res_out=out)
                return out
            self.tp.scatter(t)
            return self.tp.finish_reduce()
        import torch.distributed as dist
        dist.all_reduce(t)
        K._count()
        return t

    # ------------------------------------------------------------------ hyper-connection
    def _hyper_read(self, hw: _Hyper, ws: dict, T: int, pending, inject_buf: torch.Tensor | None):
        """Apply the pending write-back, norm the lanes and return ``(mixed [T, H], inject | None)``."""
        c = self.cfg
        H, hc = c.hidden_size, c.hc_count
        stream, normed = ws["stream"], ws["normed"]
        bo, inj = pending if pending is not None else (None, None)
        K.hyper_norm(stream, hw.gain, normed, H=H, hc=hc, eps=self.eps, block_out=bo, inject=inj)
        if T <= 8:
            self._linear(hw.Wd, normed, ws["low"])
            K.hyper_up(normed, ws["low"], hw.Wu, hw.Wi, ws["mixed"], inject_buf if hw.Wi is not None else None, H=H, hc=hc)
            return ws["mixed"], (inject_buf if hw.Wi is not None else None)
        low = K.gemm(normed, hw.Wd)
        act = torch.nn.functional.silu(low.float() / hc).to(torch.bfloat16)
        gate = torch.sigmoid(K.gemm(act, hw.Wu).float())
        torch.mul(gate, normed.float(), out=gate)
        ws["mixed"].copy_(gate.view(T, hc, H).mean(1))
        K._count(4)
        inject = None
        if hw.Wi8 is not None:
            inject_buf.copy_(2.0 * torch.sigmoid(K.gemm(normed, hw.Wi8)[:, :hc].float() / hc))
            inject = inject_buf
            K._count(1)
        return ws["mixed"], inject

    # ------------------------------------------------------------------ PLE
    def _ple(self, L, j: int, stream: torch.Tensor, tokens: list[int], slot: int, record: dict | None = None) -> torch.Tensor:
        """n-gram injection for consecutive tokens of one sequence: returns the fp32 term ``[T, hc*H]``
        to add to the stream and advances the slot's n-gram context and conv history.  With ``record``
        (a verify pass) the slot is left untouched and the window + context are kept so that ``commit``
        can advance by the accepted prefix."""
        c, P = self.cfg, L.ple
        hc, H = c.hc_count, c.hidden_size
        ctx = self.ple_ctx[j][slot]
        ids = P.hasher.ids(tokens, ctx)
        emb = P.table.gather(ids).float()                                   # [T, E]
        T = emb.shape[0]

        def gnorm(x, g):
            xf = x.reshape(T, hc, H)
            return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).reshape(T, hc * H) * g

        key = gnorm(emb @ P.key_w.t(), P.g_key)
        val = emb @ P.val_w.t()
        qry = gnorm(stream.float(), P.g_query)
        g = (key.view(T, hc, H) * qry.view(T, hc, H)).sum(-1, keepdim=True) / math.sqrt(H)
        g = g.abs().clamp_min(1e-6).sqrt() * g.sign()
        gv = (torch.sigmoid(g) * val[:, None, :]).reshape(T, hc * H)
        gvn = gnorm(gv, P.g_conv)
        hist = self.ple_hist[j, slot]
        seq = torch.cat([hist, gvn], 0)
        k, dil, span = c.ple_conv_kernel_size, c.ple_conv_dilation, c.ple_conv_state_len
        conv = torch.zeros_like(gvn)
        for tap in range(k):
            conv += seq[tap * dil:tap * dil + T] * P.conv_w[:, tap]
        if record is not None:
            record[j] = (seq, list(ctx), [int(t) for t in tokens])
        else:
            hist.copy_(seq[seq.shape[0] - span:])
            self.ple_ctx[j][slot] = (ctx + [int(t) for t in tokens])[-c.ple_context_len:]
        K._count(12)
        return gv + torch.nn.functional.silu(conv)

    # ------------------------------------------------------------------ mixers
    def _gdn(self, L, li: int, ws: dict, T: int, mixed, out, *, slot=None, pos0=None, slots=None, positions=None,
             verify: bool = False):
        """``verify``: the ``T`` rows are consecutive tokens of one sequence scored without touching its
        state - the per-token updates are recorded for ``commit``."""
        c = self.cfg
        j = self.lin_ids[li]
        proj = ws["proj"][:, :L.w_in.shape[0]]
        self._linear(L.w_in, mixed, proj)
        act = ws["act"][:, :c.lin_vdim]
        kw = dict(nk=c.linear_num_key_heads, nv=c.linear_num_value_heads, dk=c.linear_key_head_dim,
                  dv=c.linear_value_head_dim, eps=self.eps, gate_sigmoid=self.gate_sigmoid)
        if verify:
            K.gdn_decode(proj, L.conv_w, L.A_log, L.dt_bias, L.norm_w, self.ring[j], self.state[j], ws["one_slot"],
                         ws["one_pos"], act, ntok=T, record=ws["record"][j], write_state=False, **kw)
        elif slots is not None:
            K.gdn_decode(proj, L.conv_w, L.A_log, L.dt_bias, L.norm_w, self.ring[j], self.state[j], slots, positions, act, **kw)
        else:
            K.gdn_prefill(proj, L.conv_w, L.A_log, L.dt_bias, L.norm_w, self.ring[j, slot], self.state[j, slot],
                          ws["gdn"], act, pos0=pos0, **kw)
        self._linear(L.w_out, act, out)

    def _qsa(self, L, li: int, ws: dict, T: int, mixed, out, *, block_tables, positions_host: list[int],
             shared_table: bool, pool: int | None = None, keep_selection: bool = False, slots_host=None):
        """``positions_host[t]`` is the position of row ``t``; with ``shared_table`` all rows belong to
        one sequence (a prefill chunk) whose pages are ``block_tables`` (1-D).  ``pool``: which set of
        paged pools the layer owns (default: the layer's own; the draft head has the last one).
        ``keep_selection`` (decode rows): attend through the blocks selected by the previous call on
        this workspace instead of selecting again."""
        c = self.cfg
        j = self.full_ids[li] if pool is None else pool
        nh, nkv, hd, rot = c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.rotary_dim
        ni, di, ratio = c.indexer_n_heads, c.indexer_head_dim, c.indexer_compress_ratio
        proj = ws["proj"][:, :L.w_in.shape[0]]
        self._linear(L.w_in, mixed, proj)
        pos, kv_slot = ws["pos"], ws["kv_slot"]
        rcos, rsin, ridx = ws.get("rope") or (self.cos, self.sin, pos)
        K.attn_prep(proj, L.qg, L.kg, rcos, rsin, ridx, kv_slot, ws["q"], self.kpool[j], self.vpool[j],
                    nh=nh, nkv=nkv, hd=hd, rot=rot, eps=self.eps)
        K.qsa_index_prep(proj, L.idx_col, L.iqg, rcos, rsin, ridx, kv_slot, ws["iq"], self.ipool[j],
                         ni=ni, di=di, rot=rot, eps=self.eps)
        # rotary rows of block starts: the sequence's recorded rows when the model keeps them
        cached = self.rc_cos is not None and pool is None and slots_host is not None

        def start_rows(slot):
            return (self.rc_cos[slot], self.rc_sin[slot]) if cached and slot >= 0 else (self.cos, self.sin)
        # keys of the blocks that this pass completed
        if shared_table:
            b0, b1 = positions_host[0] // ratio, (positions_host[-1] + 1) // ratio
            bc, bs = start_rows(slots_host[0] if slots_host else -1)
            K.qsa_block_keys(self.ipool[j], self.bkpool[j], L.ikg, bc, bs, block_tables, b0, b1,
                             ratio=ratio, di=di, rot=rot, eps=self.eps)
        elif positions_host is None:
            # inside a CUDA graph: which rows complete a block is decided on the device
            K.qsa_block_keys_rows(self.ipool[j], self.bkpool[j], L.ikg, self.cos, self.sin, block_tables, pos,
                                  ratio=ratio, di=di, rot=rot, eps=self.eps)
        else:
            for r, p in enumerate(positions_host):
                if p >= 0 and (p + 1) % ratio == 0:
                    bc, bs = start_rows(slots_host[r] if slots_host else -1)
                    K.qsa_block_keys(self.ipool[j], self.bkpool[j], L.ikg, bc, bs, block_tables[r],
                                     p // ratio, p // ratio + 1, ratio=ratio, di=di, rot=rot, eps=self.eps)
        act = ws["act"][:, :nh * hd]
        if T <= 8 and not shared_table:
            if not keep_selection:
                K.qsa_select(ws["iq"], self.bkpool[j], block_tables, pos, ws["scores"], ws["sel"], ws["nsel"],
                             ni=ni, di=di, ratio=ratio, topk=c.block_topk, full_factor=c.full_select_factor)
            K.attn_sparse(ws["q"], proj, pos, block_tables, self.kpool[j], self.vpool[j], ws["sel"], ws["nsel"],
                          ws["part_o"], ws["part_ml"], ws["tickets"], act, nh=nh, nkv=nkv, hd=hd, ratio=ratio,
                          nsplit=ws["nsplit"])
        else:
            nb_last = (positions_host[-1] + 1) // ratio
            keep = None
            if nb_last > c.block_topk and nb_last > c.block_topk * c.full_select_factor:
                K.qsa_select(ws["iq"], self.bkpool[j], block_tables, pos, ws["scores"], ws["sel"], ws["nsel"],
                             ni=ni, di=di, ratio=ratio, topk=c.block_topk, full_factor=c.full_select_factor,
                             mask=ws["mask"], shared_table=True)
                keep = ws["mask"]
            K.attn_prefill(ws["q"], proj, self.kpool[j], self.vpool[j], block_tables, act, q_pos0=positions_host[0],
                           nh=nh, nkv=nkv, hd=hd, keep=keep, ratio=ratio)
        self._linear(L.w_out, act, out)

    # ------------------------------------------------------------------ layer stack
    def _run(self, ws: dict, T: int, *, tokens_host, slot=None, pos0=None, block_table=None, slots=None,
             positions=None, positions_host=None, block_tables=None, row_slots=None, verify: dict | None = None) -> torch.Tensor:
        """All layers over the ``T`` rows staged in ``ws['stream']``.  Prefill: one sequence
        (``slot``, ``pos0``, ``block_table``).  Decode: one token of each of ``T`` sequences
        (``slots`` / ``positions`` device tensors, ``block_tables [T, pages]``).  Returns the mixed
        final hidden state ``[T, H]``."""
        c = self.cfg
        decode = slots is not None
        pending = None
        for li, L in enumerate(self.layers):
            if self.layer_hook is not None:
                self.layer_hook(li, ws["stream"])
            if L.ple is not None:
                stream = ws["stream"]
                if pending is not None:                      # PLE reads the stream with the last write-back applied
                    stream.add_((pending[0].float()[:, None, :] * pending[1][:, :, None]).flatten(1).to(stream.dtype))
                    pending = None
                    K._count()
                j = self.ple_ids[li]
                if decode:
                    for r in range(T):
                        if row_slots[r] >= 0:
                            stream[r:r + 1].add_(self._ple(L, j, stream[r:r + 1], [tokens_host[r]], row_slots[r]).to(stream.dtype))
                else:
                    stream.add_(self._ple(L, j, stream, tokens_host, slot, record=verify).to(stream.dtype))
            inj_a, inj_b = ws["inject"]
            mixed, inject = self._hyper_read(L.h_attn, ws, T, pending, inj_a)
            out = ws["out"][0]
            if L.kind == LINEAR:
                if decode:
                    self._gdn(L, li, ws, T, mixed, out, slots=slots, positions=positions)
                else:
                    self._gdn(L, li, ws, T, mixed, out, slot=slot, pos0=pos0, verify=verify is not None)
            else:
                if decode:
                    self._qsa(L, li, ws, T, mixed, out, block_tables=block_tables, positions_host=positions_host,
                              shared_table=False, slots_host=row_slots)
                else:
                    self._qsa(L, li, ws, T, mixed, out, block_tables=block_table,
                              positions_host=list(range(pos0, pos0 + T)), shared_table=True, slots_host=[slot])
            mixed, inject2 = self._hyper_read(L.h_mlp, ws, T, (out, inject), inj_b)
            out2 = ws["out"][1]
            out2.copy_(L.moe.apply(mixed.contiguous(), self))
            pending = (out2, inject2)
        mixed, _ = self._hyper_read(self.final, ws, T, pending, None)
        return mixed                      # ws["stream"] now holds the un-collapsed lanes (last write-back applied)

    # ------------------------------------------------------------------ engine interface
    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor, pos0: int, slot: int, block_table: torch.Tensor, embeds=None,
                cos_sin=None, want_logits: bool = True, want_hidden: bool = False, want_lanes: bool = False):
        """One chunk of one sequence at positions ``pos0 .. pos0 + T - 1``; returns the fp32 logits of
        the last token (or ``None``).  ``want_lanes``: keep the un-collapsed lanes of every row in
        ``last_lanes`` (what the draft head pairs with the following token)."""
        if cos_sin is not None and self.rc_cos is None:
            raise ValueError("per-token rotary rows need the rotary-row cache (build the model with mrope_cache=True)")
        c = self.cfg
        T = int(tokens.numel())
        assert 0 < T <= self.max_chunk
        if T <= 8:                      # a short tail runs through the decode path (same kernels, fewer buffers)
            rows = [int(t) for t in tokens.tolist()]
            out = None
            kept = []
            for i, tok in enumerate(rows):
                self.set_rows(1, [tok], [pos0 + i], [slot], [block_table.tolist()])
                if cos_sin is not None:
                    self._staged["rope_rows"] = (cos_sin[0][i:i + 1], cos_sin[1][i:i + 1])
                if embeds is not None:
                    self._staged["embeds"] = embeds[i:i + 1]
                _, logits = self.decode(1, want_logits=want_logits and i == T - 1)
                out = logits[0] if logits is not None else None
                if want_lanes:
                    kept.append(self._work(1)["stream"].clone())
            self.last_lanes = torch.cat(kept) if want_lanes else None
            return out
        ws = self._work(T)
        e = self._embed(tokens) if embeds is None else embeds.to(torch.bfloat16)
        ws["stream"].copy_(e.repeat(1, c.hc_count))
        pos = torch.arange(pos0, pos0 + T, dtype=torch.int64, device=self.device)
        ws["pos"].copy_(pos)
        ws["kv_slot"].copy_(block_table.to(torch.int64)[pos // K.BLOCK] * K.BLOCK + pos % K.BLOCK)
        self._set_rope(ws, rows=cos_sin, ridx=ws["pos"], slots=[slot] * T, positions=list(range(pos0, pos0 + T)))
        mixed = self._run(ws, T, tokens_host=[int(t) for t in tokens.tolist()] if self.ple_ids else None,
                          slot=slot, pos0=pos0, block_table=block_table)
        self.last_hidden = mixed if want_hidden else None
        self.last_lanes = ws["stream"].clone() if want_lanes else None
        if not want_logits:
            return None
        logits = torch.empty(1, c.vocab_size, dtype=torch.float32, device=self.device)
        self._linear(self.lm_head, mixed[T - 1:T].contiguous(), logits)
        return logits[0]

    def set_rows(self, M: int, tokens, positions, slots, block_tables, rope_deltas=None) -> None:
        n = len(tokens)
        dev = self.device
        bt = torch.zeros(n, self.max_blocks_per_seq, dtype=torch.int32)
        for r, row in enumerate(block_tables):
            bt[r, :len(row)] = torch.as_tensor(row, dtype=torch.int32)
        deltas = [int(d) for d in rope_deltas] if rope_deltas else [0] * n
        if any(deltas) and self.rc_cos is None:
            raise ValueError("rotary position offsets need the rotary-row cache (build the model with mrope_cache=True)")
        # the device copies live in buffers that persist per row count, so that a captured step finds its inputs
        # at fixed addresses
        rb = self._rowbuf.get(n)
        if rb is None:
            rb = self._rowbuf[n] = {"bt": torch.zeros(n, self.max_blocks_per_seq, dtype=torch.int32, device=dev),
                                    "ridx": torch.zeros(n, dtype=torch.int32, device=dev),
                                    "tok": torch.zeros(n, dtype=torch.int64, device=dev),
                                    "pos": torch.zeros(n, dtype=torch.int32, device=dev),
                                    "slot": torch.zeros(n, dtype=torch.int32, device=dev)}
        rb["bt"].copy_(bt)
        rb["ridx"].copy_(torch.tensor([max(0, int(p) + d) for p, d in zip(positions, deltas)], dtype=torch.int32))
        rb["tok"].copy_(torch.tensor([int(t) for t in tokens], dtype=torch.int64))
        rb["pos"].copy_(torch.tensor([int(p) for p in positions], dtype=torch.int32))
        rb["slot"].copy_(torch.tensor([int(s) for s in slots], dtype=torch.int32))
        self._staged = dict(n=n, M=M, tokens=[int(t) for t in tokens], positions=[int(p) for p in positions],
                            slots=[int(s) for s in slots], bt=rb["bt"], deltas=deltas, ridx_dev=rb["ridx"],
                            tok_dev=rb["tok"], pos_dev=rb["pos"], slot_dev=rb["slot"])

    def graph_ok(self) -> bool:
        """Whether a decode step of this model can be captured: every decision of the step must be made on
        the device.  The n-gram injection hashes token ids on the host and the rotary-row cache is indexed
        with host lists, so models with either run the step eagerly."""
        return not self.ple_ids and self.rc_cos is None and self.device.type == "cuda"

    def _decode_body(self, n: int, M: int, want_logits: bool, host: bool):
        """The step over the ``n`` staged rows.  ``host=False``: nothing depends on host copies of the rows
        (block-key completion is decided by the kernel), which is what a CUDA graph needs."""
        c, st = self.cfg, self._staged
        ws = self._work(n)
        e = st["embeds"].to(torch.bfloat16) if st.get("embeds") is not None else self._embed(st["tok_dev"])
        ws["stream"].copy_(e.repeat(1, c.hc_count))
        ws["pos"].copy_(st["pos_dev"])
        p64 = st["pos_dev"].to(torch.int64)
        ws["kv_slot"].copy_(st["bt"].to(torch.int64).gather(1, (p64 // K.BLOCK)[:, None])[:, 0] * K.BLOCK + p64 % K.BLOCK)
        if host:
            self._set_rope(ws, rows=st.get("rope_rows"), ridx=st["ridx_dev"], slots=st["slots"], positions=st["positions"])
        else:
            ws["rope"] = (self.cos, self.sin, st["ridx_dev"])
        mixed = self._run(ws, n, tokens_host=st["tokens"] if host else None, slots=st["slot_dev"], positions=st["pos_dev"],
                          positions_host=st["positions"] if host else None, block_tables=st["bt"],
                          row_slots=st["slots"] if host else None)
        b = self._rows.get(M)
        if b is None:
            b = self._rows[M] = {"logits": torch.zeros(M, c.vocab_size, dtype=torch.float32, device=self.device),
                                 "next": torch.zeros(M, dtype=torch.int64, device=self.device)}
        if not want_logits:
            return b["next"], None
        self._linear(self.lm_head, mixed.contiguous(), b["logits"][:n])
        K.argmax(b["logits"], b["next"])
        return b["next"], b["logits"]

    @torch.no_grad()
    def decode(self, M: int, graph: bool = True, want_logits: bool = True):
        """One token for each staged row.  Returns ``(next_tokens [M], logits [M, vocab])``; rows beyond
        the staged ones are zero.  ``graph``: replay the step as a CUDA graph (captured per row count on
        first use) when the model allows it (``graph_ok``) - the reference runs this family eagerly only
        (``models/qwen4exp/engine.py:12-24``), which leaves a step bound by its ~50 launches per layer."""
        st = self._staged
        n = st["n"]
        if (not graph or not GRAPH_DECODE or not self.graph_ok() or not want_logits or st.get("embeds") is not None
                or st.get("rope_rows") is not None or any(st["deltas"])):
            return self._decode_body(n, M, want_logits, host=True)
        key = (n, M)
        g = self._graphs.get(key)
        if g is None:
            # warm-up runs on a side stream (workspaces, kernel attributes), then the capture; the staged rows
            # are real, so the warm-up steps are replays of the same step: state-changing kernels (delta-net
            # update, KV append) rewrite the same values, and the state is put back before the graph runs
            snaps = [self.snapshot_state(s_) for s_ in st["slots"]]
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._decode_body(n, M, True, host=False)
                    for s_, sn in zip(st["slots"], snaps):
                        self.restore_state(s_, sn)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            if self.graph_pool is None:
                self.graph_pool = torch.cuda.graph_pool_handle()
            with K.capture_graph(g, pool=self.graph_pool):
                self._decode_body(n, M, True, host=False)
            self._graphs[key] = g
            for s_, sn in zip(st["slots"], snaps):      # the capture itself does not run the kernels; states are as staged
                self.restore_state(s_, sn)
        g.replay()
        b = self._rows[M]
        return b["next"], b["logits"]

    def advance_rows(self, M: int) -> None:
        st = self._staged
        nxt = self._rows[M]["next"][:st["n"]].tolist()
        self.set_rows(M, nxt, [p + 1 for p in st["positions"]], st["slots"],
                      [row.tolist() for row in st["bt"].cpu()], st["deltas"])

    # ------------------------------------------------------------------ speculative decoding
    VERIFY_WIDTHS = (2, 4, 8)

    def _stage_rows(self, ws: dict, T: int, tokens, pos0: int, block_table: torch.Tensor, embeds=None) -> None:
        """Stage ``T`` consecutive rows of one sequence: embeddings into every lane, positions, KV slots."""
        c = self.cfg
        tok = torch.as_tensor(list(tokens), dtype=torch.int64).to(self.device) if not isinstance(tokens, torch.Tensor) else tokens
        e = self._embed(tok) if embeds is None else embeds
        ws["stream"].copy_(e.repeat(1, c.hc_count))
        pos = torch.arange(pos0, pos0 + T, dtype=torch.int64, device=self.device)
        ws["pos"].copy_(pos)
        ws["kv_slot"].copy_(block_table.to(torch.int64)[pos // K.BLOCK] * K.BLOCK + pos % K.BLOCK)

    @torch.no_grad()
    def verify_batch(self, rows: list[tuple]) -> torch.Tensor:
        """Score ``C`` (2..8) consecutive tokens - the last sampled token followed by drafts - of each
        row ``(tokens[C], pos0, slot, block_table, rope_delta)``; returns logits ``[n, C, vocab]``.
        K / V / index keys of all positions are written (rejected ones are overwritten later), the
        delta-net states and the n-gram windows are left untouched: the per-token updates are recorded
        and ``commit_batch`` applies each row's accepted prefix.  Each row is one pass (the rows of this
        family do not share a forward); the un-collapsed lanes of every scored position are kept for the
        draft head (``verify_lanes``)."""
        c = self.cfg
        C = len(rows[0][0])
        if not 2 <= C <= 8 or any(len(r[0]) != C for r in rows):
            raise ValueError("a verify pass scores 2..8 tokens, the same number for every row")
        out = torch.empty(len(rows), C, c.vocab_size, dtype=torch.float32, device=self.device)
        self._verify = {"C": C, "rows": []}
        for i, (tokens, pos0, slot, table, _delta) in enumerate(rows):
            if pos0 + C > self.max_seq:
                raise ValueError(f"positions {pos0}..{pos0 + C - 1} exceed max_seq {self.max_seq}")
            bt = table if isinstance(table, torch.Tensor) else torch.tensor(list(table), dtype=torch.int32, device=self.device)
            ws = self._work(C, tag=f"verify{i}" if i else "")
            if "record" not in ws:
                first = self._work(C)
                for k_ in ("record", "one_slot", "one_pos", "steps"):
                    ws[k_] = torch.zeros_like(first[k_])
            self._stage_rows(ws, C, tokens, pos0, bt)
            ridx = (ws["pos"] + int(_delta)).to(torch.int32) if _delta else ws["pos"]
            self._set_rope(ws, ridx=ridx, slots=[slot] * C, positions=list(range(pos0, pos0 + C)))
            ws["one_slot"].fill_(slot)
            ws["one_pos"].fill_(pos0)
            rec: dict = {}
            mixed = self._run(ws, C, tokens_host=[int(t) for t in tokens], slot=slot, pos0=pos0, block_table=bt, verify=rec)
            self._linear(self.lm_head, mixed.contiguous(), out[i])
            self._verify["rows"].append({"ws": ws, "ple": rec, "slot": slot})
        return out

    def commit_batch(self, slots: list[int], steps: list[int]) -> None:
        """Advance row ``i`` of the last ``verify_batch`` by its first ``steps[i]`` tokens."""
        c, v = self.cfg, self._verify
        assert v is not None and len(slots) == len(steps) == len(v["rows"])
        span = c.ple_conv_state_len
        for row, slot, n in zip(v["rows"], slots, steps):
            assert slot == row["slot"] and 0 <= n <= v["C"]
            ws = row["ws"]
            ws["steps"].fill_(n)
            for li, j in self.lin_ids.items():
                K.gdn_commit(self.state[j], ws["record"][j], ws["one_slot"], ws["steps"], nv=c.linear_num_value_heads,
                             dk=c.linear_key_head_dim, dv=c.linear_value_head_dim)
            for j, (seq, ctx, toks) in row["ple"].items():
                self.ple_hist[j, slot].copy_(seq[n:n + span])
                self.ple_ctx[j][slot] = (ctx + toks[:n])[-c.ple_context_len:]

    def verify(self, tokens: list[int], pos0: int, slot: int, block_table: torch.Tensor, rope_delta: int = 0) -> torch.Tensor:
        return self.verify_batch([(tokens, pos0, slot, block_table, rope_delta)])[0]

    def commit(self, slot: int, steps: int) -> None:
        self.commit_batch([slot], [steps])

    def verify_lanes(self, row: int = 0) -> torch.Tensor:
        """Un-collapsed lanes ``[C, hc*H]`` of the positions scored by row ``row`` of the last verify pass."""
        return self._verify["rows"][row]["ws"]["stream"]

    # ------------------------------------------------------------------ draft head (MTP)
    @torch.no_grad()
    def mtp_run(self, next_tokens, lanes: torch.Tensor, pos0: int, block_table: torch.Tensor, add_embedding: bool = True,
                keep_selection: bool = False):
        """The draft head over ``T`` rows at positions ``pos0 ..`` of one sequence: row ``t`` pairs the
        lanes of position ``pos0 + t`` (``lanes [T, hc*H]``: the main model's, or the head's own ``multi``
        on a chained draft step) with the token that follows that position, and predicts the one after.
        Returns ``(sample [T, H], multi [T, hc*H])`` - views of the head's workspace, valid until its next
        call with the same ``T``.  The head's K / V / index keys live in its own paged pools under the
        sequence's block table, so truncating or sharing the sequence's pages carries the head along.
        A single row runs the decode kernels (block selection + split-KV sparse attention; with
        ``keep_selection`` the previous call's blocks are reused, the reference's ``DraftIndexPlan``,
        ``models/qwen4exp/mtp.py:63-128``); more rows run the prefill kernels.  Reference: ``mtp.py:146-330``."""
        D, c = self.mtp, self.cfg
        if D is None:
            raise RuntimeError("this model was built without the draft head (with_mtp=True)")
        H, hc = c.hidden_size, c.hc_count
        T = lanes.shape[0]
        ws = self._work(T, tag="mtp")
        tok = torch.as_tensor(list(next_tokens), dtype=torch.int64).to(self.device) if not isinstance(next_tokens, torch.Tensor) else next_tokens
        pos = torch.arange(pos0, pos0 + T, dtype=torch.int64, device=self.device)
        ws["pos"].copy_(pos)
        ws["kv_slot"].copy_(block_table.to(torch.int64)[pos // K.BLOCK] * K.BLOCK + pos % K.BLOCK)
        if "bo" not in ws:
            ws["bo"] = torch.empty(T, H, dtype=torch.bfloat16, device=self.device)
            ws["en"] = torch.empty(T, H, dtype=torch.bfloat16, device=self.device)
        K.rmsnorm(self._embed(tok), D.g_e, self.eps, out=ws["en"])
        self._linear(D.fc_e, ws["en"], ws["bo"])
        K.rmsnorm(lanes.contiguous(), D.g_h, self.eps, out=ws["normed"])              # ONE norm over all hc*H channels
        self._linear(D.fc_h, ws["normed"].view(T * hc, H), ws["stream"].view(T * hc, H))
        pending = (ws["bo"], ws["ones"]) if add_embedding else None       # unit write gate: the embedding enters every lane
        L = D.layer
        inj_a, inj_b = ws["inject"]
        mixed, inject = self._hyper_read(L.h_attn, ws, T, pending, inj_a)
        out = ws["out"][0]
        single = T == 1
        self._qsa(L, -1, ws, T, mixed, out, block_tables=block_table[None] if single else block_table,
                  positions_host=list(range(pos0, pos0 + T)), shared_table=not single, pool=self.mtp_pool,
                  keep_selection=keep_selection and single)
        mixed, inject2 = self._hyper_read(L.h_mlp, ws, T, (out, inject), inj_b)
        out2 = ws["out"][1]
        out2.copy_(L.moe.apply(mixed.contiguous(), self))
        sample, _ = self._hyper_read(D.final, ws, T, (out2, inject2), None)
        return sample, ws["stream"]

    def head_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        out = torch.empty(hidden.shape[0], self.cfg.vocab_size, dtype=torch.float32, device=self.device)
        return self._linear(self.lm_head, hidden.contiguous(), out)

    @torch.no_grad()
    def spec_generate(self, prompt: list[int], max_new: int, k: int = 3, slot: int = 0, block_table: torch.Tensor | None = None,
                      index_reuse: bool = True, draft_hook=None):
        """Greedy speculative decoding of one request with the draft head: ``k`` chained drafts, one
        verify pass of ``k + 1`` tokens, the longest agreeing prefix is kept - token for token the result of
        plain greedy decoding.  Unlike the reference's validation path (``models/qwen4exp/model.py:681-818``,
        which recomputes the whole context with both models every round) everything is incremental: the
        head's pools follow the main model's pages, the head appends exactly the rows the verify pass
        accepted (its last appended row IS the first draft), rejected delta-net updates are never applied.
        ``draft_hook(position, drafts) -> drafts`` lets a caller replace the drafts (tests of the accept
        paths).  Returns ``(tokens, stats)``."""
        c = self.cfg
        if self.mtp is None:
            raise RuntimeError("spec_generate needs the draft head (with_mtp=True)")
        if not prompt or k < 1 or k > 7:
            raise ValueError("spec_generate needs a prompt and 1 <= k <= 7")
        n = len(prompt)
        if n + max_new + k + 1 > self.max_seq:
            raise ValueError("prompt + generation + drafts exceed max_seq")
        bt = block_table if block_table is not None else torch.arange(
            1 + slot * self.max_blocks_per_seq, 1 + (slot + 1) * self.max_blocks_per_seq, dtype=torch.int32, device=self.device)
        ratio = c.indexer_compress_ratio
        self.zero_state(slot)
        toks = torch.tensor(prompt, dtype=torch.int64, device=self.device)
        lanes = []
        logits = None
        for p0 in range(0, n, self.max_chunk):
            part = toks[p0:p0 + self.max_chunk]
            logits = self.prefill(part, p0, slot, bt, want_logits=p0 + part.numel() >= n, want_lanes=True)
            lanes.append(self.last_lanes)
        lanes = torch.cat(lanes)
        out = [int(logits.argmax())]
        stats = {"rounds": 0, "drafted": 0, "accepted": 0, "index_reuse": 0}
        done = 0                                   # positions appended to the head
        for p0 in range(0, n - 1, self.max_chunk):
            p1 = min(n - 1, p0 + self.max_chunk)
            self.mtp_run(toks[p0 + 1:p1 + 1], lanes[p0:p1], p0, bt)
            done = p1
        pend_lanes, pend_next = lanes[n - 1:n].clone(), [out[-1]]
        while len(out) < max_new:
            stats["rounds"] += 1
            T = len(pend_next)
            sample, multi = self.mtp_run(pend_next, pend_lanes, done, bt)
            done += T                              # == the main model's committed length
            drafts = [int(self.head_logits(sample[T - 1:T])[0].argmax())]
            multi = multi[T - 1:T].clone()
            sel_blocks = done // ratio             # complete blocks seen by the selection of the first chained step
            selected = False
            for step in range(1, k):
                pos = done + step - 1
                reuse = index_reuse and selected and (pos + 1) // ratio == sel_blocks
                sample, m2 = self.mtp_run(drafts[-1:], multi, pos, bt, add_embedding=False, keep_selection=reuse)
                if reuse:
                    stats["index_reuse"] += 1
                else:
                    selected, sel_blocks = True, (pos + 1) // ratio
                multi = m2.clone()
                drafts.append(int(self.head_logits(sample)[0].argmax()))
            if draft_hook is not None:
                drafts = list(draft_hook(n + len(out), drafts))[:k]
            stats["drafted"] += len(drafts)
            fed = [out[-1]] + drafts
            C = next(w for w in self.VERIFY_WIDTHS if len(fed) <= w)
            fed_p = fed + [fed[-1]] * (C - len(fed))
            picked = self.verify(fed_p, done, slot, bt).argmax(-1).tolist()
            a = 0
            while a < len(drafts) and picked[a] == drafts[a]:
                a += 1
            stats["accepted"] += a
            self.commit(slot, a + 1)
            new = drafts[:a] + [picked[a]]
            out.extend(new)
            pend_lanes, pend_next = self.verify_lanes()[:a + 1].clone(), new
        stats["acceptance"] = stats["accepted"] / max(stats["drafted"], 1)
        return out[:max_new], stats

