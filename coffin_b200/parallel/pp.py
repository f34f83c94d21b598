"""Pipeline parallelism: contiguous layer ranges, one stage per GPU, hidden states relayed with
NCCL point-to-point over NVLink.

Every rank runs the same engine loop (the control plane fans the requests out, as for tensor
parallelism), so scheduling, block tables and sampling are identical everywhere; what differs is
that a rank only owns the layers of its stage (and their delta-net state and KV pool).  A step is

    stage 0: embed -> layers[lo0:hi0] -> send hidden
    stage s: recv hidden -> layers[lo:hi] -> send hidden
    last   : recv hidden -> layers -> final norm -> lm_head -> argmax;  broadcast tokens + logits

Overlap comes from two places.  Prefill is chunked, and a stage forwards chunk ``c`` the moment it
is computed (the send is asynchronous on the stream), so stage ``s`` works on chunk ``c`` while
stage ``s-1`` already runs chunk ``c+1``.  Decode splits the batch rows into micro-batch *lanes*
(each with its own buffers and CUDA graph), so that stage ``s`` runs lane 1 while stage ``s+1``
runs lane 0.  The reference relays hidden states through UDP/shared memory with strictly serial
stages and lets every rank recompute the logits (``models/qwen35/parallel.py:220-236`` layer
ranges, ``:849-884`` which tensors a stage keeps, ``models/qwen35/model.py:515-560`` the relay).
"""
from __future__ import annotations

import dataclasses
import re

import torch

from ..config import ModelConfig
from ..weights.init import LM


def layer_range(n_layers: int, stage: int, n_stages: int) -> tuple[int, int]:
    """Contiguous ``[lo, hi)`` of stage ``stage``; the first ``n_layers % n_stages`` stages hold one more."""
    if not 0 <= stage < n_stages:
        raise ValueError(f"stage {stage} outside 0..{n_stages - 1}")
    if n_stages > n_layers:
        raise ValueError(f"{n_stages} pipeline stages for {n_layers} layers")
    base, extra = divmod(n_layers, n_stages)
    lo = stage * base + min(stage, extra)
    return lo, lo + base + (1 if stage < extra else 0)


def stage_config(cfg: ModelConfig, lo: int, hi: int) -> ModelConfig:
    """Geometry of the layers ``[lo, hi)`` as a model of its own."""
    return dataclasses.replace(cfg, num_hidden_layers=hi - lo, layer_types=tuple(cfg.layer_types[lo:hi]),
                               name=f"{cfg.name}-pp{lo}-{hi}")


_LAYER = re.compile(re.escape(LM) + r"layers\.(\d+)\.(.*)")


def stage_state_dict(sd: dict[str, torch.Tensor], lo: int, hi: int, first: bool, last: bool) -> dict[str, torch.Tensor]:
    """The tensors a stage keeps, with its layers renumbered from 0.  The embedding stays on the
    first stage, and on the last one when the head is tied to it; the final norm and ``lm_head``
    stay on the last stage."""
    out: dict[str, torch.Tensor] = {}
    tied = "lm_head.weight" not in sd
    for key, t in sd.items():
        m = _LAYER.match(key)
        if m:
            i = int(m.group(1))
            if lo <= i < hi:
                out[f"{LM}layers.{i - lo}.{m.group(2)}"] = t
        elif key == LM + "embed_tokens.weight":
            if first or (last and tied):
                out[key] = t
        elif key == "lm_head.weight":
            if last:
                out[key] = t
        elif key == LM + "norm.weight":
            out[key] = t                                   # a few KB; the stage constructor reads it
        elif not key.startswith("mtp."):
            out[key] = t
    return out


def split_lanes(n_rows: int, n_lanes: int) -> list[tuple[int, int]]:
    """Row ranges of the decode micro-batches: at most ``n_lanes`` non-empty, sizes within one."""
    n_lanes = max(1, min(n_lanes, n_rows))
    base, extra = divmod(n_rows, n_lanes)
    out, lo = [], 0
    for i in range(n_lanes):
        hi = lo + base + (1 if i < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out


class PipelineModel:
    """One pipeline stage behind the model interface the engine drives.

    ``stage`` is a model built from ``stage_config`` / ``stage_state_dict`` with ``pp_first`` /
    ``pp_last`` set.  ``group`` is the process group whose ranks are the stages in order (NCCL on
    GPUs; gloo for the CPU twin).  Results (next tokens and logits) are broadcast from the last
    stage, so every rank's engine samples and schedules identically.
    """

    def __init__(self, stage, rank: int, world: int, full_cfg: ModelConfig, group=None, lanes: int = 2) -> None:
        self.stage, self.rank, self.world, self.group = stage, rank, world, group
        self.cfg = full_cfg
        self.first, self.last = rank == 0, rank == world - 1
        self.lanes = max(1, lanes)
        self.device = stage.device
        self.max_seq, self.num_slots, self.max_chunk = stage.max_seq, stage.num_slots, stage.max_chunk
        self.max_blocks_per_seq, self.num_blocks = stage.max_blocks_per_seq, stage.num_blocks
        self._hid: dict = {}
        self._out: dict = {}
        self._plan: list[tuple[int, int, int]] = []     # (lane, rows, bucket)
        self.relay_bytes = 0
        self.dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32

    # ------------------------------------------------------------------ plumbing
    def _dist(self):
        import torch.distributed as dist
        return dist

    def _send(self, t: torch.Tensor) -> None:
        self.relay_bytes += t.numel() * t.element_size()
        self._dist().send(t.contiguous(), dst=self._global(self.rank + 1), group=self.group)

    def _recv(self, t: torch.Tensor) -> None:
        self._dist().recv(t, src=self._global(self.rank - 1), group=self.group)

    def _global(self, r: int) -> int:
        dist = self._dist()
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    def _bcast(self, t: torch.Tensor) -> None:
        self._dist().broadcast(t, src=self._global(self.world - 1), group=self.group)

    def _buf(self, pool: dict, key, shape, dtype) -> torch.Tensor:
        t = pool.get(key)
        if t is None:
            t = pool[key] = torch.zeros(*shape, dtype=dtype, device=self.device)
        return t

    # ------------------------------------------------------------------ delegated state hooks
    def zero_state(self, slot: int) -> None:
        self.stage.zero_state(slot)

    def snapshot_state(self, slot: int):
        return self.stage.snapshot_state(slot)

    def restore_state(self, slot: int, snap) -> None:
        self.stage.restore_state(slot, snap)

    def copy_block(self, src: int, dst: int) -> None:
        self.stage.copy_block(src, dst)

    def bucket_for(self, n: int) -> int:
        return self.stage.bucket_for(n)

    def mrope_rows(self, positions3):
        return self.stage.mrope_rows(positions3)

    def sample(self, logits, temps, us):
        return self.stage.sample(logits, temps, us)

    def embed_tokens(self, tokens: torch.Tensor) -> torch.Tensor:
        """Token embeddings on every rank (image rows are scattered into them by the runner): the
        first stage owns the table and broadcasts the rows."""
        H = self.cfg.hidden_size
        out = torch.empty(tokens.numel(), H, dtype=self.dtype, device=self.device)
        if self.first:
            out.copy_(self.stage.embed_tokens(tokens))
        self._dist().broadcast(out, src=self._global(0), group=self.group)
        return out

    def weight_bytes(self) -> int:
        return self.stage.weight_bytes() if hasattr(self.stage, "weight_bytes") else 0

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor, pos0: int, slot: int, block_table: torch.Tensor, embeds=None,
                cos_sin=None, want_logits: bool = True, want_hidden: bool = False):
        """One chunk through this stage.  Only the call that wants logits ends in a broadcast, so
        consecutive chunks flow through the stages without a rendezvous."""
        T = int(tokens.numel())
        H = self.cfg.hidden_size
        if not self.first:
            embeds = self._buf(self._hid, ("pf", T), (T, H), self.dtype)
            self._recv(embeds)
        out = self.stage.prefill(tokens, pos0, slot, block_table, embeds=embeds, cos_sin=cos_sin,
                                 want_logits=want_logits and self.last, want_hidden=want_hidden and self.last)
        if not self.last:
            self._send(self.stage.last_prenorm[:T])
        if not want_logits:
            return None
        logits = self._buf(self._out, "pf_logits", (self.cfg.vocab_size,), torch.float32)
        if self.last:
            logits.copy_(out)
        self._bcast(logits)
        return logits

    # ------------------------------------------------------------------ decode
    def set_rows(self, M: int, tokens, positions, slots, block_tables, rope_deltas=None) -> None:
        """Stage the rows, split over micro-batch lanes."""
        n = len(tokens)
        self._plan = []
        self._M = M
        for lane, (lo, hi) in enumerate(split_lanes(n, self.lanes)):
            m = self.stage.bucket_for(hi - lo)
            self.stage.lane = lane
            self.stage.set_rows(m, tokens[lo:hi], positions[lo:hi], slots[lo:hi], block_tables[lo:hi],
                                rope_deltas[lo:hi] if rope_deltas else None)
            self._plan.append((lane, hi - lo, m))
        self.stage.lane = 0

    @torch.no_grad()
    def decode(self, M: int, graph: bool = True):
        """One decode step of the staged rows: lanes run back to back on this stage, each received
        from the previous stage and forwarded as soon as it is done."""
        st, H, V = self.stage, self.cfg.hidden_size, self.cfg.vocab_size
        nxt = self._buf(self._out, ("next", M), (M,), torch.int64)
        logits = self._buf(self._out, ("logits", M), (M, V), torch.float32)
        row = 0
        for lane, n, m in self._plan:
            st.lane = lane
            if not self.first:
                hid = self._buf(self._hid, ("dec", lane, m), (m, H), self.dtype)
                self._recv(hid)
                st.input_hidden = hid
            t, lg = st.decode(m, graph=graph)
            st.input_hidden = None
            if not self.last:
                self._send(st.stage_hidden(m))
            else:
                nxt[row:row + n].copy_(t[:n])
                logits[row:row + n].copy_(lg[:n])
            row += n
        st.lane = 0
        self._bcast(nxt)
        self._bcast(logits)
        return nxt, logits

    def advance_rows(self, M: int) -> None:
        """Feed the broadcast tokens back into the lanes and advance their positions."""
        nxt = self._out[("next", M)]
        row = 0
        for lane, n, m in self._plan:
            self.stage.lane = lane
            b = self.stage._row_buffers(m)
            b["next"][:n].copy_(nxt[row:row + n])
            self.stage.advance_rows(m)
            row += n
        self.stage.lane = 0

    def verify(self, *a, **k):
        raise NotImplementedError("speculative verification is not available under pipeline parallelism")

    commit = verify


def build_stage(cfg: ModelConfig, sd: dict[str, torch.Tensor], rank: int, world: int, group=None,
                lanes: int = 2, factory=None, **kw) -> PipelineModel:
    """Cut ``sd`` for stage ``rank`` of ``world`` and wrap the stage model."""
    lo, hi = layer_range(cfg.num_hidden_layers, rank, world)
    first, last = rank == 0, rank == world - 1
    scfg = stage_config(cfg, lo, hi)
    ssd = stage_state_dict(sd, lo, hi, first, last)
    if factory is None:
        from ..models.qwen35.model import Qwen35Model as factory
    stage = factory(scfg, ssd, pp_first=first, pp_last=last, **kw)
    return PipelineModel(stage, rank, world, cfg, group=group, lanes=lanes)
