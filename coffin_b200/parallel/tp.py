"""Tensor parallelism: weight sharding and the peer-memory communicator behind the fused
GEMV + all-reduce kernels.

Sharding follows the usual column/row split: the fused input projections, gate/up and the lm_head
are split by output rows (heads, intermediate channels, vocabulary), ``o_proj`` / ``out_proj`` /
``down_proj`` by input columns, so each layer needs two all-reduces of the hidden vector.  During
decode those all-reduces are not calls: the row-parallel projection pushes its partial sums into
every rank's inbox and a one-CTA kernel per row (or the consumer phase of the persistent decode
kernel) adds them (``_C/tp.cuh``).  In prefill the tcgen05 GEMM epilogue leaves its partial
rows in this rank's peer-visible buffer and a reduce/gather kernel on every rank pulls the rows it owns from all
ranks, adds them and stores the sums to every rank.  KV heads are replicated when there are fewer of them
than ranks (reference ``local_config``, ``models/qwen35/parallel.py:670-718``; sharding by key
suffix ``:734-846``; ``RowParallelProjection`` ``:1015-1061``).
"""
from __future__ import annotations

import ctypes
import dataclasses
import os

import torch

from ..config import ModelConfig
from ..weights.init import LM

MAX_WORLD = 8
OS_ROWS = 64          # rows of a one-shot all-reduce (a decode bucket); kOsRows of _C/comm.cu


# ---------------------------------------------------------------------------------------------
# sharding
def local_config(cfg: ModelConfig, world: int) -> ModelConfig:
    """Per-rank geometry. Raises when a dimension does not divide."""
    def div(n: int, what: str) -> int:
        if n % world:
            raise ValueError(f"{what}={n} is not divisible by tensor-parallel world {world}")
        return n // world
    nkv = cfg.num_key_value_heads
    if nkv >= world:
        nkv_local = div(nkv, "num_key_value_heads")
    else:
        if world % nkv:
            raise ValueError(f"world {world} must be a multiple of num_key_value_heads {nkv}")
        nkv_local = 1
    return dataclasses.replace(
        cfg, num_attention_heads=div(cfg.num_attention_heads, "num_attention_heads"),
        num_key_value_heads=nkv_local,
        linear_num_key_heads=div(cfg.linear_num_key_heads, "linear_num_key_heads"),
        linear_num_value_heads=div(cfg.linear_num_value_heads, "linear_num_value_heads"),
        intermediate_size=div(cfg.intermediate_size, "intermediate_size") if cfg.intermediate_size else 0,
        name=f"{cfg.name}-tp{world}")


TP_MARK = "__tp_shard__"      # key a state dict carries when its tensors are already one rank's slices


def _span(n: int, rank: int, world: int, unit: int = 1) -> tuple[int, int]:
    per = (n // unit) // world
    return rank * per * unit, (rank + 1) * per * unit


def slice_plan(cfg: ModelConfig, key: str, rank: int, world: int):
    """How rank ``rank`` of ``world`` cuts the tensor stored under ``key``: ``None`` (whole tensor),
    ``("rows", [(a, b), ...])`` = concatenation of output-row ranges, or ``("cols", [(a, b)])`` = a range
    of input columns.  One description serves dense tensors, int8 / int4 containers and sliced reads
    from a safetensors file, so a rank never has to hold (or read) more than its part."""
    if not key.startswith(LM + "layers."):
        return None
    nk, nv, dk, dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
    kdim = nk * dk
    nh, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    name = key.split(".", 4)[-1]            # e.g. linear_attn.in_proj_qkv.weight
    if name in ("linear_attn.in_proj_qkv.weight", "linear_attn.conv1d.weight"):
        q0, q1 = _span(kdim, rank, world, dk)
        v0, v1 = _span(nv * dv, rank, world, dv)
        return "rows", [(q0, q1), (kdim + q0, kdim + q1), (2 * kdim + v0, 2 * kdim + v1)]
    if name == "linear_attn.in_proj_z.weight":
        return "rows", [_span(nv * dv, rank, world, dv)]
    if name in ("linear_attn.in_proj_b.weight", "linear_attn.in_proj_a.weight", "linear_attn.A_log", "linear_attn.dt_bias"):
        return "rows", [_span(nv, rank, world)]
    if name == "linear_attn.out_proj.weight":
        return "cols", [_span(nv * dv, rank, world, dv)]
    if name == "self_attn.q_proj.weight":
        return "rows", [_span(nh * 2 * hd, rank, world, 2 * hd)]
    if name in ("self_attn.k_proj.weight", "self_attn.v_proj.weight"):
        if nkv >= world:
            return "rows", [_span(nkv * hd, rank, world, hd)]
        h = rank * nkv // world          # the kv head this rank's query heads attend with
        return "rows", [(h * hd, (h + 1) * hd)]
    if name == "self_attn.o_proj.weight":
        return "cols", [_span(nh * hd, rank, world, hd)]
    if name in ("mlp.gate_proj.weight", "mlp.up_proj.weight"):
        return "rows", [_span(cfg.intermediate_size, rank, world)]
    if name == "mlp.down_proj.weight":
        return "cols", [_span(cfg.intermediate_size, rank, world)]
    return None


def apply_plan(t, plan):
    """Cut a dense tensor, a ``QWeight`` or a ``W4A8Weight`` according to ``slice_plan``."""
    from ..weights.quant import QWeight, W4A8Weight
    if plan is None:
        return t
    kind, ranges = plan
    if isinstance(t, QWeight):                      # wq [N, K] + scale [N]: a column cut keeps the row scales
        if kind == "rows":
            return QWeight(torch.cat([t.wq[a:b] for a, b in ranges]).contiguous(), torch.cat([t.scale[a:b] for a, b in ranges]))
        (a, b), = ranges
        return QWeight(t.wq[:, a:b].contiguous(), t.scale)
    if isinstance(t, W4A8Weight):                   # packed [K/2, N] + scale [K/group, N]
        if kind == "rows":
            return W4A8Weight(torch.cat([t.packed[..., a:b] for a, b in ranges], -1).contiguous(),
                              torch.cat([t.scale[..., a:b] for a, b in ranges], -1).contiguous(), t.k, t.group_size)
        (a, b), = ranges
        if a % t.group_size or b % t.group_size:
            raise ValueError(f"int4 column cut [{a}, {b}) is not aligned to the group size {t.group_size}")
        return W4A8Weight(t.packed[..., a // 2:b // 2, :].contiguous(),
                          t.scale[..., a // t.group_size:b // t.group_size, :].contiguous(), b - a, t.group_size)
    if kind == "rows":
        return t[ranges[0][0]:ranges[0][1]] if len(ranges) == 1 else torch.cat([t[a:b] for a, b in ranges])
    (a, b), = ranges
    return t[:, a:b].contiguous()


def shard_state_dict(cfg: ModelConfig, sd: dict, rank: int, world: int) -> dict:
    """The slice of a full state dict that rank ``rank`` of ``world`` computes with (dense tensors and
    quantised containers alike).  Tensors that every rank needs whole (norms, embedding, router) are
    shared, not copied.  A dict that was read rank-sliced from disk (``weights.loader.load_checkpoint``
    with ``tp=(rank, world)``) carries a mark and is returned as it is."""
    mark = sd.get(TP_MARK)
    if mark is not None:
        if tuple(mark) != (rank, world):
            raise ValueError(f"state dict holds the slices of rank {mark}, not of {(rank, world)}")
        return {k: v for k, v in sd.items() if k != TP_MARK}
    lc = local_config(cfg, world)
    out = {key: apply_plan(t, slice_plan(cfg, key, rank, world)) for key, t in sd.items()}
    assert lc.hidden_size == cfg.hidden_size
    return out


# ---------------------------------------------------------------------------------------------
# communicator
class _TpPfStruct(ctypes.Structure):
    """Mirror of ``TpPfDev`` (``_C/tp.cuh``): descriptor of the prefill reduce-scatter / all-gather."""
    _fields_ = [("rank", ctypes.c_int), ("world", ctypes.c_int), ("rows_per_rank", ctypes.c_int),
                ("width", ctypes.c_int),
                ("inbox", ctypes.c_void_p * MAX_WORLD), ("out", ctypes.c_void_p * MAX_WORLD),
                ("flags1", ctypes.c_void_p * MAX_WORLD), ("flags2", ctypes.c_void_p * MAX_WORLD),
                ("arrive", ctypes.c_void_p), ("status", ctypes.c_void_p), ("wait_ns", ctypes.c_uint64),
                ("seq_dev", ctypes.c_void_p), ("os_inbox", ctypes.c_void_p * MAX_WORLD)]


class _DevView:
    """Lets torch wrap a raw device pointer (``__cuda_array_interface__``) without copying."""

    def __init__(self, ptr: int, nelem: int) -> None:
        self.__cuda_array_interface__ = {"shape": (nelem,), "typestr": "<i2", "data": (ptr, False), "version": 2}


class _TpCommStruct(ctypes.Structure):
    _fields_ = [("rank", ctypes.c_int), ("world", ctypes.c_int), ("slot_floats", ctypes.c_int64),
                ("inbox", ctypes.c_void_p * MAX_WORLD), ("flags", ctypes.c_void_p * MAX_WORLD),
                ("my_inbox", ctypes.c_void_p), ("my_flags", ctypes.c_void_p),
                ("arrive", ctypes.c_void_p), ("epoch", ctypes.c_void_p), ("status", ctypes.c_void_p),
                ("wait_ns", ctypes.c_uint64)]


class TpComm:
    """Peer-mapped inbox/flag buffers of one tensor-parallel group on one node.

    One device allocation per rank holds ``[sites][world][max_rows * hidden]`` fp32 inbox slots,
    ``[sites][world]`` flags, ``[sites]`` producer arrival counters, the step epoch and a status
    word.  ``exchange`` is a callable that all-gathers a bytes object over the control plane (CPU
    process group); with ``world == 1`` nothing is exchanged, which is how the push/pull path is
    tested on a single GPU.
    """

    def __init__(self, rank: int, world: int, hidden: int, max_rows: int, n_sites: int, exchange=None,
                 prefill_rows: int = 0, loopback: bool = False) -> None:
        """``prefill_rows`` > 0 adds the buffers of the prefill all-reduce (chunks of up to that many
        rows): per rank an inbox of ``world`` partial slices and a result buffer, both bf16.
        ``loopback``: every peer pointer is this rank's own buffer (no IPC, one GPU).  The slots of the
        other ranks are then never written, which is how a test makes a bounded wait run out."""
        from ..ops import _lib
        if world > MAX_WORLD:
            raise ValueError(f"tensor-parallel world {world} > {MAX_WORLD}")
        self.rank, self.world, self.n_sites = rank, world, n_sites
        self.slot_floats = max_rows * hidden
        inbox_b = n_sites * world * self.slot_floats * 8        # {fp32 value, epoch} pairs
        flags_b = n_sites * world * 4
        self._off_flags = (inbox_b + 255) // 256 * 256
        self._off_arrive = self._off_flags + (flags_b + 255) // 256 * 256
        self._off_epoch = self._off_arrive + (n_sites * 4 + 255) // 256 * 256
        self._off_status = self._off_epoch + 256
        self.nbytes = self._off_status + 256
        self.hidden = hidden
        self.pf_rows = 0
        if prefill_rows > 0:
            self.pf_rpr = (prefill_rows + world - 1) // world
            self.pf_rows = self.pf_rpr * world
            slab = (self.pf_rows * hidden * 2 + 255) // 256 * 256
            self._off_pf_inbox = self.nbytes
            self._off_pf_out = self._off_pf_inbox + slab
            self._off_pf_f1 = self._off_pf_out + slab
            self._off_pf_f2 = self._off_pf_f1 + 256
            self._off_pf_arrive = self._off_pf_f2 + 256
            self._off_pf_seq = self._off_pf_arrive + 128        # same 256-byte cell as the arrival counters
            self._off_pf_desc = self._off_pf_arrive + 256
            self._off_os = self._off_pf_desc + 1024
            self.nbytes = self._off_os + (2 * world * OS_ROWS * hidden * 4 + 255) // 256 * 256   # {2 x bf16, seq} pairs
        self._pf_seq = 0
        self._lib = _lib.lib()
        base = ctypes.c_void_p()
        rc = self._lib.cb_peer_alloc(ctypes.c_int64(self.nbytes), ctypes.byref(base))
        if rc:
            raise _lib.KernelError(f"cb_peer_alloc failed ({rc})")
        self.base = base.value
        self.peers = [None] * world
        self.peers[rank] = self.base
        self._opened: list[int] = []
        if world > 1 and loopback:
            self.peers = [self.base] * world
        elif world > 1:
            handle = ctypes.create_string_buffer(64)
            rc = self._lib.cb_ipc_get_handle(ctypes.c_void_p(self.base), handle)
            if rc:
                raise _lib.KernelError(f"cudaIpcGetMemHandle failed ({rc})")
            handles = exchange(bytes(handle.raw))
            for r, h in enumerate(handles):
                if r == rank:
                    continue
                p = ctypes.c_void_p()
                rc = self._lib.cb_ipc_open_handle(ctypes.create_string_buffer(h, 64), ctypes.byref(p))
                if rc:
                    raise _lib.KernelError(f"cudaIpcOpenMemHandle of rank {r} failed ({rc})")
                self.peers[r] = p.value
                self._opened.append(p.value)
        s = _TpCommStruct()
        s.rank, s.world, s.slot_floats = rank, world, self.slot_floats
        for r in range(world):
            s.inbox[r] = self.peers[r]
            s.flags[r] = self.peers[r] + self._off_flags
        # limit of a device-side wait; COFFIN_TP_WAIT_MS shortens it (tests make a wait run out on purpose)
        self.wait_ns = int(float(os.environ.get("COFFIN_TP_WAIT_MS", "2000")) * 1e6)
        s.wait_ns = self.wait_ns
        s.my_inbox, s.my_flags = self.peers[rank], self.peers[rank] + self._off_flags
        s.arrive = self.base + self._off_arrive
        s.epoch = self.base + self._off_epoch
        s.status = self.base + self._off_status
        self._struct = s
        # the serving path watches the status word (ops.kernels.poll_status / raise_on_status)
        from ..ops import kernels as K
        sv = torch.as_tensor(_DevView(self.base + self._off_status, 2), device="cuda").view(torch.int32)
        self._status_view = sv
        self._watch_label = f"tp rank {rank} @{self.base:#x}"
        K.watch_status(sv[:1], self._watch_label)
        if self.pf_rows:
            d = _TpPfStruct()
            d.rank, d.world, d.rows_per_rank, d.width = rank, world, self.pf_rpr, hidden
            for r in range(world):
                d.inbox[r] = self.peers[r] + self._off_pf_inbox
                d.out[r] = self.peers[r] + self._off_pf_out
                d.flags1[r] = self.peers[r] + self._off_pf_f1
                d.flags2[r] = self.peers[r] + self._off_pf_f2
            d.arrive = self.base + self._off_pf_arrive
            d.status = self.base + self._off_status
            d.wait_ns = self.wait_ns
            d.seq_dev = self.base + self._off_pf_seq
            for r in range(world):
                d.os_inbox[r] = self.peers[r] + self._off_os
            assert ctypes.sizeof(d) == self._lib.cb_tp_pf_desc_size() <= 1024
            rc = self._lib.cb_peer_write(ctypes.c_void_p(self.base + self._off_pf_desc), ctypes.byref(d),
                                         ctypes.c_int64(ctypes.sizeof(d)))
            if rc:
                raise _lib.KernelError(f"descriptor upload failed ({rc})")
            self._pf_struct = d
            view = torch.as_tensor(_DevView(self.base + self._off_pf_out, self.pf_rows * hidden), device="cuda")
            self.pf_out = view.view(torch.bfloat16).view(self.pf_rows, hidden)

    # ---- prefill all-reduce (reduce-scatter in the producer, all-gather here) ------------------
    def pf_desc_ptr(self):
        return ctypes.c_void_p(self.base + self._off_pf_desc)

    def next_seq(self, rows: int, width: int) -> int:
        """Validates the next all-reduce (every rank makes the same calls in the same order) and returns
        the sequence argument of its kernels: 0 = "take the number from device memory", which the
        kernels advance themselves, so that a captured CUDA graph can be replayed."""
        if not self.pf_rows or rows > self.pf_rows or width != self.hidden:
            raise ValueError(f"prefill all-reduce of [{rows}, {width}] outside the region [{self.pf_rows}, {self.hidden}]")
        self._pf_T = rows
        return 0

    def scatter(self, src: torch.Tensor) -> None:
        """First half for a producer that is not a GEMM: copy the rows of ``src [T, hidden]`` (bf16) into this
        rank's peer-visible buffer and tell every rank that they are there (the owners pull them)."""
        from ..ops import kernels as K
        T = src.shape[0]
        K.call("tp_pf_scatter", self.pf_desc_ptr(), src, src.stride(0), T, self.next_seq(T, src.shape[1]))
        K._count()

    def finish_reduce(self, residual: torch.Tensor | None = None) -> torch.Tensor:
        """Second half: pull the partial rows this rank owns from every rank (coalesced peer loads), add them
        (+ ``residual`` rows), send the sums to every rank and wait for everyone's.  Returns the reduced ``[T, hidden]`` rows (a view of the
        result buffer, valid until the next all-reduce)."""
        from ..ops import kernels as K
        T, seq = self._pf_T, 0
        K.call("tp_pf_reduce_gather", self.pf_desc_ptr(), residual, residual.stride(0) if residual is not None else 0, T, seq,
               self.world)
        K.call("tp_pf_wait", self.pf_desc_ptr(), seq)
        K._count(2)
        return self.pf_out[:T]

    def oneshot(self, src: torch.Tensor, residual: torch.Tensor | None = None, gain: torch.Tensor | None = None,
                res_out: torch.Tensor | None = None, normed: torch.Tensor | None = None, eps: float = 0.0,
                quant: tuple | None = None) -> None:
        """All-reduce of the few rows of a decode bucket (``src [M <= 64, hidden]`` bf16) in one launch and
        one NVLink crossing: CTA m of every rank stores row m into every peer's one-shot inbox (data paired
        with the sequence number), polls the peers' rows in its own inbox, adds the world's rows (rank order)
        + ``residual`` into ``res_out`` and, with ``gain``, writes ``rmsnorm(res_out) * gain`` into ``normed``
        and / or its per-row int8 quantisation into ``quant = (q, scale)`` (for an int8 projection next)."""
        from ..ops import kernels as K
        M, W = src.shape
        if not self.pf_rows or M > OS_ROWS or W != self.hidden:
            raise ValueError(f"one-shot all-reduce of [{M}, {W}] outside [{OS_ROWS}, {self.hidden}]")
        K.call("tp_os_allreduce", self.pf_desc_ptr(), src, src.stride(0), residual,
               residual.stride(0) if residual is not None else 0, gain,
               res_out, res_out.stride(0) if res_out is not None else 0, normed,
               normed.stride(0) if normed is not None else 0, M, W, float(eps), 0,
               quant[0] if quant is not None else None, quant[1] if quant is not None else None)
        K._count()

    def cstruct_ref(self):
        return ctypes.byref(self._struct)

    def epoch_bump(self) -> None:
        from ..ops import kernels as K
        K.call("tp_epoch_bump", ctypes.c_void_p(self.base + self._off_epoch))
        K._count()

    def status(self) -> int:
        """Non-zero when a device-side wait ran out (16 + the rank that never arrived)."""
        v = ctypes.c_int(0)
        self._lib.cb_peer_read_i32(ctypes.c_void_p(self.base + self._off_status), ctypes.byref(v))
        return int(v.value)

    def clear_status(self) -> None:
        self._status_view.zero_()

    def close(self) -> None:
        from ..ops import kernels as K
        K.unwatch_status(self._watch_label)
        for p in self._opened:
            self._lib.cb_ipc_close_handle(ctypes.c_void_p(p))
        self._opened = []
        if self.base:
            self._lib.cb_peer_free(ctypes.c_void_p(self.base))
            self.base = 0


def make_exchange(group=None):
    """All-gather of a bytes object over ``torch.distributed`` (any backend with object
    collectives; the control plane uses gloo)."""
    import torch.distributed as dist

    def exchange(blob: bytes) -> list[bytes]:
        out = [None] * dist.get_world_size(group)
        dist.all_gather_object(out, blob, group=group)
        return out
    return exchange
