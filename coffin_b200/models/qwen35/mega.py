"""Host side of the persistent decode kernel (``_C/decode_mega.cu``): one cooperative launch per
decode step for dense bf16 models and buckets of 1, 2, 4 or 8 rows, single GPU or tensor parallel.

``MegaDecode.plan(model)`` decides whether the model qualifies (geometry the kernel is compiled for,
every reduction length a multiple of ``32 * 8 / M``, shared memory for the activation rows) and
uploads the per-layer pointer table once; ``launch(M, advance)`` fills the argument block from the
bucket's buffers and launches on the current stream (it is captured into the bucket's CUDA graph
like any other kernel).  Models that do not qualify keep the multi-kernel step.

The reference keeps its persistent kernel to a slice of one layer (``backends/corex/kernels/mega.cu``);
the launch ledger that motivates it is ``docs/DECODE-LAUNCH-LEDGER.md:15-40``.
"""
from __future__ import annotations

import ctypes
import math
import os

import torch

from ...config import LINEAR
from ...ops import _lib, kernels as K
from ...parallel.tp import _TpCommStruct

# Off by default: measured on B200 (qwen35-4b, batch 1) the persistent step takes 3.3 ms against 2.26 ms
# of the graph of PDL-chained kernels - a grid-wide barrier costs 4-5 us here, as much as a kernel
# boundary, and a kernel boundary under programmatic dependent launch overlaps the next projection's
# weight prefetch with the previous kernel's drain, which a barrier cannot.  COFFIN_MEGA=1 switches it on.
ENABLED = os.environ.get("COFFIN_MEGA", "0") == "1"
PREFETCH_KB = int(os.environ.get("COFFIN_MEGA_PREFETCH_KB", "0"))
# most stages per warp of the weight ring (0 = off, the default: the 256-byte bulk copies that the
# fragment layout forces are slower than the warps' own 16-byte loads, 5.8 ms against 3.3 ms per step)
RING = int(os.environ.get("COFFIN_MEGA_RING", "0"))
SMEM_LIMIT = 226 * 1024
STAGE_BYTES = 5120                                          # kStageBytes of decode_mega.cu
ROWS = (1, 2, 4, 8)


class _Layer(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in
                ("w_in", "w_out", "w_gu", "w_down", "in_gain", "post_gain", "conv_w", "A_log", "dt_bias", "norm_w",
                 "qg", "kg", "ring", "state", "kpool", "vpool")] + [("kind", ctypes.c_int), ("n_in", ctypes.c_int)]


_PTRS = ("layers", "embed", "tokens_in", "slots", "block_table", "cos", "sin", "final_gain", "lm_head", "tokens",
         "positions", "rope_pos", "res0", "res1", "h", "proj", "mix", "inter", "part_o", "part_ml", "logits", "cand",
         "next", "bar", "status", "trace")
_INTS = ("n_layers", "M", "H", "I", "ld_proj", "ld_logits", "ldbt", "nk", "nv", "dk", "dv", "nh", "nkv", "rot", "nsplit",
         "vocab_local", "vocab_total", "vocab_off", "part_floats", "xs_elems", "advance", "use_res0", "prefetch", "tp_on",
         "hd", "ring_stages")


class _Args(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_void_p) for n in _PTRS] + [("wait_ns", ctypes.c_uint64)] +
                [(n, ctypes.c_int) for n in _INTS] + [("eps", ctypes.c_float), ("scale_log2", ctypes.c_float),
                                                      ("tp", _TpCommStruct)])


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


class MegaDecode:
    def __init__(self, model, grid: int, rep: int) -> None:
        self.model, self.grid, self.rep = model, grid, rep
        c, dev = model.cfg, model.device
        self.lib = _lib.lib()
        assert ctypes.sizeof(_Args) == self.lib.cb_decode_mega_args_size(), "MegaArgs layout mismatch"
        assert ctypes.sizeof(_Layer) == self.lib.cb_decode_mega_layer_size(), "MegaLayer layout mismatch"
        arr = (_Layer * len(model.layers))()
        for li, lw in enumerate(model.layers):
            e = arr[li]
            e.w_in, e.w_out, e.w_gu, e.w_down = _ptr(lw.w_in), _ptr(lw.w_out), _ptr(lw.w_gu), _ptr(lw.w_down)
            e.in_gain, e.post_gain = _ptr(lw.in_gain), _ptr(lw.post_gain)
            e.n_in = lw.w_in.shape[0]
            if lw.kind == LINEAR:
                j = model.lin_ids[li]
                e.kind = 0
                e.conv_w, e.A_log, e.dt_bias, e.norm_w = _ptr(lw.conv_w), _ptr(lw.A_log), _ptr(lw.dt_bias), _ptr(lw.norm_w)
                e.ring, e.state = _ptr(model.ring[j]), _ptr(model.state[j])
            else:
                j = model.full_ids[li]
                e.kind = 1
                e.qg, e.kg = _ptr(lw.qg), _ptr(lw.kg)
                e.kpool, e.vpool = _ptr(model.kpool[j]), _ptr(model.vpool[j])
        raw = bytes(arr)
        self.layers_dev = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(dev)
        self.bar = torch.zeros(4, dtype=torch.int32, device=dev)
        self._bufs: dict = {}
        self._args: dict = {}
        self.trace: torch.Tensor | None = None        # %globaltimer stamps of CTA 0 (see ``phase_times``)
        self.mixw = max(c.lin_vdim if model.lin_ids else 0, c.num_attention_heads * c.head_dim if model.full_ids else 0)

    # ------------------------------------------------------------------ qualification
    @staticmethod
    def _geometry(model):
        c = model.cfg
        rep = c.num_attention_heads // max(1, c.num_key_value_heads)
        Ks = [c.hidden_size, c.intermediate_size]
        if model.lin_ids:
            Ks.append(c.lin_vdim)
        if model.full_ids:
            Ks.append(c.num_attention_heads * c.head_dim)
        return rep, Ks

    @classmethod
    def plan(cls, model) -> "MegaDecode | None":
        """A ``MegaDecode`` for ``model`` or ``None`` when the model does not qualify."""
        c = model.cfg
        if not ENABLED or c.is_moe or model.quant != "none" or not (model.pp_first and model.pp_last):
            return None
        if model.ep_world > 1 or model.embed is None or model.lm_head is None or model.kv_dtype != "bf16":
            return None
        for lw in model.layers:
            if any(not isinstance(t, torch.Tensor) for t in (lw.w_in, lw.w_out, lw.w_gu, lw.w_down)):
                return None
        rep, Ks = cls._geometry(model)
        dk, dv, hd = c.linear_key_head_dim, c.linear_value_head_dim, c.head_dim
        lib = _lib.lib()
        if not lib.cb_decode_mega_supported(ctypes.c_int64(dk), ctypes.c_int64(hd), ctypes.c_int64(rep)):
            return None
        if model.lin_ids and (dv % 32 or dv > 256 or (dv // 8) & (dv // 8 - 1) or c.linear_num_value_heads % c.linear_num_key_heads
                              or 2 * dk + 32 > 512):
            return None
        if c.num_attention_heads % max(1, c.num_key_value_heads) or any(k % 8 for k in Ks) or c.rotary_dim % 2:
            return None
        if model.tp is not None and model.tp_world > 1:
            if model.tp.n_sites < 2 * len(model.layers) + 1 or model.tp.slot_floats < 16:
                return None
        # the function's shared-memory attribute is set once, for the largest bucket that fits
        fits = [cls._smem(model, M, rep, 148, cls._stages(model, M, rep)) for M in ROWS if cls._smem(model, M, rep) <= SMEM_LIMIT]
        if not fits:
            return None
        grid = lib.cb_decode_mega_grid(ctypes.c_int64(dk), ctypes.c_int64(hd), ctypes.c_int64(rep), ctypes.c_int64(max(fits)))
        if grid < 1:
            return None
        return cls(model, grid, rep)

    @staticmethod
    def _part_floats(model, M: int, grid: int) -> int:
        """Partial-sum floats the projections of a step need in shared memory (worst CTA)."""
        c = model.cfg
        S = 8 // M
        jobs = []     # (groups, K)
        H, I = c.hidden_size, c.intermediate_size
        for lw in model.layers:
            jobs.append((math.ceil(lw.w_in.shape[0] / (2 * M)), H))
            jobs.append((math.ceil(H / (2 * M)), lw.w_out.shape[1]))
            jobs.append((math.ceil(I / M), H))
            jobs.append((math.ceil(H / (2 * M)), I))
        jobs.append((math.ceil(model.vocab_local / (2 * M)), H))
        need = 0
        for groups, Kd in set(jobs):
            P = (Kd // S + 31) // 32
            ng = math.ceil(groups / grid)
            ipw = math.ceil(ng * P / 16)
            maxseg = (ipw + P - 1) // P + 1 if ipw else 1
            need = max(need, 16 * maxseg * 2 * M * M)
        return need

    @classmethod
    def _region_a(cls, model, M: int, rep: int) -> int:
        """bf16 elements of the first shared-memory region: the activation rows of the projections, or
        the scratch of the mixer phases, whichever is larger."""
        c = model.cfg
        _, Ks = cls._geometry(model)
        xs = max(Ks) * M + 8 * 32
        attn = 2 * (9 * rep * c.head_dim + 64) if model.full_ids else 0            # floats -> bf16 elements
        gdn = 2 * (2 * c.linear_key_head_dim + 36 + 2 * 16 * 32) if model.lin_ids else 0
        return max(xs, attn + 128, gdn + 128)

    @classmethod
    def _smem(cls, model, M: int, rep: int, grid: int = 148, stages: int = 0) -> int:
        part = cls._part_floats(model, M, grid)
        fixed = int(_lib.lib().cb_decode_mega_fixed_smem(ctypes.c_int64(len(model.layers)), ctypes.c_int64(stages)))
        return (cls._region_a(model, M, rep) * 2 + 255) // 256 * 256 + part * 4 + fixed + 256

    @classmethod
    def _stages(cls, model, M: int, rep: int, grid: int = 148) -> int:
        """Stages per warp of the weight ring for bucket ``M``: as many as fit (2..RING), 0 = no ring."""
        for ns in range(min(RING, 4), 1, -1):
            if cls._smem(model, M, rep, grid, ns) <= SMEM_LIMIT:
                return ns
        return 0

    def rows_ok(self, M: int) -> bool:
        """Whether bucket ``M`` runs on the persistent kernel (reduction lengths and shared memory)."""
        if M not in ROWS:
            return False
        _, Ks = self._geometry(self.model)
        S = 8 // M
        if any(k % (S * 8) for k in Ks):
            return False
        if self.model.cfg.intermediate_size % M:
            return False
        return self._smem(self.model, M, self.rep, self.grid) <= SMEM_LIMIT and len(self.model.layers) <= 96

    # ------------------------------------------------------------------ launch
    def _buffers(self, M: int) -> dict:
        key = (M, self.model.lane)
        b = self._bufs.get(key)
        if b is None:
            m, c, dev = self.model, self.model.cfg, self.model.device
            nsplit = max(1, min(64, self.grid // max(1, M * c.num_key_value_heads)))
            b = {"h": torch.zeros(M, c.hidden_size, dtype=torch.float32, device=dev),
                 "mix": torch.zeros(M, max(1, self.mixw), dtype=torch.float32, device=dev),
                 "nsplit": nsplit,
                 "part_o": torch.zeros(M, c.num_attention_heads, nsplit, c.head_dim, dtype=torch.float32, device=dev),
                 "part_ml": torch.zeros(M, c.num_attention_heads, nsplit, 2, dtype=torch.float32, device=dev),
                 "cand": torch.zeros(self.grid, M, 2, dtype=torch.float32, device=dev)}
            self._bufs[key] = b
        return b

    def _build_args(self, M: int, advance: bool) -> _Args:
        m, c = self.model, self.model.cfg
        rb, mb = m._row_buffers(M), self._buffers(M)
        a = _Args()
        a.layers = self.layers_dev.data_ptr()
        a.embed, a.tokens_in, a.slots, a.block_table = _ptr(m.embed), _ptr(rb["tokens"]), _ptr(rb["slots"]), _ptr(rb["block_table"])
        a.cos, a.sin, a.final_gain, a.lm_head = _ptr(m.cos), _ptr(m.sin), _ptr(m.final_gain), _ptr(m.lm_head)
        a.tokens, a.positions, a.rope_pos = _ptr(rb["tokens"]), _ptr(rb["positions"]), _ptr(rb["rope_pos"])
        a.res0, a.res1 = _ptr(rb["res"][0]), _ptr(rb["res"][1])
        a.h, a.proj, a.mix, a.inter = _ptr(mb["h"]), _ptr(rb["proj"]), _ptr(mb["mix"]), _ptr(rb["inter"])
        a.part_o, a.part_ml = _ptr(mb["part_o"]), _ptr(mb["part_ml"])
        a.logits, a.cand, a.next = _ptr(rb["logits_local"]), _ptr(mb["cand"]), _ptr(rb["next"])
        a.bar, a.status = self.bar.data_ptr(), K.status_word(m.device).data_ptr()
        a.trace = _ptr(self.trace)
        a.wait_ns = int(float(os.environ.get("COFFIN_MEGA_WAIT_MS", "2000")) * 1e6)
        a.n_layers, a.M, a.H, a.I = len(m.layers), M, c.hidden_size, c.intermediate_size
        a.ld_proj, a.ld_logits, a.ldbt = rb["proj"].stride(0), rb["logits_local"].stride(0), rb["block_table"].stride(0)
        a.nk, a.nv, a.dk, a.dv = c.linear_num_key_heads, c.linear_num_value_heads, c.linear_key_head_dim, c.linear_value_head_dim
        a.nh, a.nkv, a.rot, a.nsplit = c.num_attention_heads, c.num_key_value_heads, c.rotary_dim, mb["nsplit"]
        a.vocab_local, a.vocab_total, a.vocab_off = m.vocab_local, m.embed.shape[0], m.tp_rank * m.vocab_local
        _, Ks = self._geometry(m)
        a.part_floats = self._part_floats(m, M, self.grid)
        a.xs_elems = self._region_a(m, M, self.rep)
        a.hd, a.ring_stages = c.head_dim, self._stages(m, M, self.rep, self.grid)
        a.advance, a.use_res0, a.prefetch = int(advance), 0, PREFETCH_KB
        tp_on = m.tp is not None and (m.tp_world > 1 or m.tp_force)
        a.tp_on = int(tp_on)
        a.eps, a.scale_log2 = float(m.eps), float(c.head_dim ** -0.5 * math.log2(math.e))
        if tp_on:
            ctypes.memmove(ctypes.byref(a.tp), ctypes.byref(m.tp._struct), ctypes.sizeof(_TpCommStruct))
            a.tp.status = a.status        # one status word for barriers and peer waits
        return a

    def launch(self, M: int, advance: bool = False) -> None:
        key = (M, self.model.lane, bool(advance))
        ent = self._args.get(key)
        if ent is None:
            a = self._build_args(M, advance)
            ent = self._args[key] = (a, self._smem(self.model, M, self.rep, self.grid, a.ring_stages))
        a, smem = ent
        c = self.model.cfg
        fn = self.lib.cb_decode_mega
        fn.restype = ctypes.c_int
        rc = fn(ctypes.byref(a), ctypes.c_int64(a.dk), ctypes.c_int64(c.head_dim), ctypes.c_int64(self.rep),
                ctypes.c_int64(self.grid), ctypes.c_int64(smem), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc != 0:
            raise _lib.KernelError(f"cb_decode_mega failed ({rc})")
        K._count()

    STAMPS_PER_LAYER = 14
    PHASES = ("in: prologue", "in: projection", "barrier", "mixer", "barrier", "out: prologue", "out: projection",
              "barrier", "gate|up: prologue", "gate|up: projection", "barrier", "down: prologue", "down: projection",
              "barrier")

    def enable_trace(self, on: bool = True) -> None:
        """Make CTA 0 stamp ``%globaltimer`` at every phase boundary of the following launches."""
        n = 4 + self.STAMPS_PER_LAYER * len(self.model.layers)
        self.trace = torch.zeros(n, dtype=torch.int64, device=self.model.device) if on else None
        self._args.clear()

    def phase_times(self) -> dict:
        """Microseconds per phase kind of the last traced launch: per-layer sums split by layer kind,
        the head, and the whole step (first to last stamp)."""
        t = self.trace.cpu().tolist()
        L = len(self.model.layers)
        out = {"step_us": (t[-1] - t[0]) / 1e3, "lin": {}, "full": {}, "head": {}}
        for li, lw in enumerate(self.model.layers):
            base = 1 + li * self.STAMPS_PER_LAYER
            kind = "lin" if lw.kind == LINEAR else "full"
            for j, name in enumerate(self.PHASES):
                key = name if name != "barrier" else f"barrier {j}"
                out[kind][key] = out[kind].get(key, 0.0) + (t[base + j] - t[base + j - 1]) / 1e3
        base = 1 + L * self.STAMPS_PER_LAYER
        for j, name in enumerate(("head: prologue", "head: projection", "barrier")):
            out["head"][name] = (t[base + j] - t[base + j - 1]) / 1e3
        return out

    def reset(self) -> None:
        """After a failed step: the barrier counter may have been left between two targets."""
        self.bar.zero_()
