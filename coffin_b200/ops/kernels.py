"""Python entry points of the sm_100a kernels (thin shape-checking wrappers over ctypes).

Every function launches on the current CUDA stream and writes into caller-owned buffers
where one is passed, so a decode step can be captured in a CUDA graph with fixed addresses.
The capability list mirrors the reference's op table (``backends/protocol.py:129-498``)
at the granularity of the fused kernels, not op for op.
"""
from __future__ import annotations

import contextlib
import os

import torch

from . import _lib
from ._lib import call

BLOCK = 64          # tokens per KV block (and key tile)
RING = 16           # conv ring depth of the delta-net layers

_status: dict[int, torch.Tensor] = {}
LAUNCHES = 0        # kernels launched through this module (bench bookkeeping)
STREAM_GEMV = True   # route single-row projections to the cp.async streaming kernel (when GEMV_IMPL == 'scalar')
GEMV_IMPL = "mma"     # 'mma': tensor-core GEMV for every M <= 8; 'scalar': FMA kernels
# tensor parallel decode: pull + residual + norm in the pushing kernel's last CTA instead of a pull kernel.  Opt-in:
# measured at two ranks it is 2 % slower (1.843 vs 1.800 ms per token) - under programmatic dependent launch the
# pull kernel is already resident when the projection ends, and its 1024-thread CTA beats a 256-thread tail
TP_FUSED_TAIL = os.environ.get("COFFIN_TP_FUSED_TAIL", "0") == "1"
ATTN_TC = os.environ.get("COFFIN_ATTN_TC", "1") != "0"   # dense causal prefill attention on tcgen05 (else the mma.sync kernel)
ATTN_TC_TRACE = None  # debugging: int64 device tensor [tiles, 8] that receives the stamps of one CTA of the tcgen05 attention kernel
ATTN_TC_MIN_T = 32    # shorter query blocks (verify passes, tails) stay on the mma.sync kernel


@contextlib.contextmanager
def capture_graph(graph: "torch.cuda.CUDAGraph", pool=None):
    """``torch.cuda.graph`` with the garbage collector held off.  A collection that runs while a
    stream is capturing may finalise CUDA graphs of dead models; destroying a graph is not permitted
    during a capture and invalidates it (the next launch fails with a stream-capture error).  Dead
    objects are therefore collected before the capture starts and automatic collection is disabled
    until it ends."""
    import gc
    gc.collect()
    was_enabled = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph, pool=pool):
            yield
    finally:
        if was_enabled:
            gc.enable()


def _count(n: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += n


def status_word(device=None) -> torch.Tensor:
    """Per-device int32 status word the tensor-core kernels set when a bounded wait runs out."""
    dev = torch.device(device if device is not None else torch.cuda.current_device())
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=f"cuda:{idx}")
        _status[idx] = t
        watch_status(t[:1], f"cuda:{idx}")
    return t


def check_status() -> None:
    for idx, t in _status.items():
        code = int(t[0].item())
        if code:
            t.zero_()
            raise _lib.KernelError(f"device-side wait timed out on cuda:{idx} (role {code})")


# Status words watched by the serving path.  A bounded device-side wait that runs out sets a word and
# lets the kernel finish with whatever data it has, so the host has to look at the words after every
# step or a stalled peer turns into wrong tokens.  ``poll_status`` queues one small asynchronous copy
# per word into pinned host memory behind the step's kernels; ``raise_on_status`` reads the pinned
# values after the caller's own synchronisation (the token read-back), so the check adds no sync.
_watch: list[list] = []      # [device int32 view (1 element), pinned host int32 (1 element), label]


def watch_status(word: torch.Tensor, label: str) -> None:
    assert word.dtype == torch.int32 and word.numel() == 1 and word.is_cuda
    _watch.append([word, torch.zeros(1, dtype=torch.int32).pin_memory(), label])


def unwatch_status(label: str) -> None:
    _watch[:] = [w for w in _watch if w[2] != label]


def poll_status() -> None:
    """Queue the read-back of every watched status word on the current stream."""
    for word, host, _ in _watch:
        host.copy_(word, non_blocking=True)


def raise_on_status() -> None:
    """After a synchronisation that followed ``poll_status``: raise if any word was set (and clear it)."""
    bad = [(label, int(host[0])) for _, host, label in _watch if int(host[0])]
    if bad:
        for word, host, _ in _watch:
            word.zero_()
            host.zero_()
        raise _lib.KernelError("device-side wait timed out: " + ", ".join(f"{l} (role {c})" for l, c in bad))


# ------------------------------------------------------------------ row-wise kernels
def embed_gather(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    T, (V, H) = tokens.numel(), table.shape
    if out is None:
        out = torch.empty(T, H, dtype=table.dtype, device=table.device)
    assert tokens.dtype == torch.int64 and table.dtype == torch.bfloat16
    call("embed_gather", table, tokens, out, T, H, V)
    _count()
    return out


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor | None = None,
            add: torch.Tensor | None = None, res_out: torch.Tensor | None = None, quant: tuple | None = None):
    """``out = rmsnorm(x [+ add]) * gain``; with ``add`` the sum is also written to ``res_out``
    (which may be ``x`` itself).  ``quant = (q int8 [M, N], scale fp32 [M])``: the normalised rows are
    quantised in the same kernel (what ``quant_rows(out)`` would give) and no bf16 output is written
    unless ``out`` is passed too."""
    M, N = x.shape
    if quant is not None:
        assert gain.dtype == torch.float32 and x.stride(1) == 1 and quant[0].is_contiguous()
        call("rmsnorm_q", x, add, gain, res_out, out, M, N, x.stride(0), out.stride(0) if out is not None else 0,
             float(eps), quant[0], quant[1])
        _count()
        return quant
    if out is None:
        out = torch.empty_like(x)
    assert gain.dtype == torch.float32 and x.stride(1) == 1 and out.stride(1) == 1
    if add is not None:
        assert add.stride(0) == x.stride(0)
        if res_out is not None:
            assert res_out.stride(0) == x.stride(0)
    call("rmsnorm", x, add, gain, res_out, out, M, N, x.stride(0), out.stride(0), float(eps))
    _count()
    return out


def swiglu(gu: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    M, two_i = gu.shape
    I = two_i // 2
    if out is None:
        out = torch.empty(M, I, dtype=gu.dtype, device=gu.device)
    call("swiglu", gu, out, M, I, gu.stride(0), out.stride(0))
    _count()
    return out


_argmax_scratch: dict[int, torch.Tensor] = {}


def _argmax_ws(device: torch.device, M: int) -> torch.Tensor:
    """Zero-initialised per-device scratch of the two-stage argmax (partials + arrival tickets)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _argmax_scratch.get(idx)
    import ctypes
    fn = _lib.lib().cb_argmax_scratch_bytes
    fn.restype = ctypes.c_int64
    need = int(fn(ctypes.c_int64(max(M, 64))))
    if t is None or t.numel() < need:
        t = torch.zeros(need, dtype=torch.uint8, device=device)
        _argmax_scratch[idx] = t
    return t


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    M, V = logits.shape
    assert logits.dtype == torch.float32 and M <= 64
    if out is None:
        out = torch.empty(M, dtype=torch.int64, device=logits.device)
    call("argmax", logits, out, M, V, logits.stride(0), _argmax_ws(logits.device, M))
    _count()
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, u: torch.Tensor,
           out: torch.Tensor | None = None) -> torch.Tensor:
    """Per-row temperature sampling (``temperature[row] <= 0`` = greedy) with host-supplied
    uniforms ``u``."""
    M, V = logits.shape
    if out is None:
        out = torch.empty(M, dtype=torch.int64, device=logits.device)
    call("sample", logits, temperature, u, out, M, V, logits.stride(0))
    _count()
    return out


def block_copy(dst: torch.Tensor, src: torch.Tensor, dst_idx: torch.Tensor, src_idx: torch.Tensor) -> None:
    """``dst[dst_idx[j]] = src[src_idx[j]]`` over the leading axis (KV block COW, state snapshots)."""
    nbytes = dst[0].numel() * dst.element_size()
    assert src[0].numel() * src.element_size() == nbytes and dst_idx.dtype == torch.int64
    call("block_copy", dst, src, dst_idx, src_idx, dst_idx.numel(), nbytes)
    _count()


# ------------------------------------------------------------------ projections
# Batched decode rows: the fused add + RMSNorm prologue is repeated by every CTA of a projection
# (hundreds of CTAs x M rows of conversions), which at M >= 2 costs more issue slots than the weight
# stream leaves free.  From this many rows on, the rows are normalised once by a small kernel and the
# projection copies them.
NORM_SPLIT_ROWS = int(os.environ.get("COFFIN_NORM_SPLIT_ROWS", "2"))
_norm_scratch: dict[tuple, torch.Tensor] = {}


# Tensor-parallel decode: the partial sums of the previous row-parallel projection are pulled, added to
# the residual and normalised once per row by a one-CTA kernel; the projection then copies the result.
# (Pulling inside the projection made every one of its CTAs read world x K pairs.)
TP_PULL_SPLIT = True


def _pull_norm_rows(tp, site: int, res_in: torch.Tensor, gain: torch.Tensor, res_out, eps: float) -> torch.Tensor:
    M, K = res_in.shape
    key = (M, K, res_in.device.index)
    buf = _norm_scratch.get(key)
    if buf is None:
        buf = _norm_scratch[key] = torch.empty(M, K, dtype=torch.bfloat16, device=res_in.device)
    call("tp_pull_norm", tp.cstruct_ref(), site, res_in, gain, res_out, buf, M, K, float(eps))
    _count()
    return buf


def _norm_rows(res_in: torch.Tensor, add, gain: torch.Tensor, res_out, eps: float) -> torch.Tensor:
    """``rmsnorm(res_in + add) * gain`` into a per-shape scratch (stream-ordered reuse); ``res_out``
    receives the sum, as the fused prologue would have written it."""
    M, K = res_in.shape
    key = (M, K, res_in.device.index)
    buf = _norm_scratch.get(key)
    if buf is None:
        buf = _norm_scratch[key] = torch.empty(M, K, dtype=torch.bfloat16, device=res_in.device)
    if add is None and res_out is not None and res_out.data_ptr() != res_in.data_ptr():
        res_out.copy_(res_in)
    rmsnorm(res_in, gain, eps, out=buf, add=add, res_out=res_out)
    return buf


def gemv(W: torch.Tensor, x: torch.Tensor | None, out: torch.Tensor | None, *, swiglu: bool = False,
         norm: tuple | None = None, tp=None, pull_site: int = -1, push_site: int = -1, rows: int | None = None,
         tail: tuple | None = None) -> torch.Tensor | None:
    """Decode projection for 1, 2, 4 or 8 rows.

    ``W [N, K]`` (``[2I, K]`` gate rows then up rows with ``swiglu``); ``out [M, N]`` bf16 or fp32.
    ``norm = (res_in, add | None, gain, res_out | None, eps)`` replaces ``x`` by
    ``rmsnorm(res_in + add) * gain`` computed inside the kernel; ``res_out`` receives the sum.
    Tensor parallel (``tp`` = ``parallel.tp.TpComm``): ``push_site >= 0`` sends the fp32 partial
    outputs to every rank's inbox instead of writing ``out``; ``pull_site >= 0`` takes ``add`` as the
    sum over ranks of that site's inbox.  ``tail = (res_in, gain, res_out, eps)`` with a push: the last CTA of
    the pushing kernel also does the consumer's work (pull, residual add, RMSNorm); the projection that
    later names this site as ``pull_site`` finds the normalised rows ready and launches no pull kernel.
    """
    M = out.shape[0] if out is not None else rows
    K = W.shape[1]
    N = W.shape[0] // 2 if swiglu else W.shape[0]
    if (tail is not None and tail[1] is not None and push_site >= 0 and TP_FUSED_TAIL and TP_PULL_SPLIT and GEMV_IMPL == "mma"
            and norm is None and not swiglu and M * K * 2 <= 160 * 1024 and N % 8 == 0):
        t_res, t_gain, t_out, t_eps = tail
        key = (M, N, x.device.index)
        buf = _norm_scratch.get(key)
        if buf is None:
            buf = _norm_scratch[key] = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
        call("gemv_mma_bf16_tail", W, x, M, N, K, tp.cstruct_ref(), push_site, t_res, t_gain, t_out, buf, float(t_eps))
        if not hasattr(tp, "_fused"):
            tp._fused = {}
        tp._fused[push_site] = buf
        _count()
        return None
    f32 = out is not None and out.dtype == torch.float32
    mode = (1 if swiglu else 0) | (2 if f32 else 0)
    ldy = out.stride(0) if out is not None else N
    tpp = tp.cstruct_ref() if tp is not None and (pull_site >= 0 or push_site >= 0) else None
    if norm is None:
        assert x is not None and x.is_contiguous() and x.shape == (M, K)
        res_in = add = gain = res_out = None
        eps = 0.0
    else:
        res_in, add, gain, res_out, eps = norm
        assert res_in.is_contiguous() and res_in.shape == (M, K)
        x = None
    if norm is not None and pull_site >= 0 and TP_PULL_SPLIT:
        ready = getattr(tp, "_fused", {}).pop(pull_site, None)      # the pushing kernel's last CTA already pulled and normalised
        x = ready if ready is not None else _pull_norm_rows(tp, pull_site, res_in, gain, res_out, eps)
        res_in = add = gain = res_out = None
        pull_site = -1
        tpp = tp.cstruct_ref() if push_site >= 0 else None
    elif norm is not None and M >= NORM_SPLIT_ROWS and pull_site < 0:
        x, res_in, add, gain, res_out = _norm_rows(res_in, add, gain, res_out, eps), None, None, None, None
    if GEMV_IMPL == "mma" and M * K * 2 <= 160 * 1024:
        call("gemv_mma_bf16", W, x, out, M, N, K, ldy, mode, N, res_in, add, gain, res_out, float(eps), tpp,
             pull_site, push_site)
    elif M == 1 and STREAM_GEMV and K * 2 <= 28 * 1024:
        # batch-1 decode: weights streamed through per-warp cp.async rings
        call("gemv_stream_bf16", W, x, out, N, K, mode, N, res_in, add, gain, res_out, float(eps), tpp,
             pull_site, push_site)
    else:
        call("gemv_bf16", W, x, out, M, N, K, ldy, mode, N, res_in, add, gain, res_out, float(eps), tpp,
             pull_site, push_site)
    _count()
    return out


def gemv_i8(Wq: torch.Tensor, wscale: torch.Tensor, x: torch.Tensor | None, out: torch.Tensor | None, *,
            swiglu: bool = False, norm: tuple | None = None, tp=None, pull_site: int = -1, push_site: int = -1,
            rows: int | None = None) -> torch.Tensor | None:
    """W8A8 decode projection: int8 weights ``[N, K]`` (``[2I, K]`` with ``swiglu``) + per-row scales;
    the activation rows are quantised per token inside the kernel."""
    M = out.shape[0] if out is not None else rows
    K = Wq.shape[1]
    N = Wq.shape[0] // 2 if swiglu else Wq.shape[0]
    mode = (1 if swiglu else 0) | (2 if out is not None and out.dtype == torch.float32 else 0)
    ldy = out.stride(0) if out is not None else N
    tpp = tp.cstruct_ref() if tp is not None and (pull_site >= 0 or push_site >= 0) else None
    if norm is None:
        assert x is not None and x.is_contiguous() and x.shape == (M, K)
        res_in = add = gain = res_out = None
        eps = 0.0
    else:
        res_in, add, gain, res_out, eps = norm
        x = None
        if pull_site >= 0 and TP_PULL_SPLIT:
            x, res_in, add, gain, res_out = _pull_norm_rows(tp, pull_site, res_in, gain, res_out, eps), None, None, None, None
            pull_site = -1
            tpp = tp.cstruct_ref() if push_site >= 0 else None
        elif M >= NORM_SPLIT_ROWS and pull_site < 0:
            x, res_in, add, gain, res_out = _norm_rows(res_in, add, gain, res_out, eps), None, None, None, None
    call("gemv_i8", Wq, wscale, x, out, M, N, K, ldy, mode, N, res_in, add, gain, res_out, float(eps), tpp,
         pull_site, push_site)
    _count()
    return out


def gemv_w4(Wq: torch.Tensor, wscale: torch.Tensor, x: torch.Tensor | None, out: torch.Tensor, *,
            swiglu: bool = False, norm: tuple | None = None) -> torch.Tensor:
    """W4A8 decode projection: codes ``[N, K/2]`` uint8 (``[2I, K/2]`` with ``swiglu``), scales
    ``[N, K/128]`` fp32 (``weights.quant.W4A8Weight.to_nk``); activations quantised per token in the kernel."""
    M = out.shape[0]
    K = Wq.shape[1] * 2
    N = Wq.shape[0] // 2 if swiglu else Wq.shape[0]
    mode = (1 if swiglu else 0) | (2 if out.dtype == torch.float32 else 0)
    if norm is None:
        assert x is not None and x.is_contiguous() and x.shape == (M, K)
        res_in = add = gain = res_out = None
        eps = 0.0
    else:
        res_in, add, gain, res_out, eps = norm
        x = None
        if M >= NORM_SPLIT_ROWS:
            x, res_in, add, gain, res_out = _norm_rows(res_in, add, gain, res_out, eps), None, None, None, None
    call("gemv_w4", Wq, wscale, x, out, M, N, K, out.stride(0), mode, N, res_in, add, gain, res_out, float(eps))
    _count()
    return out


def moe_gemv_w4(Wq, wscale, x, out, slot_expert, slot_xrow, *, swiglu: bool = False) -> torch.Tensor:
    """Routed experts on W4A8 storage: ``Wq [E, rows, K/2]``, ``wscale [E, rows, K/128]``; slot ``s``
    multiplies activation row ``slot_xrow[s]`` by expert ``slot_expert[s]`` (``< 0``: skipped)."""
    n_slots = out.shape[0]
    K = Wq.shape[2] * 2
    N = Wq.shape[1] // 2 if swiglu else Wq.shape[1]
    mode = (1 if swiglu else 0) | (2 if out.dtype == torch.float32 else 0)
    call("moe_gemv_w4", Wq, wscale, x, out, n_slots, N, K, out.stride(0), mode, slot_expert, slot_xrow)
    _count()
    return out


def moe_gemv_i8(W, wscale, x, out, slot_expert, slot_xrow, *, swiglu: bool = False) -> torch.Tensor:
    """Routed experts on int8 storage: ``W [E, rows, K]`` int8, ``wscale [E, rows]`` fp32; slot ``s`` multiplies
    activation row ``slot_xrow[s]`` (bf16, quantised per row inside the kernel) by expert ``slot_expert[s]``
    (``< 0``: skipped).  ``swiglu``: ``rows = 2N`` (gate rows, then up rows)."""
    n_slots = out.shape[0]
    Kd = W.shape[2]
    N = W.shape[1] // 2 if swiglu else W.shape[1]
    assert W.dtype == torch.int8 and W.is_contiguous() and wscale.dtype == torch.float32 and wscale.is_contiguous()
    mode = (1 if swiglu else 0) | (2 if out.dtype == torch.float32 else 0)
    call("moe_gemv_i8", W, wscale, x, out, n_slots, N, Kd, out.stride(0), mode, slot_expert, slot_xrow)
    _count()
    return out


def w4_dequant(Wq: torch.Tensor, wscale: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """bf16 ``[N, K]`` from W4 codes + group scales (prefill: expanded once per projection call)."""
    N, K = Wq.shape[0], Wq.shape[1] * 2
    if out is None:
        out = torch.empty(N, K, dtype=torch.bfloat16, device=Wq.device)
    call("w4_dequant", Wq, wscale, out, N, K)
    _count()
    return out


def moe_dispatch(idx: torch.Tensor, n_experts: int) -> dict:
    """Expert-major order of the routed slots ``idx [T, k]`` (local expert id, or < 0 for a slot of
    another rank), computed on the device: ``pos [T*k]`` (sorted row of a slot, -1 = none),
    ``src_tok [T*k]`` (token feeding sorted row r) and the m-tile list consumed by
    :func:`gemm_grouped`.  No count is read back to the host."""
    T, k = idx.shape
    S = T * k
    dev = idx.device
    max_tiles = (S + 127) // 128 + n_experts
    meta = torch.empty(1 + 3 * max_tiles, dtype=torch.int32, device=dev)
    d = {"pos": torch.empty(S, dtype=torch.int32, device=dev),
         "src_tok": torch.empty(S, dtype=torch.int32, device=dev),
         "count": meta[:1], "row0": meta[1:1 + max_tiles], "rows": meta[1 + max_tiles:1 + 2 * max_tiles],
         "expert": meta[1 + 2 * max_tiles:], "max_tiles": max_tiles, "meta": meta}
    call("moe_dispatch", idx, S, k, n_experts, d["pos"], d["src_tok"], d["count"], d["row0"], d["rows"], d["expert"],
         max_tiles)
    _count()
    return d


def gemm_grouped(A: torch.Tensor, W: torch.Tensor, disp: dict, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out[r] = A[r] @ W[expert(r)].T`` for expert-sorted rows ``A [S, K]`` and a weight stack
    ``W [E, N, K]`` (bf16), tiles taken from ``disp`` (:func:`moe_dispatch`).  Rows outside the tile
    list (slots of other ranks) are left untouched."""
    S, Kd = A.shape
    E, N, _ = W.shape
    if out is None:
        out = torch.empty(S, N, dtype=torch.bfloat16, device=A.device)
    call("gemm_bf16_grouped", A, A.stride(0), W, W.stride(1), out, out.stride(0), S, E, N, Kd, disp["count"],
         disp["row0"], disp["rows"], disp["expert"], disp["max_tiles"], status_word(A.device))
    _count()
    return out


def gemm_i8_grouped(Aq: torch.Tensor, a_scale: torch.Tensor, W: torch.Tensor, wscale: torch.Tensor, disp: dict,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """``out[r] = (Aq[r] @ W[expert(r)].T) * a_scale[r] * wscale[expert(r)]`` for expert-sorted int8 rows
    ``Aq [S, K]`` (one scale per row) and an int8 stack ``W [E, N, K]`` with ``wscale [E, N]``, on the
    ``kind::i8`` tensor-core path; tiles from ``disp`` (:func:`moe_dispatch`).  Output bf16 ``[S, N]``."""
    S, Kd = Aq.shape
    E, N, _ = W.shape
    assert Aq.dtype == torch.int8 and W.dtype == torch.int8 and Aq.stride(1) == 1 and W.is_contiguous()
    assert a_scale.dtype == torch.float32 and wscale.dtype == torch.float32 and wscale.is_contiguous()
    if out is None:
        out = torch.empty(S, N, dtype=torch.bfloat16, device=Aq.device)
    call("gemm_i8_grouped", Aq, Aq.stride(0), W, W.stride(1), out, out.stride(0), a_scale, wscale, S, E, N, Kd,
         disp["count"], disp["row0"], disp["rows"], disp["expert"], disp["max_tiles"], status_word(Aq.device))
    _count()
    return out


# Routed-MoE prefill straight from the int4 expert stacks (COFFIN_W4_GROUPED=0: expand to bf16 first).
W4_GROUPED = os.environ.get("COFFIN_W4_GROUPED", "1") != "0"


def gemm_w4_grouped(A: torch.Tensor, Wq: torch.Tensor, wscale: torch.Tensor, disp: dict, *, swiglu: bool = False,
                    out: torch.Tensor | None = None, trace: torch.Tensor | None = None) -> torch.Tensor:
    """``out[r] = A[r] @ dequant(Wq[expert(r)]).T`` for expert-sorted rows ``A [S, K]`` and int4 stacks
    ``Wq [E, Nw, K/2]`` uint8 + ``wscale [E, Nw, K/128]`` fp32 (the layout the decode kernels stream): the
    codes are expanded to bf16 inside the CTA, next to the tensor core.  ``swiglu``: ``Nw = 2N`` (gate rows,
    then up rows) and ``out [S, N] = silu(gate) * up``."""
    S, Kd = A.shape
    E, Nw, half = Wq.shape
    assert half * 2 == Kd and A.stride(1) == 1 and Wq.is_contiguous() and wscale.is_contiguous() and wscale.dtype == torch.float32
    N = Nw // 2 if swiglu else Nw
    if out is None:
        out = torch.empty(S, N, dtype=torch.bfloat16, device=A.device)
    call("gemm_w4_grouped", A, A.stride(0), Wq, wscale, out, out.stride(0), S, E, Nw, Kd, int(swiglu), disp["count"],
         disp["row0"], disp["rows"], disp["expert"], disp["max_tiles"], status_word(A.device), trace)
    _count()
    return out


def w4_grouped_ok(Kd: int) -> bool:
    """The grouped int4 kernel takes rows of at most 20 scale groups, four at a time."""
    return W4_GROUPED and Kd % 512 == 0 and Kd <= 2560


def quant_rows(x: torch.Tensor, swiglu: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-row dynamic int8 quantisation of bf16 rows (optionally of ``silu(gate) * up`` of a
    ``[M, 2I]`` input). Returns ``(q int8 [M, K], scale fp32 [M])``."""
    M = x.shape[0]
    K = x.shape[1] // 2 if swiglu else x.shape[1]
    q = torch.empty(M, K, dtype=torch.int8, device=x.device)
    s = torch.empty(M, dtype=torch.float32, device=x.device)
    call("quant_rows", x, x.stride(0), q, s, M, K, int(swiglu))
    _count()
    return q, s


def gemm(A: torch.Tensor, W: torch.Tensor, out: torch.Tensor | None = None,
         residual: torch.Tensor | None = None, bn: int = 0, push=None) -> torch.Tensor | None:
    """Prefill projection on tcgen05: ``out[M, N] = A[M, K] @ W[N, K]^T (+ residual)``, bf16.

    ``push`` (a ``parallel.tp.TpComm`` with a prefill region): nothing is written to ``out``; every
    output row stays in this rank's peer-visible buffer, from which the rank that owns it pulls it (first half of the fused
    all-reduce; ``TpComm.finish_reduce`` is the second)."""
    M, K = A.shape
    N = W.shape[0]
    assert A.stride(1) == 1 and W.stride(1) == 1
    if push is not None:
        call("gemm_bf16", A, A.stride(0), W, W.stride(0), None, 0, None, 0, M, N, K, bn, push.pf_desc_ptr(),
             push.next_seq(M, N), status_word(A.device))
        _count()
        return None
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=A.device)
    assert out.stride(1) == 1
    if M <= 128 and bn == 0 and SPLITK_GEMM:
        ws, tickets = _splitk_scratch(A.device)
        call("gemm_bf16_splitk", A, A.stride(0), W, W.stride(0), out, out.stride(0), residual,
             residual.stride(0) if residual is not None else 0, M, N, K, ws, ws.numel() * 4, tickets, tickets.numel(),
             status_word(A.device))
        _count()
        return out
    call("gemm_bf16", A, A.stride(0), W, W.stride(0), out, out.stride(0), residual,
         residual.stride(0) if residual is not None else 0, M, N, K, bn, None, 0, status_word(A.device))
    _count()
    return out


# CTA-pair kernel for products of more than 256 rows (COFFIN_GEMM_PAIR=0: one-CTA kernel everywhere).
PAIR_GEMM = os.environ.get("COFFIN_GEMM_PAIR", "1") != "0"
PAIR_MIN_ROWS = 257
if not PAIR_GEMM:
    _lib.call_nostream("set_gemm_pair", 0)


def gemm_swiglu(A: torch.Tensor, Wgu: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out[M, I] = silu(A @ Wgu[:I]^T) * (A @ Wgu[I:]^T)``: the gate|up projection with the SwiGLU
    product taken in the GEMM epilogue (CTA-pair kernel; the even CTA of a pair stages gate rows, the
    odd one the matching up rows), so the ``[M, 2I]`` intermediate is never written.  Smaller products
    run as projection + ``swiglu``."""
    M, K = A.shape
    I = Wgu.shape[0] // 2
    assert A.stride(1) == 1 and Wgu.stride(1) == 1
    if out is None:
        out = torch.empty(M, I, dtype=torch.bfloat16, device=A.device)
    assert out.stride(1) == 1
    if not (PAIR_GEMM and M >= PAIR_MIN_ROWS and I >= 128):
        return swiglu(gemm(A, Wgu), out=out)
    call("gemm_bf16_swiglu", A, A.stride(0), Wgu, Wgu.stride(0), out, out.stride(0), M, I, I, K, status_word(A.device))
    _count()
    return out


def gemm_i8_swiglu(Aq: torch.Tensor, a_scale: torch.Tensor, Wq: torch.Tensor, w_scale: torch.Tensor,
                   out: torch.Tensor | None = None) -> torch.Tensor:
    """W8A8 form of :func:`gemm_swiglu`: ``out[M, I] = silu(gate) * up`` of the int8 gate|up projection, scales
    applied before the activation.  More than 256 rows only (callers fall back to projection + ``quant_rows(swiglu)``)."""
    M, K = Aq.shape
    I = Wq.shape[0] // 2
    assert PAIR_GEMM and M >= PAIR_MIN_ROWS and I >= 128
    if out is None:
        out = torch.empty(M, I, dtype=torch.bfloat16, device=Aq.device)
    call("gemm_i8_swiglu", Aq, Aq.stride(0), Wq, Wq.stride(0), out, out.stride(0), a_scale, w_scale, M, I, I, K,
         status_word(Aq.device))
    _count()
    return out


# Products with at most 128 rows (batched decode buckets of 16..64 rows, small prefill chunks) split K
# over CTAs: fp32 partial tiles in a per-device workspace, reduced by the last slice to arrive.
SPLITK_GEMM = os.environ.get("COFFIN_SPLITK_GEMM", "1") != "0"
_splitk: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}


def _splitk_scratch(device) -> tuple[torch.Tensor, torch.Tensor]:
    idx = torch.device(device).index or 0      # one compute stream per device: its launches are ordered
    s = _splitk.get(idx)
    if s is None:
        # 148 slice-tiles of 128 x 256 fp32 is the most one launch parks (tiles * slices <= SMs)
        s = _splitk[idx] = (torch.empty(160 * 128 * 256, dtype=torch.float32, device=device),
                            torch.zeros(4096, dtype=torch.int32, device=device))
    return s


def gemm_i8(Aq: torch.Tensor, a_scale: torch.Tensor, Wq: torch.Tensor, w_scale: torch.Tensor,
            out: torch.Tensor | None = None, residual: torch.Tensor | None = None, bn: int = 0,
            push=None) -> torch.Tensor | None:
    """W8A8 projection: int8 x int8 -> int32 on tcgen05 (kind::i8), ``* a_scale[m] * w_scale[n]``."""
    M, K = Aq.shape
    N = Wq.shape[0]
    if push is not None:
        call("gemm_i8", Aq, Aq.stride(0), Wq, Wq.stride(0), None, 0, None, 0, a_scale, w_scale, M, N, K, bn,
             push.pf_desc_ptr(), push.next_seq(M, N), status_word(Aq.device))
        _count()
        return None
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=Aq.device)
    if M <= 128 and bn == 0 and SPLITK_GEMM:
        ws, tickets = _splitk_scratch(Aq.device)
        call("gemm_i8_splitk", Aq, Aq.stride(0), Wq, Wq.stride(0), out, out.stride(0), residual,
             residual.stride(0) if residual is not None else 0, a_scale, w_scale, M, N, K, ws, ws.numel() * 4, tickets,
             tickets.numel(), status_word(Aq.device))
        _count()
        return out
    call("gemm_i8", Aq, Aq.stride(0), Wq, Wq.stride(0), out, out.stride(0), residual,
         residual.stride(0) if residual is not None else 0, a_scale, w_scale, M, N, K, bn, None, 0,
         status_word(Aq.device))
    _count()
    return out


# ------------------------------------------------------------------ gated delta net
def gdn_decode(proj, conv_w, A_log, dt_bias, norm_w, ring, state, slots, positions, out, *, nk, nv, dk, dv,
               eps, ntok: int = 1, record: torch.Tensor | None = None, write_state: bool = True,
               gate_sigmoid: bool = False) -> torch.Tensor:
    M = slots.numel()
    assert proj.shape[0] == M * ntok and slots.dtype == torch.int32 and positions.dtype == torch.int32
    call("gdn_decode", proj, proj.stride(0), conv_w, A_log, dt_bias, norm_w, ring, state, slots, positions,
         out, out.stride(0), record, record.shape[1] if record is not None else 0, M, ntok,
         int(write_state), nk, nv, dk, dv, float(eps), int(gate_sigmoid))
    _count()
    return out


def gdn_commit(state, record, slots, steps, *, nv, dk, dv) -> None:
    call("gdn_commit", state, record, slots, steps, record.shape[1], slots.numel(), nv, dk, dv)
    _count()


def gdn_prefill_scratch_floats(T: int, nk: int, nv: int, dk: int, dv: int) -> int:
    fn = _lib.lib().cb_gdn_prefill_scratch
    import ctypes
    fn.restype = ctypes.c_int64
    return int(fn(*[ctypes.c_int64(v) for v in (T, nk, nv, dk, dv)]))


def gdn_prefill(proj, conv_w, A_log, dt_bias, norm_w, ring_seq, state_seq, scratch, out, *, pos0, nk, nv, dk, dv,
                eps, gate_sigmoid: bool = False) -> torch.Tensor:
    T = proj.shape[0]
    assert scratch.dtype == torch.float32 and scratch.numel() >= gdn_prefill_scratch_floats(T, nk, nv, dk, dv)
    call("gdn_prefill", proj, proj.stride(0), conv_w, A_log, dt_bias, norm_w, ring_seq, state_seq, scratch,
         out, out.stride(0), T, pos0, nk, nv, dk, dv, float(eps), int(gate_sigmoid))
    _count(5)
    return out


# ------------------------------------------------------------------ attention
def attn_prep(proj, qg, kg, cos, sin, rope_idx, kv_slot, q_out, kpool, vpool, *, nh, nkv, hd, rot, eps,
              kscale=None, vscale=None) -> None:
    """``kscale`` / ``vscale`` (fp32 ``[slots, nkv]``): the pools are int8 and the appended rows are
    quantised per (token, kv head)."""
    T = proj.shape[0]
    assert (kscale is None) == (vscale is None) and (kscale is None) == (kpool.dtype != torch.int8)
    call("attn_prep", proj, proj.stride(0), qg, kg, cos, sin, rope_idx, kv_slot, q_out, kpool, vpool,
         T, nh, nkv, hd, rot, float(eps), kscale, vscale)
    _count()


def attn_prefill(q, proj, kpool, vpool, block_table, out, *, q_pos0, nh, nkv, hd, causal: bool = True,
                 kv_len: int = 0, keep: torch.Tensor | None = None, ratio: int = 0, kscale=None, vscale=None) -> torch.Tensor:
    """``proj`` supplies the per-head output gate (``None``: no gate). ``causal=False`` attends to the
    first ``kv_len`` keys of the block table (bidirectional, used by the vision tower).  ``keep``
    (int32 ``[T, words]`` bit mask over blocks of ``ratio`` tokens) restricts query ``t`` to the kept
    blocks plus the tokens after its last complete block."""
    T = q.shape[0]
    if (ATTN_TC and causal and keep is None and kscale is None and T >= ATTN_TC_MIN_T and hd in (64, 256)
            and kpool.dtype == torch.bfloat16 and q.is_contiguous() and kpool.is_contiguous() and vpool.is_contiguous()):
        # dense causal attention over bf16 pages: the tcgen05 kernel (TMA pages, TMEM accumulators)
        call("attn_prefill_tc", q, proj, proj.stride(0) if proj is not None else 0, kpool, vpool, kpool.shape[0],
             block_table, out, out.stride(0), T, q_pos0, nh, nkv, hd, status_word(q.device), ATTN_TC_TRACE)
        _count()
        return out
    call("attn_prefill", q, proj, proj.stride(0) if proj is not None else 0, kpool, vpool, block_table, out,
         out.stride(0), T, q_pos0, nh, nkv, hd, int(causal), kv_len, keep,
         keep.stride(0) if keep is not None else 0, ratio, kscale, vscale)
    _count()
    return out


def attn_sparse(q, proj, positions, block_table, kpool, vpool, sel, nsel, part_o, part_ml, tickets, out, *,
                nh, nkv, hd, ratio, nsplit) -> torch.Tensor:
    """Block-selected decode attention: ``q [M, nh, hd]`` normed and rotated, the step's K/V already in
    the pool; row ``m`` reads blocks ``sel[m, :nsel[m]]`` (``nsel < 0``: everything visible) and its tail."""
    M = positions.numel()
    call("attn_sparse", q, proj, proj.stride(0), positions, block_table, block_table.stride(0), kpool, vpool, sel,
         nsel, sel.shape[1], ratio, part_o, part_ml, tickets, out, out.stride(0), M, nh, nkv, hd, nsplit)
    _count()
    return out


# ------------------------------------------------------------------ Qwen4-exp: hyper-connection, QSA indexer
def hyper_norm(stream, gain, normed, *, H, hc, eps, block_out=None, inject=None, add=None) -> torch.Tensor:
    """Grouped zero-centred RMSNorm of the ``hc`` lanes of ``stream [M, hc*H]`` into ``normed``; a
    pending write-back (``stream += add``, then ``stream += block_out (x) inject``) is applied first, in place."""
    M = stream.shape[0]
    assert stream.is_contiguous() and normed.is_contiguous()
    call("hyper_norm", stream, gain, block_out, inject, add, normed, M, H, hc, float(eps))
    _count()
    return normed


def hyper_up(normed, low, Wu, Wi, mixed, inject, *, H, hc) -> None:
    """Read gate + lane mix (``mixed [M, H]``) and write gates (``inject [M, hc]`` fp32) for M <= 8 rows."""
    M, R = low.shape
    call("hyper_up", normed, low, Wu, Wi, mixed, inject, M, H, hc, R)
    _count()


def qsa_index_prep(proj, col0, qgain, cos, sin, rope_idx, kv_slot, iq, ipool, *, ni, di, rot, eps) -> None:
    T = proj.shape[0]
    call("qsa_index_prep", proj, proj.stride(0), col0, qgain, cos, sin, rope_idx, kv_slot, iq, ipool, T, ni, di,
         rot, float(eps))
    _count()


def qsa_block_keys(ipool, bkpool, kgain, cos, sin, block_table, b0, b1, *, ratio, di, rot, eps) -> None:
    """Keys of the blocks ``[b0, b1)`` of the sequence behind ``block_table`` (all their tokens stored)."""
    if b1 > b0:
        call("qsa_block_keys", ipool, bkpool, kgain, cos, sin, block_table, b0, b1, ratio, di, rot, float(eps))
        _count()


def qsa_block_keys_rows(ipool, bkpool, kgain, cos, sin, block_tables, positions, *, ratio, di, rot, eps) -> None:
    """For every decode row whose token completes a block, that block's key (decided on the device)."""
    call("qsa_block_keys_rows", ipool, bkpool, kgain, cos, sin, block_tables, block_tables.stride(0), positions,
         positions.numel(), ratio, di, rot, float(eps))
    _count()


def qsa_select(iq, bkpool, block_table, positions, scores, sel, nsel, *, ni, di, ratio, topk, full_factor,
               mask=None, row_seq=None, shared_table: bool = False) -> None:
    """Top-``topk`` blocks per query row (``sel`` ascending, ``nsel``; -1 = attend to everything)."""
    rows = positions.numel()
    ldbt = 0 if shared_table else block_table.stride(0)
    call("qsa_select", iq, bkpool, block_table, ldbt, positions, row_seq, scores, sel, nsel, mask,
         mask.stride(0) if mask is not None else 0, rows, ni, di, ratio, topk, full_factor, scores.shape[1])
    _count()


def attn_decode(proj, qg, kg, cos, sin, positions, rope_pos, block_table, kpool, vpool, part_o, part_ml, tickets,
                out, *, nh, nkv, hd, rot, nsplit, eps, kscale=None, vscale=None) -> torch.Tensor:
    """``tickets``: zero-initialised int32 ``[M, nkv]`` arrival counters (re-armed by the kernel)."""
    M = positions.numel()
    call("attn_decode", proj, proj.stride(0), qg, kg, cos, sin, positions, rope_pos, block_table,
         block_table.stride(0), kpool, vpool, part_o, part_ml, tickets, out, out.stride(0), M, nh, nkv, hd, rot,
         nsplit, float(eps), kscale, vscale)
    _count()
    return out


def decode_splits(nkv: int, rows: int) -> int:
    """Key-tile splits so that a decode attention launch (one 8-warp CTA per kv head, split and
    row) covers about one wave of SMs."""
    pairs = max(1, nkv * rows)
    if pairs >= ATTN_BATCH_PAIRS:       # tensor-core batch kernel: two 4-warp CTAs per SM
        return max(1, min(32, 296 // pairs))
    return max(1, min(32, 148 // pairs))


# (row, kv head) pairs from which cb_attn_decode runs the tensor-core batch kernel
ATTN_BATCH_PAIRS = int(os.environ.get("COFFIN_ATTN_BATCH_PAIRS", "32"))
if ATTN_BATCH_PAIRS != 32:
    _lib.call_nostream("set_attn_batch_ctas", ATTN_BATCH_PAIRS)
