"""Prefill/decode disaggregation: export a prefilled sequence, adopt it elsewhere.

The exported state is what a decode instance needs to continue without recomputing: the KV rows
of every attention layer for the prompt positions, the delta-net recurrent state and conv window,
the prompt ids and the logits of the last position.  Two transports:

* ``file``: plain ``torch.save`` archives in ``out_dir`` (``state.pt``; with tensor parallelism each
  rank writes ``rank<i>.pt`` and a barrier separates writers from readers) - device -> host -> file ->
  host -> device, the reference's route (``engine/prefix_engine.py:207-413``,
  ``serving/runtime_parts.py:1135-1267``).
* ``device``: the exporter packs everything into ONE device buffer and publishes its CUDA IPC handle
  plus a layout table (a small JSON descriptor, ``state.json``); the adopter maps the buffer and copies
  device to device - once over NVLink when the two engines sit on different GPUs of the node, no
  host staging of the KV rows.  The exporter keeps the buffer until ``release_export`` (or until it
  exports the next sequence under the same token).
"""
from __future__ import annotations

import ctypes
import json
import os
from pathlib import Path

import torch

BLOCK = 64
_exports: dict[str, tuple[int, int]] = {}        # token -> (device pointer, bytes) of buffers this process has published


def export_state(model, slot: int, table: list[int], prompt: list[int], logits: torch.Tensor, out_dir: Path,
                 rank: int = 0) -> int:
    out_dir.mkdir(parents=True, exist_ok=True)
    n = len(prompt)
    pos = torch.arange(n)
    slots = torch.tensor(table, dtype=torch.long)[pos // BLOCK] * BLOCK + pos % BLOCK
    slots = slots.to(model.kpool.device)
    payload = {
        "prompt": list(prompt), "n": n,
        "k": model.kpool[:, slots].cpu(), "v": model.vpool[:, slots].cpu(),
        "ks": model.kscale[:, slots].cpu() if getattr(model, "kscale", None) is not None else None,
        "vs": model.vscale[:, slots].cpu() if getattr(model, "vscale", None) is not None else None,
        "state": [t.cpu() for t in model.snapshot_state(slot)],
        "logits": logits.float().cpu(),
    }
    path = out_dir / ("state.pt" if rank == 0 else f"rank{rank}.pt")
    torch.save(payload, path)
    return path.stat().st_size


def adopt_state(model, slot: int, in_dir: Path, first_block: int = 1, rank: int = 0, max_new: int = 4096):
    """Load an exported sequence into ``slot`` using blocks ``first_block ..``.  Returns
    ``(table, prompt, logits)``."""
    path = in_dir / ("state.pt" if rank == 0 else f"rank{rank}.pt")
    payload = torch.load(path, map_location="cpu", weights_only=False)
    n = payload["n"]
    nblk = (n + max_new + BLOCK) // BLOCK
    nblk = min(nblk, model.num_blocks - first_block, (model.max_seq + BLOCK - 1) // BLOCK)
    if nblk * BLOCK < n + 1:
        raise RuntimeError("not enough KV blocks to adopt the exported sequence")
    table = list(range(first_block, first_block + nblk))
    pos = torch.arange(n)
    slots = (torch.tensor(table, dtype=torch.long)[pos // BLOCK] * BLOCK + pos % BLOCK).to(model.kpool.device)
    if payload["k"].dtype != model.kpool.dtype:
        raise RuntimeError(f"exported KV is {payload['k'].dtype}, this engine's pool is {model.kpool.dtype}")
    model.kpool[:, slots] = payload["k"].to(model.kpool.device, model.kpool.dtype)
    model.vpool[:, slots] = payload["v"].to(model.vpool.device, model.vpool.dtype)
    if payload.get("ks") is not None:
        model.kscale[:, slots] = payload["ks"].to(model.kscale.device)
        model.vscale[:, slots] = payload["vs"].to(model.vscale.device)
    snap = model.snapshot_state(slot)
    model.restore_state(slot, tuple(t.to(s.device, s.dtype) for t, s in zip(payload["state"], snap)))
    return table, payload["prompt"], payload["logits"].to(getattr(model, "device", "cpu"))


# ---------------------------------------------------------------------------------------------------
# device transport
def _parts(model, slot: int, table: list[int], n: int, logits: torch.Tensor) -> list[tuple[str, torch.Tensor]]:
    pos = torch.arange(n)
    slots = (torch.tensor(table, dtype=torch.long)[pos // BLOCK] * BLOCK + pos % BLOCK).to(model.kpool.device)
    parts = [("k", model.kpool[:, slots].contiguous()), ("v", model.vpool[:, slots].contiguous())]
    if getattr(model, "kscale", None) is not None:
        parts += [("ks", model.kscale[:, slots].contiguous()), ("vs", model.vscale[:, slots].contiguous())]
    parts += [(f"state{i}", t.contiguous()) for i, t in enumerate(model.snapshot_state(slot)) if isinstance(t, torch.Tensor)]
    parts.append(("logits", logits.float().contiguous()))
    return parts


def export_state_device(model, slot: int, table: list[int], prompt: list[int], logits: torch.Tensor, out_dir: Path,
                        token: str = "default") -> int:
    """Pack the sequence into one IPC-exportable device buffer and write its descriptor to
    ``out_dir/state.json``.  Returns the bytes published."""
    from ..ops import _lib
    lib = _lib.lib()
    out_dir.mkdir(parents=True, exist_ok=True)
    release_export(token)
    parts = _parts(model, slot, table, len(prompt), logits)
    layout, off = [], 0
    for name, t in parts:
        nb = t.numel() * t.element_size()
        layout.append({"name": name, "dtype": str(t.dtype).replace("torch.", ""), "shape": list(t.shape), "offset": off, "bytes": nb})
        off += (nb + 255) // 256 * 256
    base = ctypes.c_void_p()
    rc = lib.cb_peer_alloc(ctypes.c_int64(max(off, 256)), ctypes.byref(base))
    if rc:
        raise _lib.KernelError(f"cb_peer_alloc failed ({rc})")
    stream = torch.cuda.current_stream(model.device).cuda_stream
    for (name, t), ent in zip(parts, layout):
        rc = lib.cb_copy_d2d(ctypes.c_void_p(base.value + ent["offset"]), ctypes.c_void_p(t.data_ptr()), ctypes.c_int64(ent["bytes"]),
                             ctypes.c_void_p(stream))
        if rc:
            raise _lib.KernelError(f"cb_copy_d2d failed ({rc})")
    torch.cuda.synchronize(model.device)          # the adopter may map the buffer as soon as it sees the descriptor
    handle = ctypes.create_string_buffer(64)
    rc = lib.cb_ipc_get_handle(base, handle)
    if rc:
        raise _lib.KernelError(f"cb_ipc_get_handle failed ({rc})")
    _exports[token] = (base.value, off)
    desc = {"transport": "device", "pid": os.getpid(), "ptr": base.value, "handle": handle.raw.hex(), "bytes": off,
            "device": torch.device(model.device).index or 0, "prompt": list(prompt), "n": len(prompt), "layout": layout, "token": token}
    (out_dir / "state.json").write_text(json.dumps(desc))
    return off


def release_export(token: str = "default") -> bool:
    """Free the buffer published under ``token`` (after the adopter has copied it)."""
    from ..ops import _lib
    ent = _exports.pop(token, None)
    if ent is None:
        return False
    _lib.lib().cb_peer_free(ctypes.c_void_p(ent[0]))
    return True


def adopt_state_device(model, slot: int, in_dir: Path, first_block: int = 1, max_new: int = 4096):
    """Map the exporter's buffer (CUDA IPC; the same process uses the pointer directly) and copy the
    sequence device to device into ``slot`` / blocks ``first_block ..``.  Returns ``(table, prompt, logits)``."""
    from ..ops import _lib
    lib = _lib.lib()
    desc = json.loads((in_dir / "state.json").read_text())
    n = desc["n"]
    nblk = min((n + max_new + BLOCK) // BLOCK, model.num_blocks - first_block, (model.max_seq + BLOCK - 1) // BLOCK)
    if nblk * BLOCK < n + 1:
        raise RuntimeError("not enough KV blocks to adopt the exported sequence")
    table = list(range(first_block, first_block + nblk))
    opened = None
    if desc["pid"] == os.getpid():
        src = desc["ptr"]
    else:
        p = ctypes.c_void_p()
        rc = lib.cb_ipc_open_handle(ctypes.create_string_buffer(bytes.fromhex(desc["handle"]), 64), ctypes.byref(p))
        if rc:
            raise _lib.KernelError(f"cb_ipc_open_handle failed ({rc})")
        src = opened = p.value
    try:
        dev = model.kpool.device
        stream = torch.cuda.current_stream(dev).cuda_stream
        got: dict[str, torch.Tensor] = {}
        for ent in desc["layout"]:
            t = torch.empty(ent["shape"], dtype=getattr(torch, ent["dtype"]), device=dev)
            rc = lib.cb_copy_d2d(ctypes.c_void_p(t.data_ptr()), ctypes.c_void_p(src + ent["offset"]), ctypes.c_int64(ent["bytes"]),
                                 ctypes.c_void_p(stream))
            if rc:
                raise _lib.KernelError(f"cb_copy_d2d failed ({rc})")
            got[ent["name"]] = t
        torch.cuda.synchronize(dev)
    finally:
        if opened is not None:
            lib.cb_ipc_close_handle(ctypes.c_void_p(opened))
    if got["k"].dtype != model.kpool.dtype:
        raise RuntimeError(f"exported KV is {got['k'].dtype}, this engine's pool is {model.kpool.dtype}")
    pos = torch.arange(n)
    slots = (torch.tensor(table, dtype=torch.long)[pos // BLOCK] * BLOCK + pos % BLOCK).to(dev)
    model.kpool[:, slots] = got["k"]
    model.vpool[:, slots] = got["v"]
    if "ks" in got:
        model.kscale[:, slots] = got["ks"]
        model.vscale[:, slots] = got["vs"]
    snap = model.snapshot_state(slot)
    it = iter(sorted((k for k in got if k.startswith("state")), key=lambda k: int(k[5:])))
    model.restore_state(slot, tuple(got[next(it)].to(s.dtype) if isinstance(s, torch.Tensor) else s for s in snap))
    return table, desc["prompt"], got["logits"]


def adopt_any(model, slot: int, in_dir: Path, **kw):
    """Adopt whatever ``in_dir`` holds: a device descriptor (``state.json``) or a file archive."""
    if (in_dir / "state.json").exists():
        kw.pop("rank", None)
        return adopt_state_device(model, slot, in_dir, **kw)
    return adopt_state(model, slot, in_dir, **kw)
