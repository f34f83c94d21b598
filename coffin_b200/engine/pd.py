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


REQUIRED = ("prompt", "n", "k", "v", "state", "logits", "meta")


def layer_span(model) -> tuple[int, int]:
    """Global layer range ``[lo, hi)`` this model instance owns: a pipeline stage's configuration carries its
    range in its name (``parallel.pp.stage_config``), a whole model owns ``[0, num_hidden_layers)``."""
    import re
    m = re.search(r"-pp(\d+)-(\d+)$", getattr(model.cfg, "name", ""))
    return (int(m.group(1)), int(m.group(2))) if m else (0, int(model.cfg.num_hidden_layers))


def describe(model) -> dict:
    """What an exported state must agree with on the adopting side (the reference checks the same items in
    ``engine/prefix_engine.py:653-750`` ``_check_state``)."""
    lo, hi = layer_span(model)
    c = model.cfg
    return {"block": BLOCK, "layer_begin": lo, "layer_end": hi, "kv_layers": int(model.kpool.shape[0]),
            "nkv": int(model.kpool.shape[2]), "hd": int(model.kpool.shape[3]), "kv_dtype": str(model.kpool.dtype),
            "kv_scaled": getattr(model, "kscale", None) is not None,
            "state_shapes": [tuple(t.shape) for t in model.snapshot_state(0) if isinstance(t, torch.Tensor)],
            "vocab": int(c.vocab_size), "hidden": int(c.hidden_size), "model": str(getattr(c, "name", ""))}


def build_payload(model, slot: int, table: list[int], prompt: list[int], logits: torch.Tensor | None) -> dict:
    n = len(prompt)
    pos = torch.arange(n)
    slots = torch.tensor(table, dtype=torch.long)[pos // BLOCK] * BLOCK + pos % BLOCK
    slots = slots.to(model.kpool.device)
    return {
        "prompt": list(prompt), "n": n,
        "k": model.kpool[:, slots].cpu(), "v": model.vpool[:, slots].cpu(),
        "ks": model.kscale[:, slots].cpu() if getattr(model, "kscale", None) is not None else None,
        "vs": model.vscale[:, slots].cpu() if getattr(model, "vscale", None) is not None else None,
        "state": [t.cpu() for t in model.snapshot_state(slot)],
        "logits": logits.float().cpu() if logits is not None else None,
        "meta": describe(model),
    }


def export_state(model, slot: int, table: list[int], prompt: list[int], logits: torch.Tensor, out_dir: Path,
                 rank: int = 0) -> int:
    out_dir.mkdir(parents=True, exist_ok=True)
    path = out_dir / ("state.pt" if rank == 0 else f"rank{rank}.pt")
    torch.save(build_payload(model, slot, table, prompt, logits), path)
    return path.stat().st_size


def _check(meta: dict, n: int, prompt_len: int, shapes: dict, has_scales: bool, model, span) -> None:
    mine = describe(model)
    lo, hi = span if span is not None else (mine["layer_begin"], mine["layer_end"])
    if (int(meta["layer_begin"]), int(meta["layer_end"])) != (lo, hi):
        raise ValueError(f"this instance owns layers [{lo}, {hi}) but the state was exported from "
                         f"[{meta['layer_begin']}, {meta['layer_end']}): the pipeline split differs")
    if int(meta["block"]) != BLOCK:
        raise ValueError(f"block size {meta['block']} != local {BLOCK}: the block tables are not interchangeable")
    for key, what in (("kv_layers", "pooled attention layers"), ("nkv", "KV heads"), ("hd", "head width"),
                      ("kv_dtype", "KV dtype"), ("kv_scaled", "KV scale rows"), ("vocab", "vocabulary"), ("hidden", "hidden size")):
        if meta[key] != mine[key]:
            raise ValueError(f"{what}: the state has {meta[key]}, this instance {mine[key]}")
    if n != prompt_len or n < 1:
        raise ValueError(f"the state disagrees with itself: {n} positions for a prompt of {prompt_len} tokens")
    if n + 1 > int(model.max_seq):
        raise ValueError(f"the state holds {n} tokens, beyond this instance's max_seq {model.max_seq}")
    want_kv = (mine["kv_layers"], n, mine["nkv"], mine["hd"])
    for name in ("k", "v"):
        if tuple(shapes[name]) != want_kv:
            raise ValueError(f"{name}: shape {tuple(shapes[name])}, expected {want_kv}")
    if mine["kv_scaled"] and not has_scales:
        raise ValueError("int8 KV rows came without their scales")
    if len(shapes["state"]) != len(mine["state_shapes"]):
        raise ValueError(f"{len(shapes['state'])} recurrent-state tensors, expected {len(mine['state_shapes'])}")
    for i, (got, shape) in enumerate(zip(shapes["state"], mine["state_shapes"])):
        if tuple(got) != tuple(shape):
            raise ValueError(f"recurrent state {i}: shape {tuple(got)}, expected {tuple(shape)}")
    lg = shapes.get("logits")
    if lg is not None and (len(lg) != 1 or int(lg[0]) != mine["vocab"]):
        raise ValueError(f"logits of shape {tuple(lg)} for a vocabulary of {mine['vocab']}")


def check_state(payload: dict, model, span: tuple[int, int] | None = None) -> None:
    """Compare a foreign state with this instance BEFORE any pool row is touched.  Every mismatch means "it
    would load and run, but the output would belong to another model", so each one raises instead of being
    patched over: missing fields (``KeyError``); layer range, block size, pooled layers, heads, head width, KV
    dtype / scaling, tensor shapes, token count, vocabulary (``ValueError``)."""
    missing = [k for k in REQUIRED if k not in payload]
    if missing:
        raise KeyError(f"prefill state is missing {missing}")
    shapes = {"k": payload["k"].shape, "v": payload["v"].shape, "state": [t.shape for t in payload["state"]],
              "logits": payload["logits"].shape if payload["logits"] is not None else None}
    _check(payload["meta"], int(payload["n"]), len(payload["prompt"]), shapes,
           payload.get("ks") is not None and payload.get("vs") is not None, model, span)


def check_descriptor(desc: dict, model) -> None:
    """The same checks for a device-transport descriptor (``state.json``), from its layout table - before the
    exporter's buffer is mapped or a byte is copied."""
    missing = [k for k in ("n", "prompt", "layout", "meta") if k not in desc]
    if missing:
        raise KeyError(f"prefill state descriptor is missing {missing}")
    by = {e["name"]: e["shape"] for e in desc["layout"]}
    for name in ("k", "v", "logits"):
        if name not in by:
            raise KeyError(f"prefill state descriptor has no '{name}' entry")
    states = [by[k] for k in sorted((k for k in by if k.startswith("state")), key=lambda k: int(k[5:]))]
    _check(desc["meta"], int(desc["n"]), len(desc["prompt"]), {"k": by["k"], "v": by["v"], "state": states, "logits": by["logits"]},
           "ks" in by and "vs" in by, model, None)


def merge_parts(parts: list[dict]) -> dict:
    """One state from the exports of several pipeline stages (complementary layer ranges, any order): KV rows
    and recurrent states are stacked along their layer axis in global layer order, the logits come from the
    stage that has them (the last).  Raises when the ranges leave a gap or overlap, or when the parts disagree
    on the prompt, the block size or the head geometry (reference: ``engine/prefix_engine.py:753-874``)."""
    if not parts:
        raise ValueError("no prefill states to merge")
    for p in parts:
        missing = [k for k in REQUIRED if k not in p]
        if missing:
            raise KeyError(f"prefill state is missing {missing}")
    parts = sorted(parts, key=lambda p: int(p["meta"]["layer_begin"]))
    first = parts[0]
    for a, b in zip(parts, parts[1:]):
        if int(a["meta"]["layer_end"]) != int(b["meta"]["layer_begin"]):
            raise ValueError(f"layer ranges [{a['meta']['layer_begin']}, {a['meta']['layer_end']}) and "
                             f"[{b['meta']['layer_begin']}, {b['meta']['layer_end']}) do not join")
        for key in ("block", "nkv", "hd", "kv_dtype", "kv_scaled", "vocab", "hidden"):
            if a["meta"][key] != b["meta"][key]:
                raise ValueError(f"the parts disagree on {key}: {a['meta'][key]} vs {b['meta'][key]}")
        if a["prompt"] != b["prompt"] or int(a["n"]) != int(b["n"]):
            raise ValueError("the parts were exported for different prompts")
    logits = [p["logits"] for p in parts if p["logits"] is not None]
    if len(logits) != 1:
        raise ValueError(f"{len(logits)} parts carry logits; exactly one stage (the last) must")
    cat = lambda name: torch.cat([p[name] for p in parts], 0) if first[name] is not None else None
    meta = dict(first["meta"])
    meta.update(layer_begin=int(first["meta"]["layer_begin"]), layer_end=int(parts[-1]["meta"]["layer_end"]),
                kv_layers=sum(int(p["meta"]["kv_layers"]) for p in parts),
                state_shapes=[(sum(int(p["meta"]["state_shapes"][i][0]) for p in parts), *first["meta"]["state_shapes"][i][1:])
                              for i in range(len(first["meta"]["state_shapes"]))])
    return {"prompt": list(first["prompt"]), "n": int(first["n"]), "k": cat("k"), "v": cat("v"), "ks": cat("ks"), "vs": cat("vs"),
            "state": [torch.cat([p["state"][i] for p in parts], 0) for i in range(len(first["state"]))],
            "logits": logits[0], "meta": meta}


def adopt_payload(model, slot: int, payload: dict, first_block: int = 1, max_new: int = 4096):
    """Check ``payload`` against this instance, then write it into ``slot`` using blocks ``first_block ..``.
    Returns ``(table, prompt, logits)``."""
    check_state(payload, model)
    n = payload["n"]
    nblk = (n + max_new + BLOCK) // BLOCK
    nblk = min(nblk, model.num_blocks - first_block, (model.max_seq + BLOCK - 1) // BLOCK)
    if nblk * BLOCK < n + 1:
        raise RuntimeError("not enough KV blocks to adopt the exported sequence")
    table = list(range(first_block, first_block + nblk))
    pos = torch.arange(n)
    slots = (torch.tensor(table, dtype=torch.long)[pos // BLOCK] * BLOCK + pos % BLOCK).to(model.kpool.device)
    model.kpool[:, slots] = payload["k"].to(model.kpool.device, model.kpool.dtype)
    model.vpool[:, slots] = payload["v"].to(model.vpool.device, model.vpool.dtype)
    if payload.get("ks") is not None:
        model.kscale[:, slots] = payload["ks"].to(model.kscale.device)
        model.vscale[:, slots] = payload["vs"].to(model.vscale.device)
    snap = model.snapshot_state(slot)
    model.restore_state(slot, tuple(t.to(s.device, s.dtype) for t, s in zip(payload["state"], snap)))
    logits = payload["logits"]
    if os.environ.get("COFFIN_PD_TRACE"):
        print(f"[pd] adopt slot={slot} pos={n} blocks={len(table)} first_block={first_block} "
              f"kv_layers={payload['k'].shape[0]} state_tensors={len(payload['state'])}", flush=True)
    if os.environ.get("COFFIN_PD_VERIFY"):
        for line in verify_adopted(model, slot, table, payload):
            print(line, flush=True)
    return table, payload["prompt"], logits.to(getattr(model, "device", "cpu")) if logits is not None else None


def verify_adopted(model, slot: int, table: list[int], payload: dict) -> list[str]:
    """Read back what ``adopt_payload`` just wrote and count the elements that differ, one line per
    tensor.  Repeated output after an adopt can come from a bad write (rows never reached the pool) or a
    bad read (the block table points elsewhere); the read-back tells the two apart.  Printed under
    ``COFFIN_PD_VERIFY`` (reference ``serving/runtime_parts.py:1487-1511``)."""
    n = payload["n"]
    pos = torch.arange(n)
    slots = (torch.tensor(table, dtype=torch.long)[pos // BLOCK] * BLOCK + pos % BLOCK).to(model.kpool.device)
    lines = []
    for name, pool in (("k", model.kpool), ("v", model.vpool)):
        want = payload[name].to(pool.device, pool.dtype)
        got = pool[:, slots]
        for i in range(want.shape[0]):
            bad = int((got[i] != want[i]).sum())
            lines.append(f"[pdverify] {name} layer={i} slot={slot} pos={n} mismatch={bad}/{want[i].numel()}")
    for i, (got, want) in enumerate(zip(model.snapshot_state(slot), payload["state"])):
        bad = int((got.cpu() != want.to(got.dtype).cpu()).sum())
        lines.append(f"[pdverify] state tensor={i} slot={slot} mismatch={bad}/{want.numel()}")
    return lines


def adopt_state(model, slot: int, in_dir: Path, first_block: int = 1, rank: int = 0, max_new: int = 4096):
    """Load an exported sequence into ``slot`` using blocks ``first_block ..``.  Returns
    ``(table, prompt, logits)``."""
    path = in_dir / ("state.pt" if rank == 0 else f"rank{rank}.pt")
    return adopt_payload(model, slot, torch.load(path, map_location="cpu", weights_only=False), first_block, max_new)


def adopt_merged(model, slot: int, in_dirs: list[Path], first_block: int = 1, max_new: int = 4096):
    """Adopt a sequence whose prefill ran as a pipeline: ``in_dirs`` hold one export per stage."""
    parts = [torch.load(Path(d) / "state.pt", map_location="cpu", weights_only=False) for d in in_dirs]
    return adopt_payload(model, slot, merge_parts(parts), first_block, max_new)


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
            "device": torch.device(model.device).index or 0, "prompt": list(prompt), "n": len(prompt), "layout": layout, "token": token,
            "meta": {k: (list(map(list, v)) if k == "state_shapes" else v) for k, v in describe(model).items()}}
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
    check_descriptor(desc, model)
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
