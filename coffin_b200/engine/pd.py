"""Prefill/decode disaggregation: export a prefilled sequence, adopt it elsewhere.

The exported state is what a decode instance needs to continue without recomputing: the KV rows
of every attention layer for the prompt positions, the delta-net recurrent state and conv window,
the prompt ids and the logits of the last position.  Files are plain ``torch.save`` archives in
``out_dir`` (``state.pt``); with tensor parallelism each rank writes ``rank<i>.pt`` and a barrier
separates writers from readers.  Reference: ``engine/prefix_engine.py:207-413`` (export / adopt /
adopt_merged), ``serving/runtime_parts.py:1135-1267``.
"""
from __future__ import annotations

from pathlib import Path

import torch

BLOCK = 64


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
