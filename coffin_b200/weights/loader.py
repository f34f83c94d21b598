"""Checkpoint readers: HF safetensors directories and pre-quantised ``quant_index.json`` trees.

``load_checkpoint`` returns a state dict in the canonical key layout of ``weights/init.py``
(routed experts as fused 3-D stacks whatever the on-disk spelling).  Reference loader:
``models/qwen35/weights.py:58-167`` (prefix handling), ``models/qwen35/moe.py:65-145``
(expert fusion), ``quantized_load.py:190-396`` (quantised directories).
"""
from __future__ import annotations

import json
import re
from pathlib import Path

import torch

KEEP_PREFIXES = ("model.language_model.", "mtp.", "lm_head.", "model.visual.")


def shard_files(model_dir: Path) -> list[Path]:
    idx = model_dir / "model.safetensors.index.json"
    if idx.exists():
        names = sorted(set(json.loads(idx.read_text())["weight_map"].values()))
        return [model_dir / n for n in names]
    files = sorted(p for p in model_dir.glob("*.safetensors") if not p.name.startswith("quant-"))
    if not files:
        raise FileNotFoundError(f"no safetensors shards in {model_dir}")
    return files


def fuse_experts(sd: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """Per-expert ``experts.{e}.{gate,up,down}_proj.weight`` and ``gate_up_stack/down_stack``
    spellings -> ``experts.gate_up_proj [E, 2I, H]`` / ``experts.down_proj [E, H, I]``."""
    pat = re.compile(r"^(.*\.mlp\.experts\.)(\d+)\.(gate_proj|up_proj|down_proj)\.weight$")
    groups: dict[str, dict[str, dict[int, torch.Tensor]]] = {}
    for k in list(sd):
        m = pat.match(k)
        if m:
            groups.setdefault(m.group(1), {}).setdefault(m.group(3), {})[int(m.group(2))] = sd.pop(k)
    for base, g in groups.items():
        n = len(g["gate_proj"])
        if any(len(g.get(x, {})) != n for x in ("up_proj", "down_proj")):
            raise ValueError(f"{base}: incomplete expert set")
        sd[base + "gate_up_proj"] = torch.stack([torch.cat([g["gate_proj"][e], g["up_proj"][e]]) for e in range(n)])
        sd[base + "down_proj"] = torch.stack([g["down_proj"][e] for e in range(n)])
    for k in list(sd):
        if k.endswith("experts.gate_up_stack"):
            sd[k[:-len("gate_up_stack")] + "gate_up_proj"] = sd.pop(k)
        elif k.endswith("experts.down_stack"):
            sd[k[:-len("down_stack")] + "down_proj"] = sd.pop(k)
    return sd


def read_sliced(fh, key: str, plan) -> torch.Tensor:
    """Read tensor ``key`` of an open safetensors file cut by a ``parallel.tp.slice_plan`` (only the
    bytes of the slice are read: ``get_slice``)."""
    if plan is None:
        return fh.get_tensor(key)
    kind, ranges = plan
    sl = fh.get_slice(key)
    if kind == "rows":
        parts = [sl[a:b] for a, b in ranges]
        return parts[0] if len(parts) == 1 else torch.cat(parts)
    (a, b), = ranges
    return sl[:, a:b].contiguous()


def load_checkpoint(model_dir: str | Path, device: str = "cpu", vision: bool = True, tp: tuple[int, int] | None = None,
                    layers: tuple[int, int] | None = None) -> dict[str, torch.Tensor]:
    """``tp=(rank, world)``: read only that tensor-parallel rank's slice of every projection (the
    returned dict is marked, ``shard_state_dict`` then passes it through).  ``layers=(l0, l1)``: read
    only the decoder layers of a pipeline stage (the embedding, final norm and head are kept).
    Reference: per-rank ``get_slice`` reads, ``models/qwen35/parallel.py:887-1012``."""
    from safetensors import safe_open
    model_dir = Path(model_dir)
    from .quant_io import is_quantized_dir, load_quantized
    cfg = plan_of = None
    if tp is not None and tp[1] > 1:
        from ..config import load_config
        from ..parallel.tp import TP_MARK, local_config, slice_plan
        cfg = load_config(model_dir)
        local_config(cfg, tp[1])                 # raises when a dimension does not divide
        plan_of = lambda k: slice_plan(cfg, k, tp[0], tp[1])

    def wanted(k: str) -> bool:
        if not k.startswith(KEEP_PREFIXES) or (not vision and k.startswith("model.visual.")):
            return False
        if layers is not None and k.startswith("model.language_model.layers."):
            li = int(k.split(".")[3])
            return layers[0] <= li < layers[1]
        return True

    if is_quantized_dir(model_dir):
        sd = load_quantized(model_dir, device=device, plan_of=plan_of, wanted=wanted)
    else:
        sd = {}
        for f in shard_files(model_dir):
            with safe_open(str(f), framework="pt", device=device) as fh:
                for k in fh.keys():
                    if wanted(k):
                        sd[k] = read_sliced(fh, k, plan_of(k) if plan_of else None)
        sd = fuse_experts(sd)
    if plan_of is not None:
        sd[TP_MARK] = (tp[0], tp[1])
    return sd
