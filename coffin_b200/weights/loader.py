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


def load_checkpoint(model_dir: str | Path, device: str = "cpu", vision: bool = True) -> dict[str, torch.Tensor]:
    from safetensors import safe_open
    model_dir = Path(model_dir)
    from .quant_io import is_quantized_dir, load_quantized
    if is_quantized_dir(model_dir):
        return load_quantized(model_dir, device=device)
    sd: dict[str, torch.Tensor] = {}
    for f in shard_files(model_dir):
        with safe_open(str(f), framework="pt", device=device) as fh:
            for k in fh.keys():
                if not k.startswith(KEEP_PREFIXES):
                    continue
                if not vision and k.startswith("model.visual."):
                    continue
                sd[k] = fh.get_tensor(k)
    return fuse_experts(sd)
