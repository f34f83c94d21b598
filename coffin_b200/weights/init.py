"""Random-init state dicts in the HF checkpoint key layout.

Benchmarks and tests have no checkpoint to load (no network), so the weights are
drawn ~N(0, 0.02) in the exact key/shape layout a Qwen3.5 checkpoint uses
(reference loader: ``models/qwen35/weights.py:58-167``; per-layer keys
``models/qwen35/linear_attn.py:74-90``, ``models/qwen35/full_attn.py:82-86``,
``models/qwen35/blocks.py:50-52,133-141``, ``models/qwen35/moe.py:65-145``).
The same dict feeds the CPU oracle and the sm_100a model, and ``save_checkpoint``
writes it as a safetensors directory that either loader (ours or the reference's) reads.
"""
from __future__ import annotations

import json
import math
from pathlib import Path
from typing import Callable

import torch

from ..config import LINEAR, ModelConfig

LM = "model.language_model."


def _layer_keys(cfg: ModelConfig, i: int, add: Callable[[str, tuple[int, ...], str], None]) -> None:
    p = f"{LM}layers.{i}."
    H = cfg.hidden_size
    add(p + "input_layernorm.weight", (H,), "norm0")
    add(p + "post_attention_layernorm.weight", (H,), "norm0")
    if cfg.layer_types[i] == LINEAR:
        q = p + "linear_attn."
        add(q + "in_proj_qkv.weight", (cfg.lin_conv_dim, H), "w")
        add(q + "in_proj_z.weight", (cfg.lin_vdim, H), "w")
        add(q + "in_proj_b.weight", (cfg.linear_num_value_heads, H), "w")
        add(q + "in_proj_a.weight", (cfg.linear_num_value_heads, H), "w")
        add(q + "conv1d.weight", (cfg.lin_conv_dim, 1, cfg.linear_conv_kernel_dim), "conv")
        add(q + "A_log", (cfg.linear_num_value_heads,), "alog")
        add(q + "dt_bias", (cfg.linear_num_value_heads,), "dt")
        add(q + "norm.weight", (cfg.linear_value_head_dim,), "norm1")
        add(q + "out_proj.weight", (H, cfg.lin_vdim), "w")
    else:
        q = p + "self_attn."
        add(q + "q_proj.weight", (cfg.num_attention_heads * 2 * cfg.head_dim, H), "w")
        add(q + "k_proj.weight", (cfg.num_key_value_heads * cfg.head_dim, H), "w")
        add(q + "v_proj.weight", (cfg.num_key_value_heads * cfg.head_dim, H), "w")
        add(q + "o_proj.weight", (H, cfg.num_attention_heads * cfg.head_dim), "w")
        add(q + "q_norm.weight", (cfg.head_dim,), "norm0")
        add(q + "k_norm.weight", (cfg.head_dim,), "norm0")
    m = p + "mlp."
    if cfg.is_moe:
        E, I = cfg.num_experts, cfg.moe_intermediate_size
        add(m + "gate.weight", (E, H), "w")
        add(m + "experts.gate_up_proj", (E, 2 * I, H), "w")
        add(m + "experts.down_proj", (E, H, I), "w")
        if cfg.shared_expert_intermediate_size:
            S = cfg.shared_expert_intermediate_size
            add(m + "shared_expert.gate_proj.weight", (S, H), "w")
            add(m + "shared_expert.up_proj.weight", (S, H), "w")
            add(m + "shared_expert.down_proj.weight", (H, S), "w")
            add(m + "shared_expert_gate.weight", (1, H), "w")
    else:
        I = cfg.intermediate_size
        add(m + "gate_proj.weight", (I, H), "w")
        add(m + "up_proj.weight", (I, H), "w")
        add(m + "down_proj.weight", (H, I), "w")


def tensor_plan(cfg: ModelConfig, mtp: bool = False) -> list[tuple[str, tuple[int, ...], str]]:
    """``(key, shape, kind)`` for every tensor of a checkpoint of this geometry."""
    plan: list[tuple[str, tuple[int, ...], str]] = []
    add = lambda k, s, kind: plan.append((k, s, kind))
    add(LM + "embed_tokens.weight", (cfg.vocab_size, cfg.hidden_size), "w")
    for i in range(cfg.num_hidden_layers):
        _layer_keys(cfg, i, add)
    add(LM + "norm.weight", (cfg.hidden_size,), "norm0")
    if not cfg.tie_word_embeddings:
        add("lm_head.weight", (cfg.vocab_size, cfg.hidden_size), "w")
    if mtp:
        H = cfg.hidden_size
        add("mtp.fc.weight", (H, 2 * H), "w")
        add("mtp.pre_fc_norm_embedding.weight", (H,), "norm0")
        add("mtp.pre_fc_norm_hidden.weight", (H,), "norm0")
        q = "mtp.layers.0.self_attn."
        add(q + "q_proj.weight", (cfg.num_attention_heads * 2 * cfg.head_dim, H), "w")
        add(q + "k_proj.weight", (cfg.num_key_value_heads * cfg.head_dim, H), "w")
        add(q + "v_proj.weight", (cfg.num_key_value_heads * cfg.head_dim, H), "w")
        add(q + "o_proj.weight", (H, cfg.num_attention_heads * cfg.head_dim), "w")
        add(q + "q_norm.weight", (cfg.head_dim,), "norm0")
        add(q + "k_norm.weight", (cfg.head_dim,), "norm0")
        add("mtp.layers.0.input_layernorm.weight", (H,), "norm0")
        add("mtp.layers.0.post_attention_layernorm.weight", (H,), "norm0")
        I = cfg.intermediate_size or cfg.shared_expert_intermediate_size
        add("mtp.layers.0.mlp.gate_proj.weight", (I, H), "w")
        add("mtp.layers.0.mlp.up_proj.weight", (I, H), "w")
        add("mtp.layers.0.mlp.down_proj.weight", (H, I), "w")
        add("mtp.norm.weight", (H,), "norm0")
    return plan


def _draw(shape, kind: str, gen: torch.Generator, device, dtype, std: float) -> torch.Tensor:
    if kind == "alog":          # A in [1, 16): per-step decay exp(-A*softplus(.)) stays in (0,1)
        u = torch.rand(shape, generator=gen, device=device, dtype=torch.float32)
        return torch.log(1.0 + 15.0 * u)
    if kind == "dt":
        return torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * 0.5
    t = torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
    if kind == "norm1":         # plain gain around one (gated norm of the delta-net output)
        return (1.0 + std * t).to(dtype)
    if kind == "conv":          # taps large enough that the conv output is not ~0
        return (t * 0.3).to(dtype)
    return (t * std).to(dtype)  # "w" matrices and zero-centred "norm0" gains


def random_state_dict(cfg: ModelConfig, seed: int = 0, dtype: torch.dtype = torch.float32,
                      device: str | torch.device = "cpu", std: float = 0.02,
                      mtp: bool = False) -> dict[str, torch.Tensor]:
    """Draw every tensor of ``tensor_plan``; ``A_log`` and ``dt_bias`` stay fp32.

    Drawn on ``device`` directly so that an 8 GB model does not cross PCIe; the
    generator is seeded per tensor (seed + index) so that any subset (a pipeline stage,
    a tensor-parallel shard source) sees the same values as the whole.
    """
    if getattr(cfg, "architecture", "") == "qwen4_exp":
        from ..models.qwen4exp.weights import random_state_dict as qwen4_random
        return qwen4_random(cfg, seed, dtype=dtype, device=device, std=std)
    sd: dict[str, torch.Tensor] = {}
    dev = torch.device(device)
    for idx, (key, shape, kind) in enumerate(tensor_plan(cfg, mtp)):
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed * 1_000_003 + idx)
        sd[key] = _draw(shape, kind, gen, dev, dtype, std)
    return sd


def param_count(cfg: ModelConfig) -> int:
    return sum(math.prod(s) for _, s, _ in tensor_plan(cfg))


def save_checkpoint(cfg: ModelConfig, sd: dict[str, torch.Tensor], out_dir: str | Path,
                    shard_bytes: int = 4 << 30, split_experts: bool = False) -> Path:
    """Write ``config.json`` + ``model-XXXXX-of-YYYYY.safetensors`` + the shard index.

    ``split_experts`` writes routed experts as per-expert ``experts.{e}.gate_proj.weight``
    keys (the older HF layout) instead of the fused 3-D stacks.
    """
    from safetensors.torch import save_file
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    (out / "config.json").write_text(json.dumps(cfg.to_hf(), indent=1))
    items: list[tuple[str, torch.Tensor]] = []
    for k, v in sd.items():
        if split_experts and k.endswith("experts.gate_up_proj"):
            base = k[: -len("gate_up_proj")]
            I = v.shape[1] // 2
            for e in range(v.shape[0]):
                items.append((f"{base}{e}.gate_proj.weight", v[e, :I].contiguous()))
                items.append((f"{base}{e}.up_proj.weight", v[e, I:].contiguous()))
        elif split_experts and k.endswith("experts.down_proj"):
            base = k[: -len("down_proj")]
            for e in range(v.shape[0]):
                items.append((f"{base}{e}.down_proj.weight", v[e].contiguous()))
        else:
            items.append((k, v.contiguous()))
    shards: list[dict[str, torch.Tensor]] = [{}]
    size = 0
    for k, v in items:
        nb = v.numel() * v.element_size()
        if size and size + nb > shard_bytes:
            shards.append({})
            size = 0
        shards[-1][k] = v.cpu()
        size += nb
    weight_map = {}
    for n, shard in enumerate(shards):
        name = f"model-{n + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(shard, str(out / name))
        weight_map.update({k: name for k in shard})
    (out / "model.safetensors.index.json").write_text(
        json.dumps({"metadata": {}, "weight_map": weight_map}, indent=1))
    return out
