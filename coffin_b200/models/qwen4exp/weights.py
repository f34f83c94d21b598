"""Tensor plan and random initialisation of a Qwen4-exp checkpoint.

Key names are the ``model.language_model.*`` checkpoint names of the family (module tree of the
reference: ``models/qwen4exp/blocks.py:52-110`` for a layer, ``gated_residual.py:66-90`` for a
hyper-connection, ``qsa.py:436-460`` for the indexer, ``ngram.py:759-790`` for a PLE layer,
``model.py:250-262`` for the stem and the final mixer).  The model has no pre-norms and no final
norm: every normalisation sits inside a hyper-connection.
"""
from __future__ import annotations

import math

import torch

from ...weights.init import _draw
from .config import LINEAR, Qwen4Config
from .ngram import NGramHasher

LM = "model.language_model."


def _hyper(prefix: str, cfg: Qwen4Config, add, write_gate: bool = True) -> None:
    W, R = cfg.hc_hidden, cfg.hc_lowrank
    add(prefix + "hc_norm.weight", (W,), "norm0")
    add(prefix + "input_mix_weight_down.weight", (R, W), "w")
    add(prefix + "input_mix_weight_up.weight", (W, R), "wide")
    if write_gate:
        add(prefix + "block_inject_weight.weight", (cfg.hc_count, W), "w")


def tensor_plan(cfg: Qwen4Config) -> list[tuple[str, tuple[int, ...], str]]:
    plan: list[tuple[str, tuple[int, ...], str]] = []
    add = lambda k, s, kind: plan.append((k, s, kind))
    H = cfg.hidden_size
    add(LM + "embed_tokens.weight", (cfg.vocab_size, H), "w")
    for i, kind in enumerate(cfg.layer_types):
        p = f"{LM}layers.{i}."
        if kind == LINEAR:
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
            nh, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
            add(q + "q_proj.weight", (nh * 2 * hd, H), "w")
            add(q + "k_proj.weight", (nkv * hd, H), "w")
            add(q + "v_proj.weight", (nkv * hd, H), "w")
            add(q + "o_proj.weight", (H, nh * hd), "w")
            add(q + "q_norm.weight", (hd,), "norm0")
            add(q + "k_norm.weight", (hd,), "norm0")
            add(q + "indexer.index_qk_proj.weight", ((cfg.indexer_n_heads + 1) * cfg.indexer_head_dim, H), "w")
            add(q + "indexer.q_layernorm.weight", (cfg.indexer_head_dim,), "norm0")
            add(q + "indexer.k_layernorm.weight", (cfg.indexer_head_dim,), "norm0")
        m = p + "mlp."
        E, I, S = cfg.num_experts, cfg.moe_intermediate_size, cfg.shared_expert_intermediate_size
        add(m + "gate.weight", (E, H), "wide")
        add(m + "experts.gate_up_proj", (E, 2 * I, H), "w")
        add(m + "experts.down_proj", (E, H, I), "w")
        add(m + "shared_expert.gate_proj.weight", (S, H), "w")
        add(m + "shared_expert.up_proj.weight", (S, H), "w")
        add(m + "shared_expert.down_proj.weight", (H, S), "w")
        add(m + "shared_expert_gate.weight", (1, H), "w")
        _hyper(p + "attn_hyper_connection.", cfg, add)
        _hyper(p + "mlp_hyper_connection.", cfg, add)
        j = cfg.ple_index(i)
        if j is not None:
            q = p + "ple."
            rows = NGramHasher(cfg, j).rows
            add(q + "ple_embedding.ngram_embedding.weight", (rows, cfg.ngram_head_dim), "wide")
            add(q + "key_proj.weight", (cfg.hc_hidden, cfg.ple_embed_dim), "wide")
            add(q + "value_proj.weight", (H, cfg.ple_embed_dim), "wide")
            for n in ("norm_key", "norm_query", "norm_conv"):
                add(q + n + ".weight", (cfg.hc_hidden,), "norm0")
            add(q + "conv1d.weight", (cfg.hc_hidden, 1, cfg.ple_conv_kernel_size), "conv")
    _hyper(LM + "hyper_connection_mixer.", cfg, add, write_gate=False)
    if not cfg.tie_word_embeddings:
        add("lm_head.weight", (cfg.vocab_size, H), "w")
    return plan


def random_state_dict(cfg: Qwen4Config, seed: int = 0, dtype: torch.dtype = torch.float32,
                      device: str | torch.device = "cpu", std: float = 0.02) -> dict[str, torch.Tensor]:
    """Every tensor of ``tensor_plan``.  "wide" matrices (router, read-gate up-projection, PLE
    projections) are drawn ten times wider so that gates and routing are not degenerate at the
    tiny test widths; the generator is seeded per tensor."""
    sd: dict[str, torch.Tensor] = {}
    dev = torch.device(device)
    for idx, (key, shape, kind) in enumerate(tensor_plan(cfg)):
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed * 1_000_003 + idx)
        if kind == "wide":
            sd[key] = _draw(shape, "w", gen, dev, dtype, std * 10)
        else:
            sd[key] = _draw(shape, kind, gen, dev, dtype, std)
    return sd


def param_count(cfg: Qwen4Config) -> int:
    return sum(math.prod(s) for _, s, _ in tensor_plan(cfg))
