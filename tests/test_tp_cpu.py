"""Tensor-parallel sharding algebra on the CPU oracle: the per-rank partial outputs of every
row-parallel projection sum to the unsharded layer output, for worlds that shard the KV heads and
for worlds that replicate them."""
import pytest
import torch

from coffin_b200.config import LINEAR, preset
from coffin_b200.oracle.model import OracleModel
from coffin_b200.parallel.tp import local_config, shard_state_dict
from coffin_b200.weights.init import LM, random_state_dict


@pytest.mark.parametrize("world", [2, 4])
@torch.no_grad()
def test_sharded_partials_sum_to_full(world):
    cfg = preset("tiny")
    sd = random_state_dict(cfg, 0)
    full = OracleModel(cfg, sd)
    lcfg = local_config(cfg, world)
    assert lcfg.num_attention_heads == cfg.num_attention_heads // world
    assert lcfg.num_key_value_heads == max(1, cfg.num_key_value_heads // world)
    shards = [OracleModel(lcfg, shard_state_dict(cfg, sd, r, world)) for r in range(world)]
    T = 9
    h = torch.randn(T, cfg.hidden_size)
    pos = torch.arange(T)
    cos, sin = full._cos_sin(pos, None)
    for i, kind in enumerate(cfg.layer_types):
        st = full.new_state()
        if kind == LINEAR:
            ref = full._linear_attn(i, h, st)
            got = sum(m._linear_attn(i, h, m.new_state()) for m in shards)
        else:
            ref = full._full_attn(i, h, st, cos, sin, pos)
            got = sum(m._full_attn(i, h, m.new_state(), cos, sin, pos) for m in shards)
        assert (ref - got).abs().max() < 1e-4, f"layer {i} ({kind})"
        p = f"{LM}layers.{i}.mlp."
        assert (full._ffn(p, h) - sum(m._ffn(p, h) for m in shards)).abs().max() < 1e-4


def test_indivisible_world_is_rejected():
    with pytest.raises(ValueError):
        local_config(preset("tiny"), 3)
