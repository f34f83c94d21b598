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


def _same(a, b) -> bool:
    from coffin_b200.weights.quant import QWeight, W4A8Weight
    if isinstance(a, QWeight):
        return isinstance(b, QWeight) and torch.equal(a.wq, b.wq) and torch.equal(a.scale, b.scale)
    if isinstance(a, W4A8Weight):
        return isinstance(b, W4A8Weight) and a.k == b.k and torch.equal(a.codes(), b.codes()) and torch.equal(a.scale, b.scale)
    return torch.equal(a, b)


@pytest.mark.parametrize("scheme", ["none", "int8", "w4a8"])
@torch.no_grad()
def test_rank_sliced_reads_equal_slicing_the_full_checkpoint(tmp_path, scheme):
    """Two ranks read a (pre-quantised) checkpoint directory with ``tp=(rank, 2)``: each gets exactly
    the slices that ``shard_state_dict`` cuts from the whole state dict, for dense tensors, int8
    containers (column cuts keep the row scales) and int4 containers (cuts on group boundaries); the
    sliced int8 partial products still sum to the unsharded product; a pipeline stage reads only its layers."""
    from coffin_b200.parallel.tp import TP_MARK
    from coffin_b200.weights.init import save_checkpoint
    from coffin_b200.weights.loader import load_checkpoint
    from coffin_b200.weights.quant import QWeight, W4A8Weight
    from coffin_b200.weights.quant_io import write_quantized
    cfg = preset("tiny")
    sd = random_state_dict(cfg, 0)
    src = save_checkpoint(cfg, sd, tmp_path / "src")
    path = src
    if scheme != "none":
        write_quantized(src, load_checkpoint(src), tmp_path / "q", scheme=scheme)
        path = tmp_path / "q"
    full = load_checkpoint(path)
    world = 2
    parts = []
    for r in range(world):
        got = load_checkpoint(path, tp=(r, world))
        assert got[TP_MARK] == (r, world)
        ref = shard_state_dict(cfg, full, r, world)
        assert shard_state_dict(cfg, got, r, world).keys() == ref.keys()       # a marked dict passes through
        with pytest.raises(ValueError):
            shard_state_dict(cfg, got, 1 - r, world)
        for k, v in ref.items():
            assert _same(got[k], v), k
        parts.append(got)
    if scheme == "int8":
        key = f"{LM}layers.0.mlp.down_proj.weight"
        x = torch.randn(3, cfg.intermediate_size)
        half = cfg.intermediate_size // 2
        whole = x @ full[key].dequant().t()
        summed = sum(x[:, r * half:(r + 1) * half] @ parts[r][key].dequant().t() for r in range(world))
        assert (whole - summed).abs().max() < 1e-4
        assert isinstance(parts[0][key], QWeight)
    if scheme == "w4a8":
        assert isinstance(parts[0][f"{LM}layers.0.mlp.down_proj.weight"], W4A8Weight)
    stage = load_checkpoint(path, layers=(2, 4))
    assert any(k.startswith(f"{LM}layers.2.") for k in stage) and not any(k.startswith(f"{LM}layers.0.") for k in stage)
    assert f"{LM}embed_tokens.weight" in stage and f"{LM}norm.weight" in stage


def test_single_process_all_reduce_contract():
    """One process, several ranks: every rank receives the same rank-ordered sum; mismatched inputs are
    refused (the device path is exercised on a multi-GPU box)."""
    from coffin_b200.parallel.peer_allreduce import PeerAllReduce
    ar = PeerAllReduce(["cpu", "cpu", "cpu"])
    xs = [torch.randn(4, 8).to(torch.bfloat16) for _ in range(3)]
    out = ar.all_reduce(xs)
    ref = (xs[0].float() + xs[1].float() + xs[2].float()).to(torch.bfloat16)
    assert all(torch.equal(o, ref) for o in out)
    ar.all_reduce(xs, out=xs)                      # in place
    assert all(torch.equal(x, ref) for x in xs)
    with pytest.raises(ValueError):
        ar.all_reduce(xs[:2])
    with pytest.raises(ValueError):
        ar.all_reduce([xs[0], xs[1], xs[2].float()])
    with pytest.raises(ValueError):
        ar.all_reduce([x.to(torch.int32) for x in xs])
    with pytest.raises(ValueError):
        PeerAllReduce([0, 0])
