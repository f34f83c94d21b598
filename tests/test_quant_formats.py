"""Quantised weight containers and the on-disk ``quant_index.json`` formats (both schemes,
dense + MoE kinds): round trip, layout facts, error paths, and the oracle GEMMs."""
import json

import pytest
import torch

from coffin_b200.config import preset
from coffin_b200.oracle import ops as O
from coffin_b200.weights.init import random_state_dict, save_checkpoint
from coffin_b200.weights.loader import load_checkpoint
from coffin_b200.weights.quant import QWeight, W4A8Weight, is_quantizable
from coffin_b200.weights.quant_io import INDEX_NAME, load_quantized, read_index, write_quantized


def test_int8_container():
    w = torch.randn(37, 200)
    q = QWeight.quantize(w)
    assert q.wq.dtype == torch.int8 and q.scale.shape == (37,)
    assert (q.dequant() - w).abs().max() <= q.scale.max() * 0.51
    kn, sc = q.to_kn()
    assert kn.shape == (200, 37) and torch.equal(QWeight.from_kn(kn, sc).wq, q.wq)
    x = torch.randn(5, 200)
    ref = x @ w.t()
    got = O.w8a8_linear(x, q.wq, q.scale)
    assert (got - ref).abs().max() / ref.abs().max() < 0.03


def test_w4a8_container_layout_and_oracle():
    w = torch.randn(24, 300)
    q = W4A8Weight.quantize(w)
    # K is padded to whole groups before packing (3 groups of 128 -> 192 rows), as the reference's writer does
    assert q.packed.shape == (192, 24) and q.scale.shape == (3, 24) and q.k == 300
    codes = q.codes()
    assert codes.shape == (300, 24) and codes.min() >= -8 and codes.max() <= 7
    # low nibble holds even k
    assert int(q.packed[0, 0] & 0xF) - 8 == int(codes[0, 0]) and int(q.packed[0, 0] >> 4) - 8 == int(codes[1, 0])
    assert (q.dequant() - w).abs().max() <= q.scale.max() * 0.51
    x = torch.randn(4, 300)
    got = O.w4a8_linear(x, q.packed, q.scale, q.k)
    ref = x @ q.dequant().t()
    assert (got - ref).abs().max() / ref.abs().max() < 0.03


def test_w4a8_k_not_a_multiple_of_the_group():
    """K = 192: the writer stores ceil(K/128)*64 = 128 packed rows; a tensor of ceil(K/2) = 96 rows
    (the unpadded form) is read as the same weight."""
    from coffin_b200.oracle import ops as O
    w = torch.randn(16, 192)
    q = W4A8Weight.quantize(w)
    assert q.packed.shape == (128, 16) and q.scale.shape == (2, 16)
    assert bool((q.packed[96:] == 0x88).all())                      # padding rows are zero codes
    short = W4A8Weight(q.packed[:96].contiguous(), q.scale, 192)
    assert torch.equal(short.dequant(), q.dequant())
    x = torch.randn(3, 192)
    assert torch.allclose(O.w4a8_linear(x, q.packed, q.scale, q.k), O.w4a8_linear(x, short.packed, short.scale, 192))


@pytest.mark.parametrize("scheme,name", [("int8", "tiny"), ("w4a8", "tiny-moe"), ("int8", "tiny-moe")])
def test_disk_round_trip(tmp_path, scheme, name):
    cfg = preset(name)
    sd = random_state_dict(cfg, 0)
    src = save_checkpoint(cfg, sd, tmp_path / "src", split_experts=(scheme == "int8"))
    dense = load_checkpoint(src)
    assert set(dense) == set(sd)           # per-expert keys are fused back into stacks
    idx = write_quantized(src, dense, tmp_path / "q", scheme=scheme)
    assert (tmp_path / "q" / INDEX_NAME).is_file() and read_index(tmp_path / "q")["format"] == idx["format"]
    assert idx["files"][0].startswith("quant-w4a8-" if scheme == "w4a8" else "quant-0")
    q = load_checkpoint(tmp_path / "q")    # goes through load_quantized
    kinds = idx["kinds"]
    assert kinds.get("dense", 0) > 0 and any(k.startswith("q") for k in kinds)
    for key, t in sd.items():
        v = q[key]
        if is_quantizable(key, t):
            assert isinstance(v, (QWeight, W4A8Weight)), key
            tol = 0.02 if scheme == "int8" else 0.2
            assert (v.dequant() - t).abs().max() <= tol * t.abs().max() + 1e-6
        else:
            assert torch.equal(v, t), key
    if name == "tiny-moe":
        moe_key = next(k for k in idx["tensors"] if k.endswith("gate_up_stack"))
        assert idx["tensors"][moe_key]["kind"] == ("q4-moe" if scheme == "w4a8" else "q8-moe")
        if scheme == "int8":
            assert idx["tensors"][moe_key]["nk_key"].endswith("#nk")
    d = load_quantized(tmp_path / "q", quant=False)
    assert all(isinstance(v, torch.Tensor) for v in d.values())
    # a different config.json is refused
    cfgp = tmp_path / "q" / "config.json"
    cfgp.write_text(cfgp.read_text() + " ")
    with pytest.raises(ValueError, match="config.json"):
        load_quantized(tmp_path / "q")
