"""Qwen4-exp family on the CPU: config round trip, n-gram hashing, oracle self-consistency."""
import pytest
import torch

from coffin_b200.models.qwen4exp.config import Qwen4Config, tiny_qwen4
from coffin_b200.models.qwen4exp.ngram import NGramHasher, NGramTable, is_prime, layer_multipliers, splitmix64
from coffin_b200.models.qwen4exp.oracle import Qwen4Oracle, qsa_select
from coffin_b200.models.qwen4exp.weights import param_count, random_state_dict, tensor_plan


def test_config_round_trip_and_derived_fields():
    cfg = tiny_qwen4()
    assert cfg.layer_types.count("indexed_attention") == 2 and cfg.block_topk == 4
    assert cfg.ple_index(1) == 0 and cfg.ple_index(0) is None
    again = Qwen4Config.from_hf(cfg.to_hf(), name=cfg.name)
    for f in ("layer_types", "hc_count", "indexer_budget", "ple_layer_ids", "mrope_section", "rotary_dim", "ngram_heads"):
        assert getattr(again, f) == getattr(cfg, f), f
    assert param_count(cfg) == sum(torch.Size(s).numel() for _, s, _ in tensor_plan(cfg))


def test_ngram_hash_properties():
    assert splitmix64(0) == 0xE220A8397B1DCDAF            # published test vector of the generator
    m = layer_multipliers(1024, 3, 0, 1234)
    assert all(v % 2 == 1 and v > 0 for v in m) and len(set(m)) == 3
    cfg = tiny_qwen4()
    h = NGramHasher(cfg, 0)
    assert all(is_prime(s) and s >= cfg.ngram_vocab_size_base for s in h.sizes) and len(set(h.sizes)) == h.heads
    ids = h.ids([5, 9, 9, 5, 1, 5, 9], None)
    assert ids.shape == (7, h.heads)
    for j in range(h.heads):
        assert (ids[:, j] >= h.offsets[j]).all() and (ids[:, j] < h.offsets[j] + h.sizes[j]).all()
    # same 3-gram -> same rows; history does not cross the end-of-sequence token (id 1)
    a = h.ids([7, 5, 9], None)[2]
    b = h.ids([3, 3, 7, 5, 9], None)[4]
    assert torch.equal(a, b)
    after_eos = h.ids([5, 9, 1, 9], None)[3]
    fresh = h.ids([9], None)[0]
    assert torch.equal(after_eos, fresh)
    # incremental hashing with a carried context equals hashing the whole history
    whole = h.ids([4, 8, 15, 16, 23], None)
    step = h.ids([16, 23], [8, 15])
    assert torch.equal(whole[3:], step)


def test_ngram_table_gather_on_cpu():
    w = torch.arange(40, dtype=torch.float32).reshape(10, 4)
    t = NGramTable(w, "cpu")
    ids = torch.tensor([[0, 9], [3, 3]])
    assert torch.equal(t.gather(ids), torch.cat([w[0], w[9], w[3], w[3]]).reshape(2, 8))


def test_block_selection_rule():
    cfg = tiny_qwen4()                       # ratio 4, topk 4, full-select factor 2
    g = torch.Generator().manual_seed(0)
    iq = torch.randn(cfg.indexer_n_heads, cfg.indexer_head_dim, generator=g)
    bk = torch.randn(30, cfg.indexer_head_dim, generator=g)
    assert qsa_select(iq, bk, 35, cfg).all()                       # 8 blocks <= 2 * topk: everything
    keep = qsa_select(iq, bk, 103, cfg)                            # 25 blocks + 3 tail tokens
    assert keep[100:].all() and int(keep.sum()) == 4 * 4 + 3
    s = torch.relu(iq @ bk[:25].t()).sum(0)
    best = int(s.argmax())
    assert keep[best * 4:(best + 1) * 4].all()


def test_oracle_chunked_and_incremental_equal_one_shot():
    cfg = tiny_qwen4()
    sd = random_state_dict(cfg, 0)
    o = Qwen4Oracle(cfg, sd)
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, cfg.vocab_size, (80,), generator=g)
    toks[30] = cfg.eos_token_id
    full = o.forward(toks, o.new_state())
    st = o.new_state()
    parts = [o.forward(toks[:33], st), o.forward(toks[33:72], st)] + [o.forward(toks[i:i + 1], st) for i in range(72, 80)]
    assert torch.allclose(torch.cat(parts), full, atol=2e-5)
    assert o.last_selected[7].shape == (1, 80) and int(o.last_selected[7].sum()) == 16     # sparse at 80 tokens
    # a cloned state continues identically
    st2 = o.new_state()
    o.forward(toks[:40], st2)
    st3 = st2.clone()
    assert torch.equal(o.forward(toks[40:50], st2), o.forward(toks[40:50], st3))


def test_streaming_loader_plan_check_and_expert_parallel_reads(tmp_path):
    """Shard index -> plan check without reading data -> shard-by-shard reads; an expert-parallel rank
    reads only its expert range (fused stacks through ``get_slice``, per-expert files by name) and the MoE
    module takes the pre-cut stack as it is; a checkpoint that does not match the plan is refused."""
    import torch
    from coffin_b200.models.qwen4exp.config import tiny_qwen4
    from coffin_b200.models.qwen4exp.weights import (checkpoint_index, load_streaming, random_state_dict, tensor_plan,
                                                    verify_plan)
    from coffin_b200.weights.init import save_checkpoint
    cfg = tiny_qwen4()
    sd = random_state_dict(cfg, 0)
    E = cfg.num_experts
    for split in (False, True):
        d = save_checkpoint(cfg, sd, tmp_path / f"ck{int(split)}", split_experts=split, shard_bytes=1 << 20)
        idx = checkpoint_index(d)
        assert len(set(idx.values())) > 1                       # really sharded
        rep = verify_plan(cfg, d, idx)
        assert rep == {"missing": [], "unexpected": [], "shape": []}
        full = load_streaming(d)
        assert set(full) == {k for k, _, _ in tensor_plan(cfg)}
        for r in range(2):
            part = load_streaming(d, ep=(r, 2))
            assert part["__ep_shard__"] == (r, 2)
            for k, v in sd.items():
                if k.endswith(("experts.gate_up_proj", "experts.down_proj")):
                    assert torch.equal(part[k], v[r * E // 2:(r + 1) * E // 2]), k
                else:
                    assert torch.equal(part[k], v), k
    # a checkpoint of another geometry is refused before any data is read
    other = tiny_qwen4(hidden_size=256)
    assert verify_plan(other, d)["shape"]
    import pytest
    with pytest.raises(ValueError, match="tensor plan"):
        load_streaming(d, cfg=other)


def test_qwen4_quantiser_streams_and_round_trips(tmp_path):
    """``tools/quant_disk_qwen4``: per-expert source files are fused per layer while streaming, the chosen
    families are quantised (hyper-connection, PLE, router and embedding stay dense), the index has the
    shared formats and the loader hands back containers whose dequantised values track the source."""
    import torch
    from coffin_b200.models.qwen4exp.config import tiny_qwen4
    from coffin_b200.models.qwen4exp.weights import random_state_dict
    from coffin_b200.tools.quant_disk_qwen4 import main as quantise
    from coffin_b200.weights.init import save_checkpoint
    from coffin_b200.weights.loader import load_checkpoint
    from coffin_b200.weights.quant import QWeight, W4A8Weight
    from coffin_b200.weights.quant_io import read_index
    cfg = tiny_qwen4()
    sd = random_state_dict(cfg, 0)
    src = save_checkpoint(cfg, sd, tmp_path / "src", split_experts=True, shard_bytes=1 << 20)
    for scheme, cls, tol in (("int8", QWeight, 0.02), ("w4a8", W4A8Weight, 0.2)):
        out = tmp_path / scheme
        assert quantise(["--model", str(src), "--out", str(out), "--scheme", scheme, "--shard-gb", "0.001"]) == 0
        idx = read_index(out)
        assert len(idx["files"]) > 1 and idx["generated_by"].endswith("quant_disk_qwen4.py")
        back = load_checkpoint(out)
        assert set(back) == set(sd)
        n_q = 0
        for k, v in back.items():
            if isinstance(v, (QWeight, W4A8Weight)):
                n_q += 1
                assert isinstance(v, cls) and "hyper_connection" not in k and ".ple." not in k
                assert (v.dequant() - sd[k]).abs().max() <= tol * sd[k].abs().max() + 1e-6, k
            else:
                assert torch.equal(v, sd[k]), k
        assert n_q > 3 * cfg.num_hidden_layers
    assert not list((tmp_path / "w4a8").glob("*.tmp"))


def _greedy(o, prompt, n):
    st = o.new_state()
    out = [int(o.forward(torch.tensor(prompt), st)[-1].argmax())]
    while len(out) < n:
        out.append(int(o.forward(torch.tensor(out[-1:]), st)[-1].argmax()))
    return out


def test_draft_head_plan_has_the_checkpoint_tensor_count_and_config_guard():
    cfg = tiny_qwen4(mtp_num_hidden_layers=1)
    names = [k for k, _, _ in tensor_plan(cfg) if k.startswith("mtp.")]
    # 2 projections + 2 pre-norms + 3 final-mixer tensors + one QSA/MoE layer (9 + 7 + 2 x 4): the 31
    # ``mtp.*`` tensors of a checkpoint of the family
    assert len(names) == 31
    assert "mtp.layers.0.self_attn.indexer.index_qk_proj.weight" in names
    assert not any("block_inject" in k for k in names if k.startswith("mtp.hyper_connection_mixer."))
    shapes = {k: s for k, s, _ in tensor_plan(cfg)}
    assert shapes["mtp.pre_fc_norm_hidden.weight"] == (cfg.hc_hidden,) and shapes["mtp.fc_hidden.weight"] == (cfg.hidden_size,) * 2
    with pytest.raises(ValueError, match="exactly one layer"):
        tiny_qwen4(mtp_num_hidden_layers=2)


def test_oracle_speculative_decoding_with_the_draft_head_equals_greedy():
    """Random weights accept nothing, so a hook feeds partly correct drafts: 0, 1, 2 and all accepted
    drafts per round, with and without block-selection reuse along the chain."""
    from coffin_b200.models.qwen4exp.oracle import DraftIndexPlan
    cfg = tiny_qwen4(mtp_num_hidden_layers=1)
    o = Qwen4Oracle(cfg, random_state_dict(cfg, 0))
    assert o.has_mtp
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab_size, (50,), generator=g).tolist()       # 50 tokens: 12 blocks > 2 x 4, selection is sparse
    ref = _greedy(o, prompt, 24)
    out, stats = o.spec_generate(prompt, 24, k=3)
    assert out == ref and stats["drafted"] == 3 * stats["rounds"]
    rounds = []

    def hook(position, drafts):
        i = position - len(prompt)                      # index in ``ref`` of the first draft
        good = len(rounds) % 4                          # 0, 1, 2, 3 correct drafts in turn
        rounds.append(good)
        return [ref[i + j] if j < good and i + j < len(ref) else (drafts[j] + 1) % cfg.vocab_size for j in range(3)]

    for reuse in (True, False):
        rounds.clear()
        out, stats = o.spec_generate(prompt, 24, k=3, index_reuse=reuse, draft_hook=hook)
        assert out == ref, reuse
        assert stats["accepted"] > 0 and (stats["index_reuse"] > 0) == reuse
    # the plan refuses a negative step and re-selects after a block boundary
    plan = DraftIndexPlan()
    with pytest.raises(ValueError):
        plan.before_step(-1)
    keep = torch.ones(12, dtype=torch.bool)
    plan.record(keep, 11, cfg)                          # 3 complete blocks at position 11 (ratio 4)
    assert plan.before_step(1) is not None
    assert plan.keep_rows(plan.blocks, torch.tensor([13]), 14, cfg) is not None
    assert plan.keep_rows(plan.blocks, torch.tensor([15]), 16, cfg) is None      # a fourth block completed


def test_lazy_random_state_dict_draws_the_same_tensors_one_at_a_time():
    from coffin_b200.models.qwen4exp.weights import LazyRandomStateDict
    cfg = tiny_qwen4(mtp_num_hidden_layers=1)
    full = random_state_dict(cfg, 3, dtype=torch.bfloat16)
    lazy = LazyRandomStateDict(cfg, 3, device="cpu")
    assert set(lazy.keys()) == set(full) and "lm_head.weight" in lazy and "nope" not in lazy
    assert lazy.get("nope", 7) == 7
    assert all(torch.equal(full[k], lazy[k]) for k in full)


def test_qwen4_quantiser_writes_per_rank_trees_with_manifest_and_resumes(tmp_path, capsys):
    """``--layout ep2``: one loadable directory per expert-parallel rank holding only that rank's experts, a
    manifest at the top (not loadable, says so), progress after every rank directory; a second run finds the
    finished directories and writes nothing again, a run that lost one directory rewrites just that one."""
    import json
    import shutil

    import pytest
    from coffin_b200.models.qwen4exp.config import tiny_qwen4
    from coffin_b200.models.qwen4exp.weights import random_state_dict
    from coffin_b200.tools.quant_disk_qwen4 import PROGRESS_NAME, main as quantise
    from coffin_b200.weights.init import save_checkpoint
    from coffin_b200.weights.quant import W4A8Weight
    from coffin_b200.weights.quant_io import MANIFEST_FORMAT, load_quantized, read_index
    cfg = tiny_qwen4()
    sd = random_state_dict(cfg, 0)
    src = save_checkpoint(cfg, sd, tmp_path / "src", split_experts=True, shard_bytes=1 << 20)
    out = tmp_path / "tree"
    assert quantise(["--model", str(src), "--out", str(out), "--scheme", "w4a8", "--layout", "ep2", "--verify"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["format"] == MANIFEST_FORMAT and rep["resumed_units"] == [] and rep["worst_relative_error"] < 0.2
    man = json.loads((out / "quant_index.json").read_text())
    assert man["complete"] and man["world"] == {"ep2": 2} and sorted(man["rank_dirs"]["ep2"]) == ["0", "1"]
    with pytest.raises(ValueError, match="manifest of a per-rank tree"):
        read_index(out)
    E = cfg.num_experts
    for r in range(2):
        back = load_quantized(out / man["rank_dirs"]["ep2"][str(r)])
        assert back["__ep_shard__"] == (r, 2)
        stacks = [k for k in back if k.endswith(("experts.gate_up_proj", "experts.down_proj"))]
        assert stacks and all(isinstance(back[k], W4A8Weight) and back[k].dequant().shape[0] == E // 2 for k in stacks)
        k0 = stacks[0]
        ref = sd[k0][r * (E // 2):(r + 1) * (E // 2)]
        assert (back[k0].dequant() - ref).abs().max() <= 0.2 * ref.abs().max()
    prog = json.loads((out / PROGRESS_NAME).read_text())
    assert sorted(prog["done"]) == ["ep2/rank-0", "ep2/rank-1"]
    # resume: nothing is rewritten
    stamp = (out / "ep2" / "rank-0" / "quant_index.json").stat().st_mtime_ns
    assert quantise(["--model", str(src), "--out", str(out), "--scheme", "w4a8", "--layout", "ep2"]) == 0
    assert json.loads(capsys.readouterr().out)["resumed_units"] == ["ep2/rank-0", "ep2/rank-1"]
    assert (out / "ep2" / "rank-0" / "quant_index.json").stat().st_mtime_ns == stamp
    # a lost rank directory is rewritten, the other one is kept
    shutil.rmtree(out / "ep2" / "rank-1")
    assert quantise(["--model", str(src), "--out", str(out), "--scheme", "w4a8", "--layout", "ep2"]) == 0
    assert json.loads(capsys.readouterr().out)["resumed_units"] == ["ep2/rank-0"]
    assert load_quantized(out / "ep2" / "rank-1")["__ep_shard__"] == (1, 2)
    with pytest.raises(ValueError, match="only expert-parallel trees"):
        quantise(["--model", str(src), "--out", str(tmp_path / "t2"), "--layout", "tp4"])
