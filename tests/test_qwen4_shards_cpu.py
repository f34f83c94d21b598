"""The n-gram table as the checkpoint stores it (equal row shards, kept as mapped host views) and the loader
that hands those views over (reference: models/qwen4exp/ngram.py:363-470, checkpoint.py:102-160)."""
import dataclasses

import pytest
import torch

from coffin_b200.models.qwen4exp.ngram import NGramTable, ShardedNGramTable


def test_sharded_gather_equals_the_concatenated_table_in_request_order():
    g = torch.Generator().manual_seed(0)
    shards = [torch.randn(50, 8, generator=g).to(torch.bfloat16) for _ in range(7)]
    whole = NGramTable(torch.cat(shards), "cpu")
    table = ShardedNGramTable(shards, "cpu")
    assert table.rows == 350 and table.width == 8
    ids = torch.randint(0, 350, (33, 4), generator=g)
    ids[0] = torch.tensor([349, 0, 50, 49])                      # shard edges
    assert torch.equal(table.gather(ids), whole.gather(ids))
    table.prefetch(ids)
    assert torch.equal(table.take(ids), whole.gather(ids))
    with pytest.raises(ValueError, match="outside"):
        table.gather(torch.tensor([[350]]))
    table.close()
    assert table.shards == []


def test_unequal_or_misplaced_shards_are_refused():
    a, b = torch.zeros(10, 4), torch.zeros(11, 4)
    with pytest.raises(ValueError, match="unequal shards"):
        ShardedNGramTable([a, b], "cpu")
    with pytest.raises(ValueError, match="at least one"):
        ShardedNGramTable([], "cpu")
    with pytest.raises(ValueError, match="unequal shards"):
        ShardedNGramTable([a, a.to(torch.bfloat16)], "cpu")


def _write_sharded_checkpoint(tmp_path, n_shards=4, drop=None):
    from safetensors.torch import save_file
    from coffin_b200.models.qwen4exp.config import preset_qwen4
    from coffin_b200.models.qwen4exp.weights import random_state_dict
    cfg = preset_qwen4("tiny-qwen4")
    sd = random_state_dict(cfg, 0, dtype=torch.bfloat16)
    key = next(k for k in sd if k.endswith("ngram_embedding.weight"))
    table = sd.pop(key)
    assert table.shape[0] % n_shards == 0, table.shape
    per = table.shape[0] // n_shards
    prefix = key[:-len(".weight")]
    main = {k: v.contiguous() for k, v in sd.items() if isinstance(v, torch.Tensor)}
    save_file(main, str(tmp_path / "model-00001-of-00002.safetensors"))
    parts = {f"{prefix}.shard_{k}.weight": table[k * per:(k + 1) * per].contiguous() for k in range(n_shards) if k != drop}
    save_file(parts, str(tmp_path / "model-00002-of-00002.safetensors"))
    return cfg, key, table


def test_loader_maps_the_shards_and_the_plan_counts_them_as_one_table(tmp_path):
    from coffin_b200.models.qwen4exp.weights import ShardList, load_streaming, verify_plan
    cfg, key, table = _write_sharded_checkpoint(tmp_path)
    rep = verify_plan(cfg, tmp_path)
    assert not rep["missing"] and not rep["shape"], rep
    sd = load_streaming(tmp_path, cfg)
    got = sd[key]
    assert isinstance(got, ShardList) and len(got) == 4 and got.shape == tuple(table.shape)
    assert torch.equal(torch.cat(list(got)), table)
    t = ShardedNGramTable(list(got), "cpu", keep=got.keep)
    ids = torch.tensor([[0, table.shape[0] - 1, table.shape[0] // 2]])
    assert torch.equal(t.gather(ids), table[ids[0]].reshape(1, -1))


def test_a_missing_shard_is_reported_not_shifted(tmp_path):
    from coffin_b200.models.qwen4exp.weights import load_streaming, verify_plan
    cfg, key, table = _write_sharded_checkpoint(tmp_path, drop=2)
    rep = verify_plan(cfg, tmp_path)
    assert any(k == key for k, *_ in rep["shape"]), rep
    with pytest.raises(ValueError, match="does not match the tensor plan"):
        load_streaming(tmp_path, cfg)
    with pytest.raises(ValueError, match="are not 0.."):
        load_streaming(tmp_path, cfg, strict=False)


def test_oracle_reads_a_sharded_table(tmp_path):
    from coffin_b200.models.qwen4exp.oracle import Qwen4Oracle
    from coffin_b200.models.qwen4exp.weights import load_streaming, random_state_dict
    cfg, key, table = _write_sharded_checkpoint(tmp_path)
    toks = torch.randint(2, cfg.vocab_size, (12,), generator=torch.Generator().manual_seed(1))
    ref_sd = random_state_dict(cfg, 0, dtype=torch.bfloat16)
    ref = Qwen4Oracle(cfg, ref_sd)
    got = Qwen4Oracle(cfg, load_streaming(tmp_path, cfg))
    a = ref.forward(toks, ref.new_state())
    b = got.forward(toks, got.new_state())
    assert torch.allclose(a, b, atol=1e-5)


def test_staged_check_tool_on_a_sharded_checkpoint(tmp_path, capsys):
    import json
    from coffin_b200.tools import check_qwen4
    cfg, key, table = _write_sharded_checkpoint(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_hf()))
    assert check_qwen4.main(["--model", str(tmp_path), "--stage", "all", "--tokens", "6"]) == 0
    lines = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert [l["stage"] for l in lines] == ["geometry", "layers"]
    assert lines[0]["ok"] and lines[0]["n_missing"] == 0 and lines[0]["files"] == 2
    assert lines[1]["ok"] and lines[1]["finite"] and lines[1]["layers"] == 2 and lines[1]["ple_layers"] == [2]
    # a checkpoint that lost a shard fails at the first stage, with the table named
    bad = tmp_path / "bad"
    bad.mkdir()
    cfg2, key2, _ = _write_sharded_checkpoint(bad, drop=1)
    (bad / "config.json").write_text(json.dumps(cfg2.to_hf()))
    assert check_qwen4.main(["--model", str(bad), "--stage", "all"]) == 1
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rep["stage"] == "geometry" and not rep["ok"] and any(key2 in row[0] for row in rep["shape"])
