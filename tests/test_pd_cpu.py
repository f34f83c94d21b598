"""Prefill/decode hand-off on the CPU twin: the checks an adopting instance runs before it touches its pool,
and the merge of per-stage exports of a pipelined prefill (reference: engine/prefix_engine.py:653-874)."""
import copy

import pytest
import torch

from coffin_b200.config import preset
from coffin_b200.engine import pd
from coffin_b200.oracle.engine_model import OracleEngineModel
from coffin_b200.parallel.pp import layer_range, stage_config, stage_state_dict
from coffin_b200.weights.init import random_state_dict


def _twin(cfg, sd, **kw):
    return OracleEngineModel(cfg, sd, max_seq=256, num_slots=2, **kw)


def _prefilled(tmp_path):
    cfg = preset("tiny")
    sd = random_state_dict(cfg, 0)
    src = _twin(cfg, sd)
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, cfg.vocab_size, (70,), generator=g)
    table = list(range(1, 5))
    src.zero_state(0)
    logits = src.prefill(prompt, 0, 0, torch.tensor(table, dtype=torch.int32))
    pd.export_state(src, 0, table, prompt.tolist(), logits, tmp_path / "whole")
    return cfg, sd, src, prompt, table, logits


def _decode(model, table, tok, pos, n=4):
    out = []
    for i in range(n):
        model.set_rows(1, [tok], [pos + i], [0], [table])
        nxt, lg = model.decode(1, graph=False)
        out.append(lg[0].clone())
        tok = int(nxt[0])
    return out


def test_adopted_state_continues_like_the_source(tmp_path):
    cfg, sd, src, prompt, table, logits = _prefilled(tmp_path)
    dst = _twin(cfg, sd)
    t2, p2, lg2 = pd.adopt_state(dst, 0, tmp_path / "whole", first_block=3)
    assert p2 == prompt.tolist() and torch.equal(lg2, logits.float())
    tok = int(logits.argmax())
    for a, b in zip(_decode(src, table, tok, 70), _decode(dst, t2, tok, 70)):
        assert torch.allclose(a, b, atol=1e-5)


def test_foreign_state_is_refused_before_the_pool_is_touched(tmp_path):
    cfg, sd, src, prompt, table, logits = _prefilled(tmp_path)
    good = torch.load(tmp_path / "whole" / "state.pt", weights_only=False)
    dst = _twin(cfg, sd)
    before = dst.kpool.clone()

    def broken(edit):
        p = copy.deepcopy(good)
        edit(p)
        return p

    cases = [
        (lambda p: p.pop("state"), KeyError, "missing"),
        (lambda p: p["meta"].update(layer_begin=0, layer_end=2), ValueError, "pipeline split"),
        (lambda p: p["meta"].update(block=32), ValueError, "block size"),
        (lambda p: p["meta"].update(nkv=p["meta"]["nkv"] + 1), ValueError, "KV heads"),
        (lambda p: p["meta"].update(kv_dtype="torch.int8"), ValueError, "KV dtype"),
        (lambda p: p.update(n=p["n"] - 1), ValueError, "disagrees with itself"),
        (lambda p: p.update(k=p["k"][:, :-1]), ValueError, "k: shape"),
        (lambda p: p["state"].__setitem__(0, p["state"][0][:, :1]), ValueError, "recurrent state 0"),
        (lambda p: p.update(logits=p["logits"][:-1]), ValueError, "vocabulary"),
    ]
    for edit, exc, text in cases:
        with pytest.raises(exc, match=text):
            pd.adopt_payload(dst, 0, broken(edit))
        assert torch.equal(dst.kpool, before), text
    small = OracleEngineModel(cfg, sd, max_seq=64, num_slots=1)
    with pytest.raises(ValueError, match="max_seq"):
        pd.adopt_payload(small, 0, copy.deepcopy(good))


def test_exports_of_two_pipeline_stages_merge_into_the_whole_model(tmp_path):
    cfg, sd, src, prompt, table, logits = _prefilled(tmp_path)
    bt = torch.tensor(table, dtype=torch.int32)
    stages, hidden = [], None
    for s in range(2):
        lo, hi = layer_range(cfg.num_hidden_layers, s, 2)
        m = _twin(stage_config(cfg, lo, hi), stage_state_dict(sd, lo, hi, first=s == 0, last=s == 1), pp_first=s == 0, pp_last=s == 1)
        assert pd.layer_span(m) == (lo, hi)
        m.zero_state(0)
        lg = m.prefill(prompt, 0, 0, bt, embeds=hidden)
        hidden = m.last_prenorm
        pd.export_state(m, 0, table, prompt.tolist(), lg, tmp_path / f"stage{s}")
        stages.append(m)
    assert torch.allclose(lg, logits, atol=1e-4)
    dst = _twin(cfg, sd)
    t2, p2, lg2 = pd.adopt_merged(dst, 0, [tmp_path / "stage1", tmp_path / "stage0"], first_block=2)     # any order
    assert p2 == prompt.tolist()
    tok = int(logits.argmax())
    for a, b in zip(_decode(src, table, tok, 70), _decode(dst, t2, tok, 70)):
        assert torch.allclose(a, b, atol=1e-4)
    # a part alone does not fit the whole model, parts that leave a gap or disagree do not merge
    part0 = torch.load(tmp_path / "stage0" / "state.pt", weights_only=False)
    part1 = torch.load(tmp_path / "stage1" / "state.pt", weights_only=False)
    with pytest.raises(ValueError, match="pipeline split"):
        pd.adopt_payload(_twin(cfg, sd), 0, part1)
    with pytest.raises(ValueError, match="do not join"):
        pd.merge_parts([part0, part0])
    both = copy.deepcopy(part0)
    both["logits"] = part1["logits"].clone()
    with pytest.raises(ValueError, match="carry logits"):
        pd.merge_parts([both, part1])
    gap = copy.deepcopy(part1)
    gap["meta"]["layer_begin"] += 1
    with pytest.raises(ValueError, match="do not join"):
        pd.merge_parts([part0, gap])
    other = copy.deepcopy(part1)
    other["prompt"][0] ^= 1
    with pytest.raises(ValueError, match="different prompts"):
        pd.merge_parts([part0, other])


def test_read_back_after_adopt_reports_no_mismatch_and_sees_a_damaged_row(tmp_path, monkeypatch, capsys):
    cfg, sd, src, prompt, table, logits = _prefilled(tmp_path)
    dst = _twin(cfg, sd)
    monkeypatch.setenv("COFFIN_PD_TRACE", "1")
    monkeypatch.setenv("COFFIN_PD_VERIFY", "1")
    t2, _, _ = pd.adopt_state(dst, 0, tmp_path / "whole", first_block=3)
    said = capsys.readouterr().out
    assert "[pd] adopt slot=0 pos=70" in said
    lines = [ln for ln in said.splitlines() if ln.startswith("[pdverify]")]
    assert lines and all("mismatch=0/" in ln for ln in lines)
    payload = torch.load(tmp_path / "whole" / "state.pt", map_location="cpu", weights_only=False)
    dst.kpool[0, t2[0] * pd.BLOCK + 5] += 1.0                       # one KV row of layer 0 damaged after the write
    after = pd.verify_adopted(dst, 0, t2, payload)
    bad = [ln for ln in after if "mismatch=0/" not in ln]
    assert len(bad) == 1 and bad[0].startswith("[pdverify] k layer=0")
