"""Pipeline parallelism on the CPU twin: two gloo ranks, each owning half of the layers, must
reproduce the single-process logits for chunked prefill and micro-batched decode."""
import os
import socket

import torch

from ranks import run_ranks

RANK_TIMEOUT = 120
RANK_ENV = {"COFFIN_TP_WAIT_MS": "250", "NCCL_NVLS_ENABLE": "0", "COFFIN_RANK_LOG_DIR": os.environ.get("COFFIN_RANK_LOG_DIR", "")}

from coffin_b200.config import preset
from coffin_b200.parallel.pp import layer_range, split_lanes, stage_config, stage_state_dict
from coffin_b200.weights.init import random_state_dict


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_layer_ranges_cover_every_layer_once():
    for n, w in ((32, 4), (7, 3), (4, 4), (48, 5)):
        seen = []
        for s in range(w):
            lo, hi = layer_range(n, s, w)
            seen += list(range(lo, hi))
        assert seen == list(range(n))
    assert split_lanes(5, 2) == [(0, 3), (3, 5)]
    assert split_lanes(1, 2) == [(0, 1)]


def test_stage_state_dict_renumbers_and_keeps_the_right_ends():
    cfg = preset("tiny")
    sd = random_state_dict(cfg, 0)
    lo, hi = layer_range(cfg.num_hidden_layers, 1, 2)
    ssd = stage_state_dict(sd, lo, hi, first=False, last=True)
    sc = stage_config(cfg, lo, hi)
    assert sc.num_hidden_layers == hi - lo and sc.layer_types == tuple(cfg.layer_types[lo:hi])
    assert any(k.startswith("model.language_model.layers.0.") for k in ssd)
    assert not any(f"layers.{hi - lo}." in k for k in ssd)
    assert "model.language_model.embed_tokens.weight" in ssd          # tied head lives on the last stage
    first = stage_state_dict(sd, 0, lo, first=True, last=False)
    assert "model.language_model.embed_tokens.weight" in first


def _scenario(model, cfg):
    """Chunked prefill of two sequences, then four decode steps of both rows."""
    g = torch.Generator().manual_seed(4)
    seqs = [torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in (70, 45)]
    tables = [list(range(1, 5)), list(range(5, 9))]
    outs = []
    toks = []
    for r, s in enumerate(seqs):
        model.zero_state(r)
        bt = torch.tensor(tables[r], dtype=torch.int32)
        model.prefill(s[:32], 0, r, bt, want_logits=False)
        lg = model.prefill(s[32:], 32, r, bt)
        outs.append(lg.clone())
        toks.append(int(lg.argmax()))
    pos = [len(s) for s in seqs]
    for step in range(4):
        model.set_rows(2, toks, pos, [0, 1], tables)
        nxt, lg = model.decode(2, graph=False)
        outs.append(lg[:2].clone())
        toks = [int(t) for t in nxt[:2]]
        pos = [p + 1 for p in pos]
    return outs


def _pp_rank(rank, world, port, path):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from coffin_b200.oracle.engine_model import OracleEngineModel
    from coffin_b200.parallel.pp import build_stage
    cfg = preset("tiny")
    sd = random_state_dict(cfg, 0)
    model = build_stage(cfg, sd, rank, world, lanes=2, factory=OracleEngineModel, max_seq=256, num_slots=2)
    outs = _scenario(model, cfg)
    if rank == 0:
        torch.save({"outs": outs, "relay": model.relay_bytes}, path)
    dist.barrier()
    dist.destroy_process_group()


def test_two_stage_pipeline_matches_single_process(tmp_path):
    from coffin_b200.oracle.engine_model import OracleEngineModel
    cfg = preset("tiny")
    ref = _scenario(OracleEngineModel(cfg, random_state_dict(cfg, 0), max_seq=256, num_slots=2), cfg)
    path = str(tmp_path / "pp.pt")
    run_ranks(_pp_rank, 2, args=(_free_port(), path), timeout=RANK_TIMEOUT, env=RANK_ENV)
    got = torch.load(path)
    assert len(got["outs"]) == len(ref)
    for a, b in zip(got["outs"], ref):
        assert torch.allclose(a, b, atol=1e-4, rtol=1e-4)
    # stage 0 relayed every prefill token and every decode row once: (70 + 45 + 4 * 2) rows of H floats
    assert got["relay"] == (70 + 45 + 8) * cfg.hidden_size * 4
