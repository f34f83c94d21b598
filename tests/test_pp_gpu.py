"""Two pipeline stages on two GPUs (NCCL point-to-point relay) against the fp32 oracle."""
import os
import socket

import pytest
import torch

from ranks import run_ranks

RANK_TIMEOUT = 150
RANK_ENV = {"COFFIN_TP_WAIT_MS": "250", "NCCL_NVLS_ENABLE": "0", "COFFIN_RANK_LOG_DIR": os.environ.get("COFFIN_RANK_LOG_DIR", "")}

from coffin_b200.config import preset
from coffin_b200.oracle.model import OracleModel
from coffin_b200.weights.init import random_state_dict

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from coffin_b200.models import build_model
    cfg = preset("tiny")
    sd = random_state_dict(cfg, 0)
    dev = f"cuda:{rank}"
    model = build_model(cfg, sd, device=dev, max_seq=256, num_slots=2, pp_world=world, pp_rank=rank)
    g = torch.Generator().manual_seed(2)
    seqs = [torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in (84, 50)]
    tables = [list(range(1, 5)), list(range(5, 9))]
    logits = []
    for r, s in enumerate(seqs):
        model.zero_state(r)
        bt = torch.tensor(tables[r], dtype=torch.int32, device=dev)
        model.prefill(s[:40].to(dev), 0, r, bt, want_logits=False)
        logits.append(model.prefill(s[40:-6].to(dev), 40, r, bt).float().cpu())
    for i in range(6):
        toks = [int(s[len(s) - 6 + i]) for s in seqs]
        pos = [len(s) - 6 + i for s in seqs]
        model.set_rows(2, toks, pos, [0, 1], tables)
        _, lg = model.decode(2, graph=i >= 2)
        logits.append(lg[:2].float().cpu().clone())
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        torch.save(logits, out)
    from coffin_b200.parallel.control import shutdown
    comm = getattr(model, "tp", None)
    if hasattr(model, "_graphs"):
        model._graphs.clear()
    if comm is not None:
        comm.close()
    print("teardown finished" if shutdown(timeout_s=10.0, hard_exit=False) else "teardown did not finish: leaving", flush=True)
    os._exit(0)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_stage_pipeline_matches_oracle(tmp_path):
    out = str(tmp_path / "pp.pt")
    run_ranks(_rank_main, 2, args=(_free_port(), out), timeout=RANK_TIMEOUT, env=RANK_ENV)
    got = torch.load(out)
    cfg = preset("tiny")
    sd = random_state_dict(cfg, 0)
    sd_b = {k: (v.to(torch.bfloat16).float() if not k.endswith(("A_log", "dt_bias")) else v) for k, v in sd.items()}
    oracle = OracleModel(cfg, sd_b)
    g = torch.Generator().manual_seed(2)
    seqs = [torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in (84, 50)]
    states = [oracle.new_state() for _ in seqs]
    for r, s in enumerate(seqs):
        ref = oracle.forward(s[:-6], states[r])[-1]
        rel = ((got[r] - ref).abs().max() / ref.abs().max()).item()
        assert rel < 4e-2, (r, rel)
    for i in range(6):
        for r, s in enumerate(seqs):
            ref = oracle.forward(s[len(s) - 6 + i:len(s) - 5 + i], states[r])[-1]
            rel = ((got[2 + i][r] - ref).abs().max() / ref.abs().max()).item()
            assert rel < 5e-2, (i, r, rel)
