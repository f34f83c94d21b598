"""Prefill/decode hand-off through device memory: one buffer + CUDA IPC handle, device-to-device copy.

Same process (pointer used directly) against the file transport, then two processes - the exporter and the
adopter on different GPUs when the box has two (the copy then crosses NVLink), else on the same GPU."""
import json
import os
import time
from pathlib import Path

import pytest
import torch

from coffin_b200.config import preset
from coffin_b200.weights.init import random_state_dict
from ranks import run_ranks

pytestmark = pytest.mark.gpu


def _model(dev="cuda:0", kv_dtype="bf16"):
    from coffin_b200.models.qwen35.model import Qwen35Model
    cfg = preset("tiny")
    return cfg, Qwen35Model(cfg, random_state_dict(cfg, 0), device=dev, max_seq=256, num_slots=2, kv_dtype=kv_dtype)


def _prompt(cfg):
    return torch.randint(0, cfg.vocab_size, (70,), generator=torch.Generator().manual_seed(4)).tolist()


def _decode(model, table, tok, pos, n):
    out = []
    for i in range(n):
        model.set_rows(1, [tok], [pos + i], [0], [table])
        tok = int(model.decode(1, graph=False)[0][0])
        out.append(tok)
    return out


@torch.no_grad()
@pytest.mark.parametrize("kv_dtype", ["bf16", "int8"])
def test_device_transport_equals_file_transport_in_one_process(tmp_path, kv_dtype):
    from coffin_b200.engine import pd
    cfg, src = _model(kv_dtype=kv_dtype)
    prompt = _prompt(cfg)
    table = list(range(1, 4))
    src.zero_state(0)
    logits = src.prefill(torch.tensor(prompt, device="cuda"), 0, 0, torch.tensor(table, dtype=torch.int32, device="cuda"))
    nb = pd.export_state_device(src, 0, table, prompt, logits, tmp_path / "dev")
    assert nb > 0 and json.loads((tmp_path / "dev" / "state.json").read_text())["transport"] == "device"
    pd.export_state(src, 0, table, prompt, logits, tmp_path / "file")
    outs = []
    for d in ("dev", "file"):
        _, dst = _model(kv_dtype=kv_dtype)
        t2, p2, lg = pd.adopt_any(dst, 0, tmp_path / d, first_block=5, max_new=16)
        assert p2 == prompt and torch.equal(lg.cpu(), logits.float().cpu())
        outs.append(_decode(dst, t2, int(lg.argmax()), len(prompt), 8))
    assert outs[0] == outs[1]
    ref = _decode(src, table + [4], int(logits.argmax()), len(prompt), 8)
    assert outs[0] == ref
    assert pd.release_export() and not pd.release_export()


def _pd_rank(rank, world, work):
    """rank 0 exports and waits for the adopter's result file; rank 1 adopts, decodes, writes the tokens."""
    from coffin_b200.engine import pd
    work = Path(work)
    dev = f"cuda:{rank % torch.cuda.device_count()}"
    torch.cuda.set_device(dev)
    cfg, model = _model(dev)
    prompt = _prompt(cfg)
    with torch.no_grad():
        if rank == 0:
            table = list(range(1, 4))
            model.zero_state(0)
            logits = model.prefill(torch.tensor(prompt, device=dev), 0, 0, torch.tensor(table, dtype=torch.int32, device=dev))
            pd.export_state_device(model, 0, table, prompt, logits, work)
            ref = _decode(model, table + [4], int(logits.argmax()), len(prompt), 8)
            (work / "ref.json").write_text(json.dumps(ref))
            t0 = time.time()
            while not (work / "got.json").exists() and time.time() - t0 < 60:
                time.sleep(0.05)
            pd.release_export()
        else:
            t0 = time.time()
            while not (work / "ref.json").exists() and time.time() - t0 < 60:
                time.sleep(0.05)
            table, p2, lg = pd.adopt_any(model, 0, work, first_block=3, max_new=16)
            got = _decode(model, table, int(lg.argmax()), len(p2), 8)
            (work / "got.tmp").write_text(json.dumps({"tokens": got, "prompt_ok": p2 == prompt, "device": dev}))
            os.replace(work / "got.tmp", work / "got.json")
    os._exit(0)


def test_device_transport_between_two_processes(tmp_path):
    run_ranks(_pd_rank, 2, args=(str(tmp_path),), timeout=150)
    got = json.loads((tmp_path / "got.json").read_text())
    assert got["prompt_ok"] and got["tokens"] == json.loads((tmp_path / "ref.json").read_text())
