"""The persistent decode kernel (one cooperative launch per step) against the multi-kernel step and
the fp32 CPU oracle: every bucket of 1..8 rows, padded rows, CUDA graphs, the in-step token feedback,
the tensor-parallel exchange on one GPU (world 1), 4B-shaped layers, a bounded barrier that runs
out, and bit-equal results when the same step is run twice."""
import dataclasses

import pytest
import torch

from coffin_b200.config import ModelConfig, preset
from coffin_b200.oracle.model import OracleModel
from coffin_b200.weights.init import random_state_dict

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _mega_on(monkeypatch):
    """The persistent kernel is opt-in (``COFFIN_MEGA=1``); these tests switch it on."""
    from coffin_b200.models.qwen35 import mega
    monkeypatch.setattr(mega, "ENABLED", True)


@pytest.fixture(params=[0, 2])
def ring(request, monkeypatch):
    from coffin_b200.models.qwen35 import mega
    monkeypatch.setattr(mega, "RING", request.param)
    return request.param


def _models(cfg, sd, **kw):
    from coffin_b200.models.qwen35.model import Qwen35Model
    a = Qwen35Model(cfg, sd, max_seq=512, num_slots=8, **kw)
    b = Qwen35Model(cfg, sd, max_seq=512, num_slots=8, **kw)
    b.use_mega = False
    return a, b


def _close(got, ref, atol, rtol):
    """Per-element check: |got - ref| <= atol + rtol * |ref| everywhere."""
    got, ref = got.float().cpu(), ref.float().cpu()
    bad = (got - ref).abs() > atol + rtol * ref.abs()
    assert not bool(bad.any()), f"{int(bad.sum())} of {bad.numel()} elements off; worst {float((got - ref).abs().max()):.4g}"


@torch.no_grad()
def test_mega_step_matches_multi_kernel_step_every_bucket(ring):
    from coffin_b200.ops import kernels as K
    cfg = preset("tiny")
    sd = random_state_dict(cfg, 0)
    mega, plain = _models(cfg, sd)
    g = torch.Generator().manual_seed(3)
    lens = [40, 70, 33, 64, 21, 90, 55, 47]
    seqs = [torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in lens]
    tables = [list(range(1 + 8 * r, 9 + 8 * r)) for r in range(8)]
    for m in (mega, plain):
        for r, s in enumerate(seqs):
            m.zero_state(r)
            m.prefill(s.cuda(), 0, r, torch.tensor(tables[r], dtype=torch.int32, device="cuda"), want_logits=False)
    assert mega._mega_for(1) is not None, "the tiny model must qualify for the persistent kernel"
    pos = list(lens)
    for M, nrows in ((1, 1), (2, 2), (4, 3), (8, 8), (8, 5)):
        for step in range(3):
            toks = [int(torch.randint(0, cfg.vocab_size, (1,), generator=g)) for _ in range(nrows)]
            outs = []
            for m in (mega, plain):
                m.set_rows(M, toks, pos[:nrows], list(range(nrows)), tables[:nrows])
                nxt, lg = m.decode(M, graph=step >= 1)
                outs.append((nxt[:nrows].clone(), lg[:nrows].clone()))
            _close(outs[0][1], outs[1][1], atol=3e-2, rtol=3e-2)
            # arg-max agrees wherever the margin is clear
            top2 = outs[1][1].float().topk(2, dim=-1).values
            clear = (top2[:, 0] - top2[:, 1]) > 0.1
            assert torch.equal(outs[0][0][clear], outs[1][0][clear])
            # the kernel's own arg-max is the arg-max of its own logits
            assert torch.equal(outs[0][0], outs[0][1].argmax(-1))
            for r in range(nrows):
                pos[r] += 1
    assert mega.launches_per_step(1) == 1 and plain.launches_per_step(1) > 10
    torch.cuda.synchronize()
    K.check_status()


@torch.no_grad()
def test_mega_greedy_run_with_in_step_feedback_matches_oracle():
    """Prompt 64, then greedy steps that feed themselves (``advance``): teacher-forced against the
    oracle the tokens agree wherever the oracle's margin is clear, and positions advance on the device."""
    from coffin_b200.models.qwen35.model import Qwen35Model
    cfg = preset("tiny")
    sd = random_state_dict(cfg, 0)
    sd_b = {k: (v.to(torch.bfloat16).float() if v.dtype == torch.float32 and not k.endswith(("A_log", "dt_bias")) else v)
            for k, v in sd.items()}
    oracle = OracleModel(cfg, sd_b)
    model = Qwen35Model(cfg, sd, max_seq=512, num_slots=2)
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, cfg.vocab_size, (64,), generator=g)
    st = oracle.new_state()
    ref = oracle.forward(prompt, st)[-1]
    bt = list(range(8))
    model.zero_state(0)
    model.prefill(prompt.cuda(), 0, 0, torch.tensor(bt, dtype=torch.int32, device="cuda"))
    tok = int(ref.argmax())
    model.set_rows(1, [tok], [64], [0], [bt])
    for i in range(24):
        ref = oracle.forward(torch.tensor([tok]), st)[-1]
        nxt, lg = model.decode(1, graph=True, advance=True)
        rel = ((lg[0].float().cpu() - ref).abs().max() / ref.abs().max()).item()
        assert rel < 6e-2, f"step {i}: {rel}"
        b = model._row_buffers(1)
        assert int(b["positions"][0]) == 65 + i and int(b["tokens"][0]) == int(nxt[0])
        top2 = ref.topk(2).values
        tok = int(nxt[0])
        if top2[0] - top2[1] > 0.05:
            assert tok == int(ref.argmax()), f"step {i}"
        else:
            # follow the kernel's choice so both sides keep seeing the same sequence
            pass
    assert model.launches_per_step(1) == 1


@torch.no_grad()
def test_mega_tensor_parallel_exchange_on_one_gpu_and_run_twice_bit_equal():
    """World 1 with the exchange forced on: every row-parallel projection stores into this rank's own
    inbox and pulls it back, the arg-max goes through the inbox too.  The same step from the same
    state gives bit-identical logits (fixed summation order, no atomics on data)."""
    from coffin_b200.models.qwen35.model import Qwen35Model
    from coffin_b200.parallel.tp import TpComm
    cfg = preset("tiny")
    sd = random_state_dict(cfg, 0)
    plain = Qwen35Model(cfg, sd, max_seq=256, num_slots=2)
    plain.use_mega = False
    tp = TpComm(0, 1, cfg.hidden_size, 8, 2 * cfg.num_hidden_layers + 2)
    fused = Qwen35Model(cfg, sd, max_seq=256, num_slots=2, tp=tp)
    fused.tp_force = True
    assert fused._mega_for(1) is not None
    g = torch.Generator().manual_seed(2)
    toks = torch.randint(0, cfg.vocab_size, (40,), generator=g)
    bt = torch.arange(1, 5, dtype=torch.int32, device="cuda")
    for m in (plain, fused):
        m.zero_state(0)
        m.prefill(toks[:32].cuda(), 0, 0, bt, want_logits=False)
    snap = fused.snapshot_state(0)
    runs = []
    for rep in range(2):
        fused.restore_state(0, snap)
        lgs = []
        for i in range(32, 36):
            fused.set_rows(1, [int(toks[i])], [i], [0], [bt.tolist()])
            nxt, lg = fused.decode(1, graph=i >= 34)
            lgs.append(lg[0].clone())
            assert int(nxt[0]) == int(lg[0].argmax())
        runs.append(torch.stack(lgs))
    assert torch.equal(runs[0], runs[1]), "the persistent kernel must be deterministic"
    for j, i in enumerate(range(32, 36)):
        plain.set_rows(1, [int(toks[i])], [i], [0], [bt.tolist()])
        ref = plain.decode(1, graph=False)[1][0]
        _close(runs[0][j], ref, atol=3e-2, rtol=3e-2)
    torch.cuda.synchronize()
    assert tp.status() == 0
    tp.close()


@torch.no_grad()
def test_layers_of_the_4b_shape_match_the_oracle():
    """Four layers (three delta-net, one attention) with the 4B geometry - hidden 2560, head_dim 256,
    delta-net key/value head dims 128, 12 352-wide fused input projection - through both decode paths
    against the fp32 oracle, per element."""
    from coffin_b200.models.qwen35.model import Qwen35Model
    full = preset("qwen35-4b")
    cfg = dataclasses.replace(full, name="4b-4layers", num_hidden_layers=4, layer_types=full.layer_types[:4], vocab_size=4096)
    sd = random_state_dict(cfg, 0)
    sd_b = {k: (v.to(torch.bfloat16).float() if v.dtype == torch.float32 and not k.endswith(("A_log", "dt_bias")) else v)
            for k, v in sd.items()}
    oracle = OracleModel(cfg, sd_b)
    g = torch.Generator().manual_seed(7)
    toks = torch.randint(0, cfg.vocab_size, (80,), generator=g)
    st = oracle.new_state()
    ref_pre = oracle.forward(toks[:72], st)[-1]
    refs = [oracle.forward(toks[i:i + 1], st)[-1] for i in range(72, 80)]
    scale = float(ref_pre.abs().max())
    bt = torch.arange(0, 4, dtype=torch.int32, device="cuda")
    for use_mega in (True, False):
        model = Qwen35Model(cfg, sd, max_seq=256, num_slots=1)
        model.use_mega = use_mega
        model.zero_state(0)
        got = model.prefill(toks[:72].cuda(), 0, 0, bt)
        _close(got, ref_pre, atol=0.03 * scale, rtol=0.05)
        if use_mega:
            assert model._mega_for(1) is not None
        for j, i in enumerate(range(72, 80)):
            model.set_rows(1, [int(toks[i])], [i], [0], [bt.tolist()])
            _, lg = model.decode(1, graph=j >= 4)
            _close(lg[0], refs[j], atol=0.03 * scale, rtol=0.05)
        del model
        torch.cuda.empty_cache()


@torch.no_grad()
def test_mega_barrier_that_cannot_complete_runs_out_and_reports(monkeypatch):
    """The barrier counter's starting value is set so that the first target is never reached (a flag
    that nothing sets): the kernel must give up after the shortened limit, report 48 through the status
    word, skip every later wait and return; after a reset the next step is correct."""
    import time
    from coffin_b200.models.qwen35.model import Qwen35Model
    from coffin_b200.ops import _lib, kernels as K
    monkeypatch.setenv("COFFIN_MEGA_WAIT_MS", "30")
    cfg = preset("tiny")
    sd = random_state_dict(cfg, 0)
    model = Qwen35Model(cfg, sd, max_seq=256, num_slots=1)
    ref_model = Qwen35Model(cfg, sd, max_seq=256, num_slots=1)
    ref_model.use_mega = False
    g = torch.Generator().manual_seed(11)
    toks = torch.randint(0, cfg.vocab_size, (34,), generator=g)
    bt = torch.arange(1, 5, dtype=torch.int32, device="cuda")
    for m in (model, ref_model):
        m.zero_state(0)
        m.prefill(toks[:32].cuda(), 0, 0, bt, want_logits=False)
    assert model._mega_for(1) is not None
    snap = model.snapshot_state(0)
    model.mega.bar[1] = 1 << 20              # the kernel believes the counter starts far above its real value
    model.set_rows(1, [int(toks[32])], [32], [0], [bt.tolist()])
    t0 = time.perf_counter()
    model.decode(1, graph=False)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 2.0
    K.poll_status()
    torch.cuda.synchronize()
    with pytest.raises(_lib.KernelError, match="role 48"):
        K.raise_on_status()
    model.mega.reset()
    model.restore_state(0, snap)
    model.set_rows(1, [int(toks[32])], [32], [0], [bt.tolist()])
    _, lg = model.decode(1, graph=False)
    ref_model.set_rows(1, [int(toks[32])], [32], [0], [bt.tolist()])
    _, ref = ref_model.decode(1, graph=False)
    _close(lg[0], ref[0], atol=3e-2, rtol=3e-2)
    torch.cuda.synchronize()
    K.check_status()
