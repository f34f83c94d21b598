"""Batched speculative verification on the device: ``verify_batch`` over several sequences equals
step-by-step decoding of the same tokens (logits and, after ``commit_batch``, the delta-net states),
for the narrow path (<= 8 token rows) and the wide path (tcgen05 projections), and the engine's
speculative step produces the tokens of plain greedy decoding."""
import pytest
import torch

from coffin_b200.config import preset
from coffin_b200.weights.init import random_state_dict

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max()).item()


@torch.no_grad()
@pytest.mark.parametrize("nrows,C", [(1, 4), (2, 4), (4, 2), (4, 8), (3, 4)])
def test_verify_batch_equals_stepwise_decode(nrows, C):
    from coffin_b200.models.qwen35.model import Qwen35Model
    from coffin_b200.ops import kernels as K
    cfg = preset("tiny")
    sd = random_state_dict(cfg, 0)
    spec = Qwen35Model(cfg, sd, max_seq=512, num_slots=4)
    step = Qwen35Model(cfg, sd, max_seq=512, num_slots=4)
    g = torch.Generator().manual_seed(17 + nrows * 10 + C)
    lens = [37, 64, 50, 71][:nrows]
    seqs = [torch.randint(0, cfg.vocab_size, (n + C,), generator=g) for n in lens]
    tables = [list(range(1 + 8 * r, 9 + 8 * r)) for r in range(nrows)]
    for m in (spec, step):
        for r, s in enumerate(seqs):
            m.zero_state(r)
            m.prefill(s[:lens[r]].cuda(), 0, r, torch.tensor(tables[r], dtype=torch.int32, device="cuda"), want_logits=False)
    rows = [(seqs[r][lens[r]:lens[r] + C].tolist(), lens[r], r, tables[r], 0) for r in range(nrows)]
    logits = spec.verify_batch(rows)
    assert logits.shape[:2] == (nrows, C)
    accept = [(r % C) + 1 for r in range(nrows)]          # a different accepted length per row
    spec.commit_batch(list(range(nrows)), accept)
    for r in range(nrows):
        for j in range(C):
            step.set_rows(1, [int(seqs[r][lens[r] + j])], [lens[r] + j], [r], [tables[r]])
            _, lg = step.decode(1, graph=False)
            assert _rel(logits[r, j], lg[0]) < 4e-2, f"row {r} token {j}"
            if j + 1 == accept[r]:
                # the speculative model's state after committing accept[r] tokens == the stepwise state here
                for li in range(spec.state.shape[0]):
                    # two bf16 pipelines (batched GEMMs vs GEMVs) feed the same fp32 update: a few steps apart by ~2 %
                    assert _rel(spec.state[li, r], step.state[li, r]) < 3e-2, f"row {r} layer {li}"
    torch.cuda.synchronize()
    K.check_status()


@torch.no_grad()
def test_engine_speculative_step_on_the_device():
    from coffin_b200.engine.config import EngineConfig
    from coffin_b200.engine.llm_engine import LLMEngine
    from coffin_b200.engine.sequence import SamplingParams
    from coffin_b200.models.qwen35.model import Qwen35Model
    cfg = preset("tiny")
    sd = random_state_dict(cfg, 0)
    g = torch.Generator().manual_seed(4)
    prompts = []
    for i in range(4):
        unit = torch.randint(0, cfg.vocab_size, (5 + i,), generator=g).tolist()
        prompts.append((unit * 12)[:48 + 3 * i])

    def run(**kw):
        model = Qwen35Model(cfg, sd, max_seq=512, num_slots=4)
        eng = LLMEngine(model, EngineConfig(max_seq=512, max_num_seqs=4, **kw))
        seqs = eng.generate(prompts, SamplingParams(max_tokens=20))
        eng.bm.pool.check()
        return [s.output for s in seqs], eng.runner.stats()

    ref, _ = run()
    got, st = run(spec_k=3, spec_batch=True)
    assert st["spec"]["steps"] > 0 and st["spec"]["drafted"] > 0
    # speculation changes only the speed: tokens agree with plain greedy decoding up to the first
    # position where bf16 rounding of the two paths could flip a near-tie
    same = sum(int(a == b) for a, b in zip(got, ref))
    assert same >= 3, (got, ref)
