"""Speculative decoding on the CPU twin: output equals plain greedy decoding, drafts are accepted
on repetitive text, the delta-net state after a partial acceptance equals the plain state."""
import torch

from coffin_b200.config import preset
from coffin_b200.engine.speculative import SpeculativeDecoder
from coffin_b200.oracle.engine_model import OracleEngineModel
from coffin_b200.oracle.model import OracleModel
from coffin_b200.utils.suffix import SuffixDrafter
from coffin_b200.weights.init import random_state_dict

CFG = preset("tiny")
SD = random_state_dict(CFG, 0)


def test_suffix_drafter_proposes_true_continuations():
    d = SuffixDrafter(max_match=4, min_match=2)
    hist = [5, 6, 7, 8, 9, 5, 6, 7]
    d.observe(hist)
    assert d.draft(3) == [8, 9, 5]
    d.observe([8])
    assert d.draft(2) == [9, 5]
    d.reset()
    assert d.draft(3) == []
    d.observe([1, 2, 3])
    assert d.draft(3) == []


class OracleDrafter:
    """Drafts the true greedy continuation, except every third draft position is corrupted."""

    def __init__(self, truth):
        self.truth, self.n = truth, 0

    def reset(self):
        pass

    def observe(self, toks):
        self.n += len(toks)

    def draft(self, k):
        nxt = self.truth[self.n:self.n + k]
        return [t if (self.n + i) % 3 else (t + 1) % CFG.vocab_size for i, t in enumerate(nxt)]


@torch.no_grad()
def test_speculative_equals_plain_greedy():
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, CFG.vocab_size, (50,), generator=g).tolist()
    n = 20
    plain = OracleModel(CFG, SD).generate(prompt, n)[0]
    model = OracleEngineModel(CFG, SD, max_seq=256, num_slots=1)
    table = list(range(1, 5))
    model.zero_state(0)
    logits = model.prefill(torch.tensor(prompt), 0, 0, torch.tensor(table, dtype=torch.int32))
    drafter = OracleDrafter(prompt + plain)
    sd = SpeculativeDecoder(model, k=3, drafter=drafter)
    drafter.n = 0
    got = sd.generate(prompt, table, logits, n)
    assert got == plain
    st = sd.stats()
    assert st["accepted"] > 0 and st["accepted"] < st["drafted"]
    # state after speculation == state after plain decoding of the same tokens
    ref = OracleEngineModel(CFG, SD, max_seq=256, num_slots=1)
    ref.zero_state(0)
    ref.prefill(torch.tensor(prompt + got[:-1]), 0, 0, torch.tensor(table, dtype=torch.int32), want_logits=False)
    # the speculative model has consumed prompt + all generated tokens but the last one
    assert (model.state - ref.state).abs().max() < 1e-4


def _engine(**kw):
    from coffin_b200.engine.config import EngineConfig
    from coffin_b200.engine.llm_engine import LLMEngine
    model = OracleEngineModel(CFG, SD, max_seq=512, num_slots=4)
    return LLMEngine(model, EngineConfig(max_seq=512, max_num_seqs=4, graph=False, **kw))


def _repetitive(seed: int, n: int = 60) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    unit = torch.randint(0, CFG.vocab_size, (6,), generator=g).tolist()
    return (unit * (n // 6 + 1))[:n]


@torch.no_grad()
def test_engine_speculation_equals_plain_greedy_single_and_batched():
    """``spec_k`` in the engine: the tokens are those of plain greedy decoding, drafts are really
    verified (some accepted), no block leaks, and the counters reach the sequence."""
    from coffin_b200.engine.sequence import SamplingParams
    prompts = [_repetitive(1), _repetitive(2, 45), _repetitive(3, 70)]
    plain = _engine()
    ref = [s.output for s in plain.generate(prompts, SamplingParams(max_tokens=24))]
    # single stream
    eng = _engine(spec_k=3)
    for p, r in zip(prompts, ref):
        s = eng.generate([p], SamplingParams(max_tokens=24))[0]
        assert s.output == r
    st = eng.runner.stats()["spec"]
    assert st["steps"] > 0 and st["drafted"] > 0
    eng.bm.pool.check()
    assert eng.bm.pool.used_blocks == 0 or eng.bm.prefix_cache
    # batched rows, one of them sampling with a temperature (it must not be disturbed by the others' drafts)
    eng = _engine(spec_k=3, spec_batch=True)
    seqs = [eng.add_request(p, SamplingParams(max_tokens=24)) for p in prompts]
    hot = eng.add_request(prompts[0], SamplingParams(max_tokens=10, temperature=0.7, seed=3))
    while any(not s.finished for s in seqs + [hot]):
        eng.step()
    assert [s.output for s in seqs] == ref
    assert len(hot.output) == 10 and hot.spec_drafted == 0
    assert sum(s.spec_accepted for s in seqs) > 0
    assert eng.runner.n_decode_steps < sum(len(r) for r in ref)     # fewer forwards than tokens
    plain_hot = _engine()
    h2 = plain_hot.generate([prompts[0]], SamplingParams(max_tokens=10, temperature=0.7, seed=3))[0]
    assert h2.output == hot.output
    # a request can switch speculation on for itself, or off
    eng = _engine()
    s_on = eng.generate([prompts[0]], SamplingParams(max_tokens=24, spec_k=4))[0]
    assert s_on.output == ref[0] and s_on.spec_steps > 0
    eng = _engine(spec_k=3)
    s_off = eng.generate([prompts[0]], SamplingParams(max_tokens=24, spec_k=0))[0]
    assert s_off.output == ref[0] and s_off.spec_steps == 0


@torch.no_grad()
def test_engine_speculation_stops_at_eos_and_max_tokens():
    from coffin_b200.engine.sequence import SamplingParams
    p = _repetitive(5)
    ref = _engine().generate([p], SamplingParams(max_tokens=30))[0].output
    eos = ref[11]
    cut = ref.index(eos)
    eng = _engine(spec_k=4)
    s = eng.generate([p], SamplingParams(max_tokens=30, eos=(eos,)))[0]
    assert s.output == ref[:cut] and s.finish_reason == "stop"
    s = eng.generate([p], SamplingParams(max_tokens=7))[0]
    assert s.output == ref[:7] and s.finish_reason == "length"
    eng.reset()
    eng.bm.pool.check()


@torch.no_grad()
def test_speculation_survives_preemption_on_a_tight_pool():
    """Three rows that each grow into a third block on a pool of 8: rows are preempted and recomputed while
    the others keep drafting; the tokens stay those of plain greedy decoding and every block comes back."""
    import random
    from coffin_b200.engine.config import EngineConfig
    from coffin_b200.engine.llm_engine import LLMEngine
    from coffin_b200.engine.sequence import SamplingParams
    preempted = 0
    for seed in (0, 4, 9):
        rng = random.Random(seed)
        model = OracleEngineModel(CFG, SD, max_seq=512, num_slots=3, num_blocks=9)
        eng = LLMEngine(model, EngineConfig(max_seq=512, max_num_seqs=3, graph=False, prefix_cache=False, spec_k=3, spec_batch=True))
        prompts = []
        for _ in range(3):
            n = rng.randint(118, 127)
            unit = [rng.randrange(CFG.vocab_size) for _ in range(rng.randint(3, 9))]
            prompts.append((unit * (n // len(unit) + 1))[:n])
        limits = [rng.randint(8, 14) for _ in range(3)]
        seqs = [eng.add_request(p, SamplingParams(max_tokens=n)) for p, n in zip(prompts, limits)]
        for _ in range(3000):
            if all(s.finished for s in seqs):
                break
            eng.step()
            eng.bm.pool.check()
        for p, s, n in zip(prompts, seqs, limits):
            assert s.output == OracleModel(CFG, SD).generate(p, n)[0]
        assert eng.bm.pool.used_blocks == 0 and eng.runner.stats()["spec"]["accepted"] > 0
        preempted += eng.n_preempt
    assert preempted > 0
