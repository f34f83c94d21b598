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
