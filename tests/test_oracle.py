"""The CPU oracle is self-consistent: chunked == recurrent delta rule, split prefill ==
one-shot prefill, incremental decode == full forward."""
import torch

from coffin_b200.config import preset
from coffin_b200.oracle import ops as O
from coffin_b200.oracle.model import OracleModel
from coffin_b200.weights.init import random_state_dict


def _toks(cfg, n, seed=1):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg.vocab_size, (n,), generator=g)


@torch.no_grad()
def test_chunked_matches_recurrent_and_split_prefill():
    for name in ("tiny", "tiny-moe"):
        cfg = preset(name)
        sd = random_state_dict(cfg, 0)
        toks = _toks(cfg, 150)
        a, b = OracleModel(cfg, sd), OracleModel(cfg, sd, chunked_gdn=True)
        sa, sb, sc = a.new_state(), b.new_state(), a.new_state()
        la, lb = a.forward(toks, sa), b.forward(toks, sb)
        lc = torch.cat([a.forward(toks[:70], sc), a.forward(toks[70:], sc)])
        assert (la - lb).abs().max() < 1e-4
        assert (la - lc).abs().max() < 1e-4
        for i in sa.rec:
            assert (sa.rec[i] - sb.rec[i]).abs().max() < 1e-4


@torch.no_grad()
def test_decode_matches_full_forward():
    cfg = preset("tiny")
    m = OracleModel(cfg, random_state_dict(cfg, 0))
    toks = _toks(cfg, 40)
    full = m.forward(toks, m.new_state())
    st = m.new_state()
    rows = [m.forward(toks[:32], st)[-1]] + [m.forward(toks[i:i + 1], st)[-1] for i in range(32, 40)]
    assert (torch.stack(rows) - full[31:]).abs().max() < 1e-4


def test_delta_commit_replays_record():
    torch.manual_seed(0)
    nv, dk, dv, T = 3, 8, 8, 5
    q, k = torch.randn(T, nv, dk), torch.randn(T, nv, dk)
    v, b, g = torch.randn(T, nv, dv), torch.rand(T, nv), -torch.rand(T, nv)
    st = torch.randn(nv, dk, dv)
    base = st.clone()
    rec = [O.delta_step(q[t], k[t], v[t], b[t], g[t], st)[1:] for t in range(T)]
    mid = base.clone()
    for t in range(3):
        O.delta_step(q[t], k[t], v[t], b[t], g[t], mid)
    got = O.delta_commit(base, [r[0] for r in rec], [r[1] for r in rec], [r[2] for r in rec], 3)
    assert (got - mid).abs().max() < 1e-5


def test_mrope_equals_1d_table_for_text():
    cos, sin = O.rope_tables(64, 1e7, 50)
    pos = torch.arange(50)
    c3, s3 = O.mrope_cos_sin(pos.reshape(1, -1).expand(3, -1), 64, 1e7)
    assert torch.equal(cos, c3) and torch.equal(sin, s3)
    p3 = torch.stack([pos, pos + 3, pos + 7])
    c4, _ = O.mrope_cos_sin(p3, 64, 1e7)
    assert not torch.equal(c4, cos)
