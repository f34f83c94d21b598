"""Qwen4-exp family on the GPU: hyper-connection and QSA kernels against the fp32 oracle functions,
then the whole model (prefill + decode) against ``Qwen4Oracle``."""
import math

import pytest
import torch

from coffin_b200.models.qwen4exp.config import tiny_qwen4
from coffin_b200.models.qwen4exp.oracle import (Qwen4Oracle, grouped_rms_norm, hyper_read, hyper_write,
                                                qsa_block_keys, qsa_select)
from coffin_b200.models.qwen4exp.weights import random_state_dict
from coffin_b200.oracle import ops as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return ((a.float().cpu() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6)).item()


@pytest.mark.parametrize("M", [1, 3, 8])
def test_hyper_connection_kernels(M):
    from coffin_b200.ops import kernels as K
    cfg = tiny_qwen4(hidden_size=256, hc_lowrank=64)
    H, hc, R = cfg.hidden_size, cfg.hc_count, cfg.hc_lowrank
    g = torch.Generator().manual_seed(M)
    bf = lambda *s, sc=1.0: (torch.randn(*s, generator=g) * sc).to(torch.bfloat16)
    p = {"hc_norm.weight": torch.randn(hc * H, generator=g) * 0.1,
         "input_mix_weight_down.weight": bf(R, hc * H, sc=0.05).float(),
         "input_mix_weight_up.weight": bf(hc * H, R, sc=0.3).float(),
         "block_inject_weight.weight": bf(hc, hc * H, sc=0.05).float()}
    x, out, inj = bf(M, hc * H), bf(M, H), torch.rand(M, hc, generator=g) * 2
    # oracle: write back the pending mixer output, then read
    xw = hyper_write(x.float(), out.float(), inj, cfg).to(torch.bfloat16)
    n_ref = grouped_rms_norm(xw, p["hc_norm.weight"], H, cfg.rms_norm_eps)
    mixed_ref, inject_ref = hyper_read(xw.float(), p, "", cfg)
    stream, normed = x.to(DEV).clone(), torch.empty(M, hc * H, dtype=torch.bfloat16, device=DEV)
    K.hyper_norm(stream, (1 + p["hc_norm.weight"]).to(DEV), normed, H=H, hc=hc, eps=cfg.rms_norm_eps,
                 block_out=out.to(DEV), inject=inj.to(DEV))
    assert _rel(stream, xw) < 1e-2 and _rel(normed, n_ref) < 2e-2
    low = torch.empty(M, R, dtype=torch.float32, device=DEV)
    K.gemv(p["input_mix_weight_down.weight"].to(DEV, torch.bfloat16), normed, low)
    mixed = torch.empty(M, H, dtype=torch.bfloat16, device=DEV)
    inject = torch.empty(M, hc, dtype=torch.float32, device=DEV)
    K.hyper_up(normed, low, p["input_mix_weight_up.weight"].to(DEV, torch.bfloat16),
               p["block_inject_weight.weight"].to(DEV, torch.bfloat16), mixed, inject, H=H, hc=hc)
    assert _rel(mixed, mixed_ref) < 3e-2
    assert _rel(inject, inject_ref) < 2e-2


def test_qsa_index_kernels_and_selection():
    from coffin_b200.ops import kernels as K
    cfg = tiny_qwen4()
    ni, di, ratio, rot, topk = cfg.indexer_n_heads, cfg.indexer_head_dim, cfg.indexer_compress_ratio, cfg.rotary_dim, cfg.block_topk
    T = 150
    g = torch.Generator().manual_seed(3)
    proj = torch.randn(T, (ni + 1) * di + 8, generator=g).to(torch.bfloat16)
    qw, kw = torch.randn(di, generator=g) * 0.1, torch.randn(di, generator=g) * 0.1
    cos, sin = O.rope_tables(rot, cfg.rope_theta, 256)
    # oracle
    iq_ref = O.apply_rope(O.rms_norm(proj[:, 8:8 + ni * di].float().reshape(T, ni, di), 1 + qw, cfg.rms_norm_eps), cos[:T], sin[:T], rot)
    raw = proj[:, 8 + ni * di:].float()
    bk_ref = qsa_block_keys(raw, kw, cos, sin, ratio, rot, cfg.rms_norm_eps)
    # device: pages 3, 1, 2 hold tokens 0..63, 64..127, 128..191
    pages = torch.tensor([3, 1, 2], dtype=torch.int32, device=DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    kv_slot = (pages.long()[pos.long() // 64] * 64 + pos.long() % 64).to(torch.int32)
    iq = torch.empty(T, ni, di, dtype=torch.float32, device=DEV)
    ipool = torch.zeros(4 * 64, di, dtype=torch.bfloat16, device=DEV)
    K.qsa_index_prep(proj.to(DEV), 8, (1 + qw).to(DEV), cos.to(DEV), sin.to(DEV), pos, kv_slot, iq, ipool,
                     ni=ni, di=di, rot=rot, eps=cfg.rms_norm_eps)
    assert _rel(iq, iq_ref) < 1e-2
    assert torch.equal(ipool[kv_slot.long()].cpu(), proj[:, 8 + ni * di:])
    per_page = 64 // ratio
    bkpool = torch.zeros(4 * per_page, di, dtype=torch.float32, device=DEV)
    K.qsa_block_keys(ipool, bkpool, (1 + kw).to(DEV), cos.to(DEV), sin.to(DEV), pages, 0, T // ratio,
                     ratio=ratio, di=di, rot=rot, eps=cfg.rms_norm_eps)
    nb = T // ratio
    blk_rows = torch.tensor([int(pages[b // per_page]) * per_page + b % per_page for b in range(nb)])
    got_bk = bkpool[blk_rows.to(DEV)].cpu()
    assert _rel(got_bk, bk_ref) < 2e-2
    # selection on the device block keys (so that both sides rank identical numbers)
    rows = torch.tensor([10, 40, 99, 149], dtype=torch.int32, device=DEV)
    sel = torch.zeros(4, topk, dtype=torch.int32, device=DEV)
    nsel = torch.zeros(4, dtype=torch.int32, device=DEV)
    scores = torch.zeros(4, 64, dtype=torch.float32, device=DEV)
    mask = torch.zeros(4, 2, dtype=torch.int32, device=DEV)
    K.qsa_select(iq[rows.long()].contiguous(), bkpool, pages, rows, scores, sel, nsel, ni=ni, di=di, ratio=ratio,
                 topk=topk, full_factor=cfg.full_select_factor, mask=mask, shared_table=True)
    for i, p in enumerate(rows.tolist()):
        keep = qsa_select(iq[p].cpu(), got_bk, p + 1, cfg)
        nblk = (p + 1) // ratio
        if nblk <= topk * cfg.full_select_factor:
            assert int(nsel[i]) == -1 and int(mask[i, 0]) == -1
            continue
        want = [b for b in range(nblk) if keep[b * ratio]]
        assert int(nsel[i]) == topk and sel[i].tolist() == want
        bits = (int(mask[i, 0]) & 0xffffffff) | ((int(mask[i, 1]) & 0xffffffff) << 32)
        assert [b for b in range(64) if bits >> b & 1] == want


@torch.no_grad()
def test_qwen4_model_prefill_and_decode_match_oracle():
    from coffin_b200.models.qwen4exp.model import Qwen4ExpModel
    cfg = tiny_qwen4()
    sd = random_state_dict(cfg, 0)
    sd_b = {k: (v.to(torch.bfloat16).float() if not k.endswith(("A_log", "dt_bias")) else v) for k, v in sd.items()}
    oracle = Qwen4Oracle(cfg, sd_b)
    model = Qwen4ExpModel(cfg, sd, max_seq=256, num_slots=2)
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, cfg.vocab_size, (112,), generator=g)
    toks[40] = cfg.eos_token_id
    st = oracle.new_state()
    bt = torch.arange(1, 5, dtype=torch.int32, device=DEV)
    model.zero_state(0)
    # two chunks: the second one crosses into the sparse regime (more than 8 blocks of 4 tokens)
    model.prefill(toks[:30].to(DEV), 0, 0, bt, want_logits=False)
    got = model.prefill(toks[30:100].to(DEV), 30, 0, bt)
    ref = oracle.forward(toks[:100], st)[-1]
    assert _rel(got, ref) < 8e-2
    for i in range(100, 112):
        ref = oracle.forward(toks[i:i + 1], st)[-1]
        model.set_rows(1, [int(toks[i])], [i], [0], [bt.tolist()])
        _, logits = model.decode(1)
        assert _rel(logits[0], ref) < 8e-2, f"step {i}"
    from coffin_b200.ops import kernels as K
    torch.cuda.synchronize()
    K.check_status()


@torch.no_grad()
def test_qwen4_batched_decode_and_state_snapshot():
    from coffin_b200.models.qwen4exp.model import Qwen4ExpModel
    cfg = tiny_qwen4()
    sd = random_state_dict(cfg, 0)
    model = Qwen4ExpModel(cfg, sd, max_seq=256, num_slots=3)
    g = torch.Generator().manual_seed(5)
    seqs = [torch.randint(2, cfg.vocab_size, (n,), generator=g) for n in (70, 45)]
    tables = [list(range(1, 5)), list(range(5, 9))]
    single = []
    for r, s in enumerate(seqs):
        model.zero_state(r)
        bt = torch.tensor(tables[r], dtype=torch.int32, device=DEV)
        model.prefill(s[:-1].to(DEV), 0, r, bt, want_logits=False)
    snaps = [model.snapshot_state(r) for r in range(2)]
    # both rows in one batched step
    model.set_rows(2, [int(s[-1]) for s in seqs], [len(s) - 1 for s in seqs], [0, 1], tables)
    _, lg = model.decode(2)
    batched = lg[:2].clone()
    # the same rows one at a time from the restored states
    for r, s in enumerate(seqs):
        model.restore_state(r, snaps[r])
        model.set_rows(1, [int(s[-1])], [len(s) - 1], [r], [tables[r]])
        _, lg1 = model.decode(1)
        single.append(lg1[0].clone())
    for r in range(2):
        assert _rel(batched[r], single[r].cpu()) < 2e-2


@torch.no_grad()
@pytest.mark.parametrize("quant,tol", [("int8", 0.12), ("w4a8", 0.35)])
def test_qwen4_quantised_projections_follow_the_dense_model(quant, tol):
    """``quant``: mixer projections, experts and the head in int8 / int4 storage (``Proj`` of the reference)
    against the bf16 model on the same prompt - the error is the quantisation error, not a kernel bug:
    logits stay close and the greedy token agrees where the bf16 margin is clear."""
    from coffin_b200.models.qwen35.model import QW, QW4
    from coffin_b200.models.qwen4exp.model import Qwen4ExpModel
    cfg = tiny_qwen4()
    sd = random_state_dict(cfg, 0)
    dense = Qwen4ExpModel(cfg, sd, max_seq=256, num_slots=1)
    qm = Qwen4ExpModel(cfg, sd, max_seq=256, num_slots=1, quant=quant)
    assert isinstance(qm.layers[0].w_in, QW if quant == "int8" else QW4)
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(2, cfg.vocab_size, (60,), generator=g)
    bt = torch.arange(1, 5, dtype=torch.int32, device=DEV)
    outs = []
    for m in (dense, qm):
        m.zero_state(0)
        lg = [m.prefill(toks[:50].to(DEV), 0, 0, bt).clone()]
        for i in range(50, 56):
            m.set_rows(1, [int(toks[i])], [i], [0], [bt.tolist()])
            lg.append(m.decode(1)[1][0].clone())
        outs.append(torch.stack(lg))
    assert torch.isfinite(outs[1]).all()
    assert _rel(outs[1], outs[0].cpu()) < tol


@torch.no_grad()
def test_qwen4_runs_from_a_prequantised_directory_with_int8_embedding(tmp_path):
    """The family's quantiser output (int8, embedding included) loads into the device model: containers
    arrive as ``QWeight``, the embedding as int8 rows + scales, and decoding tracks the bf16 model."""
    from coffin_b200.config import load_config
    from coffin_b200.models.qwen4exp.model import QuantEmbedding, Qwen4ExpModel
    from coffin_b200.tools.quant_disk_qwen4 import main as quantise
    from coffin_b200.weights.init import save_checkpoint
    from coffin_b200.weights.loader import load_checkpoint
    cfg = tiny_qwen4()
    sd = random_state_dict(cfg, 0)
    src = save_checkpoint(cfg, {k: v.to(torch.bfloat16) if v.is_floating_point() and not k.endswith(("A_log", "dt_bias")) else v
                                for k, v in sd.items()}, tmp_path / "src")
    assert quantise(["--model", str(src), "--out", str(tmp_path / "q"), "--scheme", "int8", "--quant-embed"]) == 0
    qsd = load_checkpoint(tmp_path / "q")
    qm = Qwen4ExpModel(load_config(tmp_path / "q"), qsd, max_seq=256, num_slots=1)
    assert isinstance(qm.embed, QuantEmbedding)
    dense = Qwen4ExpModel(cfg, sd, max_seq=256, num_slots=1)
    g = torch.Generator().manual_seed(2)
    toks = torch.randint(2, cfg.vocab_size, (40,), generator=g)
    bt = torch.arange(1, 5, dtype=torch.int32, device=DEV)
    a = dense.prefill(toks.to(DEV), 0, 0, bt)
    b = qm.prefill(toks.to(DEV), 0, 0, bt)
    assert _rel(b, a.cpu()) < 0.15


@torch.no_grad()
def test_qwen4_verify_and_commit_follow_sequential_decode():
    """A verify pass of 4 tokens gives the logits of four sequential decode steps; committing the first
    ``n`` leaves the delta-net states and the n-gram window exactly where ``n`` decode steps leave them
    (the next decode step agrees)."""
    from coffin_b200.models.qwen4exp.model import Qwen4ExpModel
    cfg = tiny_qwen4()
    sd = random_state_dict(cfg, 0)
    seq_model = Qwen4ExpModel(cfg, sd, max_seq=256, num_slots=1)
    ver_model = Qwen4ExpModel(cfg, sd, max_seq=256, num_slots=1)
    g = torch.Generator().manual_seed(4)
    toks = torch.randint(2, cfg.vocab_size, (80,), generator=g)
    bt = torch.arange(1, 5, dtype=torch.int32, device=DEV)
    for m in (seq_model, ver_model):
        m.zero_state(0)
        m.prefill(toks[:60].to(DEV), 0, 0, bt, want_logits=False)
    ref = []
    for i in range(60, 64):
        seq_model.set_rows(1, [int(toks[i])], [i], [0], [bt.tolist()])
        ref.append(seq_model.decode(1)[1][0].clone())
    got = ver_model.verify(toks[60:64].tolist(), 60, 0, bt)
    for j in range(4):
        assert _rel(got[j], ref[j].cpu()) < 3e-2, j
    assert ver_model.verify_lanes().shape == (4, cfg.hc_hidden)
    # accept two of the four; both models then decode position 62 again with another token
    ver_model.commit(0, 2)
    seq2 = Qwen4ExpModel(cfg, sd, max_seq=256, num_slots=1)
    seq2.zero_state(0)
    seq2.prefill(toks[:60].to(DEV), 0, 0, bt, want_logits=False)
    for i in (60, 61):
        seq2.set_rows(1, [int(toks[i])], [i], [0], [bt.tolist()])
        seq2.decode(1)
    outs = []
    for m in (seq2, ver_model):
        m.set_rows(1, [int(toks[70])], [62], [0], [bt.tolist()])
        outs.append(m.decode(1)[1][0].clone())
    assert _rel(outs[1], outs[0].cpu()) < 3e-2
    from coffin_b200.ops import kernels as K
    torch.cuda.synchronize()
    K.check_status()


@torch.no_grad()
def test_qwen4_draft_head_matches_oracle_and_speculative_decoding_equals_greedy():
    from coffin_b200.models.qwen4exp.model import Qwen4ExpModel
    cfg = tiny_qwen4(mtp_num_hidden_layers=1)
    sd = random_state_dict(cfg, 0)
    sd_b = {k: (v.to(torch.bfloat16).float() if not k.endswith(("A_log", "dt_bias")) else v) for k, v in sd.items()}
    oracle = Qwen4Oracle(cfg, sd_b)
    model = Qwen4ExpModel(cfg, sd, max_seq=256, num_slots=1, with_mtp=True)
    g = torch.Generator().manual_seed(6)
    toks = torch.randint(2, cfg.vocab_size, (64,), generator=g)
    bt = torch.arange(1, 5, dtype=torch.int32, device=DEV)
    # ---- the head alone: prompt rows (prefill kernels), then chained single rows (decode kernels)
    st, mst = oracle.new_state(), oracle.new_state()
    lanes_ref = oracle.lanes(toks[:60], st)
    s_ref, m_ref = oracle.mtp_run(toks[1:60], lanes_ref[:59], mst)
    model.zero_state(0)
    model.prefill(toks[:60].to(DEV), 0, 0, bt, want_logits=False, want_lanes=True)
    lanes = model.last_lanes
    assert _rel(lanes, lanes_ref) < 6e-2
    s_got, m_got = model.mtp_run(toks[1:60].to(DEV), lanes[:59], 0, bt)
    assert _rel(s_got, s_ref) < 8e-2 and _rel(m_got, m_ref) < 8e-2
    s1_ref, m1_ref = oracle.mtp_run(toks[60:61], lanes_ref[59:60], mst)
    s1, m1 = model.mtp_run(toks[60:61].to(DEV), lanes[59:60], 59, bt)
    assert _rel(s1, s1_ref) < 8e-2
    s2_ref, _ = oracle.mtp_run(toks[61:62], m1_ref, mst, add_embedding=False)
    s2, _ = model.mtp_run(toks[61:62].to(DEV), m1.clone(), 60, bt, add_embedding=False)
    assert _rel(s2, s2_ref) < 8e-2
    # ---- speculative decoding == the model's own greedy decoding, with accepted drafts fed by a hook
    prompt = toks[:50].tolist()
    model.zero_state(0)
    lg = model.prefill(toks[:50].to(DEV), 0, 0, bt)
    ref, margin = [int(lg.argmax())], [float(lg.topk(2).values.diff().abs())]
    for i in range(23):
        model.set_rows(1, [ref[-1]], [50 + i], [0], [bt.tolist()])
        nxt, lg = model.decode(1)
        ref.append(int(nxt[0]))
        margin.append(float(lg[0].topk(2).values.diff().abs()))

    def agree(out):
        """Equal up to the first position whose top-2 margin is within the kernels' rounding noise (the
        verify pass scores with the prefill kernels, plain decoding with the decode kernels)."""
        for i, (a, b) in enumerate(zip(out, ref)):
            if a != b:
                return margin[i] < 0.02
        return len(out) == len(ref)

    out, stats = model.spec_generate(prompt, 24, k=3, slot=0, block_table=bt)
    assert agree(out) and stats["drafted"] == 3 * stats["rounds"]
    rounds = []

    def hook(position, drafts):
        i = position - len(prompt)
        good = len(rounds) % 4
        rounds.append(good)
        return [ref[i + j] if j < good and i + j < len(ref) else (drafts[j] + 1) % cfg.vocab_size for j in range(3)]

    for reuse in (True, False):
        rounds.clear()
        out, stats = model.spec_generate(prompt, 24, k=3, slot=0, block_table=bt, index_reuse=reuse, draft_hook=hook)
        assert agree(out), (reuse, out, ref)
        assert stats["accepted"] > 0
    from coffin_b200.ops import kernels as K
    torch.cuda.synchronize()
    K.check_status()


@torch.no_grad()
def test_qwen4_image_tokens_with_three_axis_rotary_positions_match_oracle():
    """A prompt with an image in the middle: the tower's embeddings replace the image tokens, their
    rotary rows come from (t, h, w) positions, the text after the image continues at index + delta on
    all axes, and block keys of blocks that complete later are rotated with the rows recorded for
    their first token.  Chunked prefill (a chunk boundary inside the image), then decode steps."""
    from coffin_b200.models import build_model
    from coffin_b200.models.qwen35.vision import patchify
    from coffin_b200.utils.mm_input import mrope_positions
    cfg = tiny_qwen4()
    sd = random_state_dict(cfg, 0)
    sd_b = {k: (v.to(torch.bfloat16).float() if not k.endswith(("A_log", "dt_bias")) else v) for k, v in sd.items()}
    oracle = Qwen4Oracle(cfg, sd_b)
    model = build_model(cfg, sd, device=DEV, max_seq=256, num_slots=2, vision="tiny")
    assert model.vision is not None and model.rc_cos is not None
    g = torch.Generator().manual_seed(8)
    image = torch.rand(3, 96, 64, generator=g)
    patches, grid = patchify(image, model.vision.cfg)
    feats = model.vision.forward(patches.to(DEV), grid)                     # [n_img, H]
    n_img = feats.shape[0]
    assert n_img == grid[0] * grid[1] * grid[2] // 4
    n_txt0, n_txt1 = 21, 40
    n = n_txt0 + n_img + n_txt1
    toks = torch.randint(2, cfg.vocab_size, (n + 6,), generator=g)
    pos3, delta = mrope_positions(n, [(n_txt0, n_txt0 + n_img)], [grid], 2)
    assert delta != 0
    emb = model.embed_tokens(toks[:n].to(DEV)).clone()
    emb[n_txt0:n_txt0 + n_img] = feats.to(emb.dtype)
    cos, sin = model.mrope_rows(pos3)
    bt = torch.arange(1, 5, dtype=torch.int32, device=DEV)
    model.zero_state(0)
    cut = n_txt0 + n_img // 2                                               # chunk boundary inside the image
    model.prefill(toks[:cut].to(DEV), 0, 0, bt, embeds=emb[:cut], cos_sin=(cos[:cut], sin[:cut]), want_logits=False)
    got = model.prefill(toks[cut:n].to(DEV), cut, 0, bt, embeds=emb[cut:n], cos_sin=(cos[cut:n], sin[cut:n]))
    st = oracle.new_state()
    ref = oracle.forward(toks[:n], st, embeds=emb.float().cpu(), pos3=pos3)[-1]
    assert _rel(got, ref) < 8e-2
    for i in range(n, n + 6):
        p3 = torch.full((3, 1), i + delta, dtype=pos3.dtype)
        ref = oracle.forward(toks[i:i + 1], st, pos3=p3)[-1]
        model.set_rows(1, [int(toks[i])], [i], [0], [bt.tolist()], [delta])
        _, logits = model.decode(1)
        assert _rel(logits[0], ref) < 8e-2, f"step {i}"
    # a text-only model refuses offsets instead of rotating with the wrong rows
    plain = build_model(cfg, sd, device=DEV, max_seq=256, num_slots=1)
    with pytest.raises(ValueError, match="rotary"):
        plain.set_rows(1, [1], [5], [0], [bt.tolist()], [3])
    from coffin_b200.ops import kernels as K
    torch.cuda.synchronize()
    K.check_status()


@torch.no_grad()
def test_qwen4_decode_as_cuda_graph_equals_the_eager_step():
    """A model without n-gram injection replays its decode step as a CUDA graph (captured per row count):
    twelve steps - block keys complete every fourth token, so the device-side completion test is hit
    three times per row - give the eager step's logits bit for bit, for one row and for three."""
    from coffin_b200.models.qwen4exp import model as qm
    cfg = tiny_qwen4(ple_layer_ids=())
    sd = random_state_dict(cfg, 0)
    g = torch.Generator().manual_seed(9)
    seqs = [torch.randint(2, cfg.vocab_size, (n + 12,), generator=g) for n in (61, 40, 52)]
    tables = [list(range(1 + 4 * r, 5 + 4 * r)) for r in range(3)]
    outs = {}
    for use_graph in (True, False):
        model = qm.Qwen4ExpModel(cfg, sd, max_seq=256, num_slots=3)
        assert model.graph_ok()
        for rows in (1, 3):
            lens = [s.numel() - 12 for s in seqs[:rows]]
            for r in range(rows):
                model.zero_state(r)
                model.prefill(seqs[r][:lens[r]].to(DEV), 0, r, torch.tensor(tables[r], dtype=torch.int32, device=DEV), want_logits=False)
            M = model.bucket_for(rows)
            for step in range(12):
                model.set_rows(M, [int(seqs[r][lens[r] + step]) for r in range(rows)], [lens[r] + step for r in range(rows)],
                               list(range(rows)), tables[:rows])
                _, lg = model.decode(M, graph=use_graph)
                outs.setdefault((use_graph, rows), []).append(lg[:rows].clone())
        assert bool(model._graphs) == use_graph
    for rows in (1, 3):
        for a, b in zip(outs[(True, rows)], outs[(False, rows)]):
            assert torch.equal(a, b), rows
    # a model with the n-gram layer keeps the eager step
    assert not qm.Qwen4ExpModel(tiny_qwen4(), random_state_dict(tiny_qwen4(), 0), max_seq=128, num_slots=1).graph_ok()
    from coffin_b200.ops import kernels as K
    torch.cuda.synchronize()
    K.check_status()
