"""Image requests on the CPU twin: mRoPE positions, placeholder expansion, chunked prefill with
scattered image embeddings equals one-shot, decode uses rope_delta, and the radix cache keys blocks
by image content (same tokens + different pixels = no hit)."""
import base64
import io

import pytest
import torch

from coffin_b200.config import preset
from coffin_b200.engine.config import EngineConfig
from coffin_b200.engine.llm_engine import LLMEngine
from coffin_b200.engine.sequence import SamplingParams
from coffin_b200.oracle import ops as O
from coffin_b200.oracle.engine_model import OracleEngineModel
from coffin_b200.oracle.model import OracleModel
from coffin_b200.serving.multimodal import decode_image, expand_placeholders
from coffin_b200.utils.mm_input import MMInput, find_image_spans, mrope_positions
from coffin_b200.weights.init import random_state_dict

CFG = preset("tiny")
SD = random_state_dict(CFG, 0)
IMG = 4000       # placeholder id inside the tiny vocabulary


def test_positions_and_expansion():
    prompt = [1, 2, IMG, 3, 4]
    out = expand_placeholders(prompt, IMG, [6])
    assert out == [1, 2] + [IMG] * 6 + [3, 4]
    spans = find_image_spans(out, IMG)
    assert spans == [(2, 8)]
    pos, delta = mrope_positions(len(out), spans, [(1, 4, 6)], merge=2)     # 2 x 3 merged patches
    assert pos[:, :2].tolist() == [[0, 1]] * 3
    assert pos[0, 2:8].tolist() == [2] * 6
    assert pos[1, 2:8].tolist() == [2, 2, 2, 3, 3, 3] and pos[2, 2:8].tolist() == [2, 3, 4, 2, 3, 4]
    assert pos[:, 8].tolist() == [5, 5, 5] and delta == 5 + 2 - len(out)
    with pytest.raises(Exception):
        expand_placeholders(prompt, IMG, [6, 6])


def _mm(prompt, embeds, digest):
    spans = find_image_spans(prompt, IMG)
    n = spans[0][1] - spans[0][0]
    pos, delta = mrope_positions(len(prompt), spans, [(1, 2, 2 * n)], merge=2)
    return MMInput(embeds=embeds, grid_thw=[(1, 2, 2 * n)], positions=pos, rope_delta=delta, digests=[digest], spans=spans)


@torch.no_grad()
def test_engine_with_image_embeddings_and_media_salted_cache():
    g = torch.Generator().manual_seed(5)
    text = torch.randint(0, 3000, (150,), generator=g).tolist()
    prompt = text[:70] + [IMG] * 8 + text[70:]
    emb_a = torch.randn(8, CFG.hidden_size, generator=g) * 0.05
    emb_b = torch.randn(8, CFG.hidden_size, generator=g) * 0.05
    # oracle: full forward with embeddings scattered and 3-axis positions
    def oracle_tokens(emb, n):
        m = OracleModel(CFG, SD)
        st = m.new_state()
        mm = _mm(prompt, emb, "x")
        x = m.embed(torch.tensor(prompt)).clone()
        x[70:78] = emb
        logits = m.forward(torch.tensor(prompt), st, embeds=x, positions3=mm.positions)[-1]
        out = []
        for _ in range(n):
            t = int(logits.argmax())
            out.append(t)
            logits = m.forward(torch.tensor([t]), st, rope_delta=mm.rope_delta)[-1]
        return out
    ref_a, ref_b = oracle_tokens(emb_a, 4), oracle_tokens(emb_b, 4)
    model = OracleEngineModel(CFG, SD, max_seq=512, num_slots=2)
    eng = LLMEngine(model, EngineConfig(max_seq=512, max_num_seqs=2, graph=False, chunk=64, prefill_quantum=64,
                                        max_num_batched_tokens=64, snapshot_interval=64))
    sa = eng.add_request(prompt, SamplingParams(max_tokens=4), mm=_mm(prompt, emb_a, "digest-a"))
    while not sa.finished:
        eng.step()
    assert sa.output == ref_a and sa.cached_tokens == 0
    # same tokens, other pixels: the shared text prefix (first block) hits, the image block does not
    sb = eng.add_request(prompt, SamplingParams(max_tokens=4), mm=_mm(prompt, emb_b, "digest-b"))
    while not sb.finished:
        eng.step()
    assert sb.output == ref_b and sb.cached_tokens == 64
    # same image again: hits through the image
    sc = eng.add_request(prompt, SamplingParams(max_tokens=4), mm=_mm(prompt, emb_a, "digest-a"))
    while not sc.finished:
        eng.step()
    assert sc.output == ref_a and sc.cached_tokens >= 128


@torch.no_grad()
def test_preempted_image_request_recomputes_to_the_same_tokens():
    """A preempted sequence re-prefills prompt + generated tokens; the rotary positions past the
    prompt continue at index + rope_delta, so the output equals the run that was never preempted."""
    g = torch.Generator().manual_seed(9)
    emb = torch.randn(8, CFG.hidden_size, generator=g) * 0.05

    def run(num_blocks):
        model = OracleEngineModel(CFG, SD, max_seq=512, num_slots=3, num_blocks=num_blocks)
        eng = LLMEngine(model, EngineConfig(max_seq=512, max_num_seqs=3, graph=False, prefix_cache=False,
                                            chunk=64, prefill_quantum=64, max_num_batched_tokens=64))
        seqs = []
        for i in range(3):
            text = torch.randint(0, 3000, (118,), generator=torch.Generator().manual_seed(20 + i)).tolist()
            prompt = text[:60] + [IMG] * 8 + text[60:]
            seqs.append(eng.add_request(prompt, SamplingParams(max_tokens=8), mm=_mm(prompt, emb, f"d{i}")))
        while any(not s.finished for s in seqs):
            eng.step()
        return [s.output for s in seqs], eng.n_preempt

    roomy, n0 = run(64)
    tight, n1 = run(9)          # three 126-token prompts hold 2 blocks each and each grows into a 3rd
    assert n0 == 0 and n1 >= 1
    assert tight == roomy


def test_decode_image_budget_and_errors():
    from PIL import Image
    from coffin_b200.serving.runtime import MMError
    buf = io.BytesIO()
    Image.new("RGB", (100, 60), (255, 0, 0)).save(buf, format="PNG")
    t, raw = decode_image(base64.b64encode(buf.getvalue()).decode(), 32 * 32, 64 * 64, 32)
    assert t.shape[0] == 3 and t.shape[1] % 32 == 0 and t.shape[2] % 32 == 0 and t.shape[1] * t.shape[2] <= 64 * 64
    assert abs(float(t[0].mean()) - 1.0) < 1e-3 and float(t[1].max()) < 1e-3
    with pytest.raises(MMError):
        decode_image("!!!notbase64", 1024, 4096, 32)
    with pytest.raises(MMError):
        decode_image(base64.b64encode(b"not an image").decode(), 1024, 4096, 32)


def test_engine_side_image_byte_limit():
    from PIL import Image
    from coffin_b200.serving.runtime import MMError
    buf = io.BytesIO()
    Image.new("RGB", (64, 64), (0, 255, 0)).save(buf, format="PNG")
    b64 = base64.b64encode(buf.getvalue()).decode()
    n = len(buf.getvalue())
    decode_image(b64, 32 * 32, 64 * 64, 32, max_bytes=n)                 # exactly at the limit
    with pytest.raises(MMError) as e:
        decode_image(b64, 32 * 32, 64 * 64, 32, max_bytes=n - 1)
    assert e.value.status == 413
