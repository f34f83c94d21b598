"""Helper of ``test_oracle_vs_reference.py``: runs the unmodified reference engine (installed under
``baseline/_ref``, its torch ``reference`` backend on the CPU) beside this repo's fp32 oracles and
prints one JSON line of differences.  Runs in a process of its own because the reference's
top-level packages (``engine``, ``models``, ``ops`` ...) would otherwise stay imported."""
from __future__ import annotations

import json
import os
import sys
import tempfile
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"


def qwen35() -> dict:
    """BASELINE config 1 (tiny hybrid, prompt 64, teacher-forced decode): logits of the reference's
    paged engine against ``oracle/model.py``."""
    from coffin_b200.config import preset
    from coffin_b200.oracle.model import OracleModel
    from coffin_b200.weights.init import random_state_dict, save_checkpoint
    cfg = preset("tiny")
    sd = random_state_dict(cfg, 0, dtype=torch.float32)
    keep = ("A_log", "dt_bias")
    tmp = tempfile.mkdtemp(prefix="tiny_ckpt_")
    save_checkpoint(cfg, {k: v if k.endswith(keep) else v.to(torch.bfloat16) for k, v in sd.items()}, tmp)
    sd_b = {k: v if k.endswith(keep) else v.to(torch.bfloat16).float() for k, v in sd.items()}
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab_size, (64,), generator=g).tolist()
    m = OracleModel(cfg, sd_b, kv_int8=True)          # the reference's paged cache stores int8 KV
    import engine_api
    from engine.prefix_engine import PrefixCacheEngine
    with torch.inference_mode():
        model = engine_api.create_model(tmp, max_seq=256, bench=False, paged=True)
        eng = PrefixCacheEngine(model, num_blocks=16, block_size=64, graph=False)
        lg = eng.prefill(prompt)
        st = m.new_state()
        mine = m.forward(torch.tensor(prompt), st)[-1]
        worst, scale, agree = 0.0, float(mine.abs().max()), 0
        for _ in range(24):
            worst = max(worst, (lg.float().reshape(-1) - mine).abs().max().item())
            t = int(lg.float().argmax())
            agree += int(t == int(mine.argmax()))
            eng.seq.reserve(1)
            lg = model.logits(t)
            eng.seq.commit_upto(model.pos1)
            mine = m.forward(torch.tensor([t]), st)[-1]
    return {"worst_abs": worst, "scale": scale, "argmax_agree": agree, "steps": 24}


def qwen4() -> dict:
    """Tiny Qwen4-exp config: the reference's torch ``CausalLM`` against ``models/qwen4exp/oracle.py``."""
    from coffin_b200.models.qwen4exp.config import tiny_qwen4
    from coffin_b200.models.qwen4exp.oracle import Qwen4Oracle
    from coffin_b200.models.qwen4exp.weights import random_state_dict
    cfg = tiny_qwen4(full_select_factor=0)
    sd = random_state_dict(cfg, 0)
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, cfg.vocab_size, (100,), generator=g)
    toks[40] = cfg.eos_token_id
    o = Qwen4Oracle(cfg, sd)
    st = o.new_state()
    mine = o.forward(toks[:90], st)
    mine_dec = [o.forward(toks[i:i + 1], st) for i in range(90, 100)]
    from models.qwen4exp.config import TextConfig
    from models.qwen4exp.model import CausalLM, causal_mask
    import models.qwen4exp.qsa as qsa
    qsa._FULL_SELECT_FACTOR = 0
    tc = TextConfig.from_dict(cfg.to_hf()["text_config"])
    ref = CausalLM(tc).float().eval()
    mapped = {k.replace("model.language_model.", "model."): v for k, v in sd.items()}
    ref.load_state_dict(mapped, strict=False)
    with torch.no_grad():
        lg, states = ref(input_ids=toks[:90].view(1, -1), attention_mask=causal_mask(1, 90, 0))
        row_diff = (lg[0] - mine).abs().amax(-1)
        dec = []
        for i in range(90, 100):
            lg, states = ref(input_ids=toks[i:i + 1].view(1, -1), attention_mask=causal_mask(1, 1, i), states=states)
            dec.append((lg[0] - mine_dec[i - 90]).abs().max().item())
    return {"prefill_last_row_abs": float(row_diff[-1]), "prefill_rows_off": int((row_diff > 1e-4).sum()),
            "decode_worst_abs": max(dec), "scale": float(mine.abs().max())}


if __name__ == "__main__":
    os.environ["COFFIN_BACKEND"] = "reference"
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(REF))
    torch.set_num_threads(max(1, (os.cpu_count() or 2) // 2))
    print(json.dumps({"qwen35": qwen35, "qwen4": qwen4}[sys.argv[1]]()))
