"""Staged self-check of a Qwen4-exp checkpoint: is it complete, does it load, does it compute.

    python -m coffin_b200.tools.check_qwen4 --model DIR --stage geometry
    python -m coffin_b200.tools.check_qwen4 --model DIR --stage layers --layers 2 --tokens 8 [--device cuda]
    python -m coffin_b200.tools.check_qwen4 --model DIR --stage all

Every stage has a verdict that can be checked on its own, so a failure says "a shard is missing", "a tensor
has another version's shape" or "the arithmetic is off" instead of showing one NaN at the end:

* ``geometry``: the shard headers against the tensor plan of the configuration - names, shapes, the row
  shards of the n-gram table counted as one table; no tensor data is read (seconds for hundreds of GB).
* ``layers``: the first N layers (default 2: the second layer carries the first n-gram injection) are read
  through the streaming loader - the n-gram table stays a set of mapped host views - and a few tokens go
  through the fp32 CPU oracle: all outputs finite, next-token distribution not degenerate.  With
  ``--device cuda`` the sm_100a model runs the same tokens and its logits are compared with the oracle's.
* ``all``: both, stopping at the first failure.

One JSON line per stage; exit status 1 when a stage fails (reference: ``models/qwen4exp/prefill_check.py``).
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def check_geometry(model_dir, cfg) -> dict:
    from ..models.qwen4exp.weights import checkpoint_index, tensor_plan, verify_plan
    t0 = time.perf_counter()
    index = checkpoint_index(model_dir)
    rep = verify_plan(cfg, model_dir, index)
    ok = not rep["missing"] and not rep["shape"]
    return {"stage": "geometry", "ok": ok, "planned": len(tensor_plan(cfg)), "in_checkpoint": len(index),
            "files": len(set(index.values())), "missing": rep["missing"][:8], "n_missing": len(rep["missing"]),
            "shape": [list(map(str, x)) for x in rep["shape"][:8]], "n_shape": len(rep["shape"]),
            "unexpected": rep["unexpected"][:8], "seconds": round(time.perf_counter() - t0, 2)}


def check_layers(model_dir, cfg, n_layers: int, n_tokens: int, device: str, tol: float) -> dict:
    import torch
    from ..models.qwen4exp.oracle import Qwen4Oracle
    from ..models.qwen4exp.weights import first_layers, load_streaming
    t0 = time.perf_counter()
    sub = first_layers(cfg, n_layers)
    sd = load_streaming(model_dir, cfg, layers=sub.num_hidden_layers)
    nbytes = sum(t.numel() * t.element_size() for v in sd.values() for t in (v if isinstance(v, list) else [v])
                 if isinstance(t, torch.Tensor))
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(2, sub.vocab_size, (n_tokens,), generator=g)
    oracle = Qwen4Oracle(sub, sd)
    ref = oracle.forward(toks, oracle.new_state())
    finite = bool(torch.isfinite(ref).all())
    probs = torch.softmax(ref[-1].float(), -1)
    out = {"stage": "layers", "layers": sub.num_hidden_layers, "tokens": n_tokens, "bytes_read": int(nbytes),
           "ple_layers": [i for i in sub.ple_layer_ids], "finite": finite, "top1_prob": round(float(probs.max()), 4),
           "logit_absmax": round(float(ref.abs().max()), 4)}
    ok = finite and float(probs.max()) < 0.999
    if device.startswith("cuda"):
        from ..models.qwen4exp.model import Qwen4ExpModel
        model = Qwen4ExpModel(sub, sd, max_seq=max(64, n_tokens + 8), num_slots=1)
        bt = torch.arange(1, model.max_blocks_per_seq + 1, dtype=torch.int32, device="cuda")
        model.zero_state(0)
        got = model.prefill(toks.cuda(), 0, 0, bt).float().cpu()
        rel = float((got - ref[-1].float()).abs().max() / ref[-1].float().abs().max())
        out["device_vs_oracle"] = round(rel, 5)
        ok = ok and rel < tol
    out["ok"] = ok
    out["seconds"] = round(time.perf_counter() - t0, 2)
    return out


def main(argv=None) -> int:
    from ..config import load_config
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="checkpoint directory (config.json + safetensors shards)")
    ap.add_argument("--stage", default="all", choices=("geometry", "layers", "all"))
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--tokens", type=int, default=8)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--tol", type=float, default=5e-2, help="device vs oracle: max |diff| / max |logit|")
    a = ap.parse_args(argv)
    cfg = load_config(a.model)
    stages = ("geometry", "layers") if a.stage == "all" else (a.stage,)
    for st in stages:
        rep = check_geometry(a.model, cfg) if st == "geometry" else check_layers(a.model, cfg, a.layers, a.tokens, a.device, a.tol)
        print(json.dumps(rep), flush=True)
        if not rep["ok"]:
            return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
