"""Write a pre-quantised checkpoint directory of a Qwen4-exp model, streaming.

    python -m coffin_b200.tools.quant_disk_qwen4 --model SRC --out DST --scheme w4a8
    python -m coffin_b200.tools.quant_disk_qwen4 --preset tiny-qwen4 --out DST --scheme int8 --verify

The source is read tensor by tensor from its shards and the output is written shard by shard, so the
tool needs memory for one tensor and one output shard - not for the model (the routed expert stacks
and the n-gram table of the PLE layer are each tens of GiB in the real geometry).  Per-expert source
spellings (``experts.{e}.gate_proj.weight`` ...) are fused into one stack per layer before quantisation,
one layer at a time.  What is quantised: the mixer projections (with the fused indexer projection),
routed and shared experts and the lm_head; the router, gates, norms, conv taps, hyper-connection
matrices, PLE tensors and the embedding stay in their source dtype.  The output carries
``quant_index.json`` in the same two formats as the Qwen3.5 tool (``coffin-int8-kn-v1`` /
``coffin-w4a8-kn-v1``) and is read back by ``weights.loader.load_checkpoint``.
Reference: ``tools/quant_disk_qwen4.py`` (streaming per-layer quantiser for this family).
"""
from __future__ import annotations

import argparse
import json
import re
import sys
import time
from pathlib import Path


def stream_tensors(model_dir: Path, index: dict[str, str]):
    """Yield ``(key, tensor)`` shard by shard; per-expert tensors of a layer are collected and yielded as
    the two fused stacks as soon as the layer is complete."""
    import torch
    from safetensors import safe_open
    pat = re.compile(r"^(.*\.mlp\.experts\.)(\d+)\.(gate_proj|up_proj|down_proj)\.weight$")
    n_exp: dict[str, int] = {}
    for k in index:
        m = pat.match(k)
        if m:
            n_exp[m.group(1)] = max(n_exp.get(m.group(1), 0), int(m.group(2)) + 1)
    pending: dict[str, dict] = {}
    by_file: dict[str, list[str]] = {}
    for k, f in index.items():
        by_file.setdefault(f, []).append(k)
    for fname in sorted(by_file):
        with safe_open(str(model_dir / fname), framework="pt") as fh:
            for k in sorted(by_file[fname]):
                m = pat.match(k)
                if not m:
                    yield k, fh.get_tensor(k)
                    continue
                base = m.group(1)
                slot = pending.setdefault(base, {"gate_proj": {}, "up_proj": {}, "down_proj": {}})
                slot[m.group(3)][int(m.group(2))] = fh.get_tensor(k)
                n = n_exp[base]
                if all(len(slot[x]) == n for x in slot):
                    yield base + "gate_up_proj", torch.stack([torch.cat([slot["gate_proj"][e], slot["up_proj"][e]]) for e in range(n)])
                    yield base + "down_proj", torch.stack([slot["down_proj"][e] for e in range(n)])
                    del pending[base]
    if pending:
        raise ValueError(f"incomplete expert sets: {sorted(pending)[:3]}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", help="source checkpoint directory (HF safetensors)")
    ap.add_argument("--preset", help="draw a random-init source of this named geometry instead (e.g. tiny-qwen4)")
    ap.add_argument("--out", required=True)
    ap.add_argument("--scheme", choices=("int8", "w4a8"), default="w4a8")
    ap.add_argument("--shard-gb", type=float, default=4.0)
    ap.add_argument("--quant-embed", action="store_true",
                    help="int8 scheme only: store the embedding table as int8 rows + per-row scales (QuantizedEmbedding)")
    ap.add_argument("--verify", action="store_true", help="reload the output and report the worst dequantisation error")
    args = ap.parse_args(argv)
    if args.quant_embed and args.scheme != "int8":
        ap.error("--quant-embed needs --scheme int8 (one format per directory)")
    import torch
    from ..config import load_config, preset
    from ..models.qwen4exp.weights import checkpoint_index, random_state_dict, verify_plan
    from ..weights.init import save_checkpoint
    from ..weights.quant import QWeight, W4A8Weight, is_quantizable_qwen4
    from ..weights.quant_io import load_quantized, summary, write_quantized
    t0 = time.time()
    if args.model:
        src = Path(args.model)
    elif args.preset:
        import tempfile
        cfg = preset(args.preset)
        src = Path(tempfile.mkdtemp(prefix="coffin_q4src_"))
        save_checkpoint(cfg, random_state_dict(cfg, 0, dtype=torch.bfloat16), src)
    else:
        ap.error("give --model or --preset")
    cfg = load_config(src)
    index = checkpoint_index(src)
    rep = verify_plan(cfg, src, index)
    if rep["missing"] or rep["shape"]:
        print(json.dumps({"ok": False, "plan": {k: v[:8] for k, v in rep.items()}}, indent=1, default=str))
        return 2
    pick = is_quantizable_qwen4
    if args.quant_embed:
        pick = lambda k, t: is_quantizable_qwen4(k, t) or k.endswith("embed_tokens.weight")
    write_quantized(src, stream_tensors(src, index), args.out, scheme=args.scheme, is_q=pick,
                    shard_bytes=int(args.shard_gb * (1 << 30)), generated_by="coffin_b200/tools/quant_disk_qwen4.py")
    out = summary(args.out)
    out["seconds"] = round(time.time() - t0, 1)
    out["unexpected_source_tensors"] = rep["unexpected"][:8]
    if args.verify:
        from ..weights.loader import load_checkpoint
        dense = load_checkpoint(src)
        back = load_quantized(args.out)
        worst = 0.0
        for k, v in back.items():
            if isinstance(v, (QWeight, W4A8Weight)):
                ref = dense[k].float()
                worst = max(worst, ((v.dequant() - ref).abs().max() / ref.abs().max().clamp_min(1e-9)).item())
        out["worst_relative_error"] = round(worst, 4)
    json.dump(out, sys.stdout, indent=1)
    print()
    return 0


if __name__ == "__main__":
    sys.exit(main())
