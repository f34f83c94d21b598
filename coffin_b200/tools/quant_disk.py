"""Write a pre-quantised checkpoint directory.

    python -m coffin_b200.tools.quant_disk --model SRC --out DST --scheme int8     # coffin-int8-kn-v1
    python -m coffin_b200.tools.quant_disk --model SRC --out DST --scheme w4a8     # coffin-w4a8-kn-v1
    python -m coffin_b200.tools.quant_disk --preset tiny --out DST --scheme int8   # random-init source

The output holds ``quant_index.json`` (format tag, source-config digest, per-tensor kinds and
shapes), ``quant-XXXXX-of-YYYYY.safetensors`` shards and a copy of ``config.json``; the loader
(``weights/loader.py``) recognises the directory and hands the engine ready containers, so a served
model starts without touching the bf16 weights.  Layouts: per-output-channel symmetric int8
(``[K, N]`` int8 + ``[N]`` fp32 scale) and group-128 int4 (``[K/2, N]`` packed nibbles + ``[G, N]``
scales); routed experts are fused into ``[E, K, N]`` stacks; the router, the shared-expert gate,
norms, conv taps and the embedding stay dense.  Reference: ``tools/quant_disk.py:147-177,229-383,
533-554`` (int8) and ``tools/quant_disk_w4a8.py:45-89,241-246`` (W4A8).
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", help="source checkpoint directory (HF safetensors)")
    ap.add_argument("--preset", help="draw a random-init source of this named geometry instead")
    ap.add_argument("--out", required=True)
    ap.add_argument("--scheme", choices=("int8", "w4a8"), default="int8")
    ap.add_argument("--shard-gb", type=float, default=4.0)
    ap.add_argument("--verify", action="store_true", help="reload the output and report the worst dequantisation error")
    args = ap.parse_args(argv)
    import torch
    from ..config import load_config, preset
    from ..weights.init import random_state_dict, save_checkpoint
    from ..weights.loader import load_checkpoint
    from ..weights.quant_io import load_quantized, summary, write_quantized
    t0 = time.time()
    if args.model:
        src_dir = args.model
        sd = load_checkpoint(src_dir)
    elif args.preset:
        import tempfile
        cfg = preset(args.preset)
        sd = random_state_dict(cfg, 0, dtype=torch.bfloat16)
        src_dir = tempfile.mkdtemp(prefix="coffin_src_")
        save_checkpoint(cfg, sd, src_dir)
    else:
        ap.error("give --model or --preset")
    load_config(src_dir)                       # fails early on an unknown family
    write_quantized(src_dir, sd, args.out, scheme=args.scheme, shard_bytes=int(args.shard_gb * (1 << 30)))
    rep = summary(args.out)
    rep["seconds"] = round(time.time() - t0, 1)
    if args.verify:
        from ..weights.quant import QWeight, W4A8Weight
        back = load_quantized(args.out)
        worst = 0.0
        for k, v in back.items():
            if isinstance(v, (QWeight, W4A8Weight)) and k in sd:
                ref = sd[k].float()
                err = ((v.dequant() - ref).abs().max() / ref.abs().max().clamp_min(1e-9)).item()
                worst = max(worst, err)
        rep["worst_relative_error"] = round(worst, 4)
    json.dump(rep, sys.stdout, indent=1)
    print()
    return 0


if __name__ == "__main__":
    sys.exit(main())
