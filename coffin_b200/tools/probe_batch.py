"""Does a batched decode step give every row what it gets alone?

    python -m coffin_b200.tools.probe_batch --preset qwen35-4b --layers 8 --rows 1 2 4 8

Prefills ``max(rows)`` different prompts, then for every row count runs one decode step over the
first ``n`` sequences together and compares each row's logits with the same sequence decoded alone
from the same state (max relative difference, argmax agreement), and prints the step time per row
count.  On-card counterpart of the reference's ``tools/probe_batch_*.py`` (batch vs single token
equality, batch scaling B = 1..8).
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--preset", default="tiny")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--prompt", type=int, default=96)
    ap.add_argument("--rows", type=int, nargs="+", default=[1, 2, 4, 8])
    ap.add_argument("--quant", default="none")
    args = ap.parse_args(argv)
    import torch
    from ..config import preset
    from ..models import build_model
    from ..weights.init import random_state_dict
    cfg = preset(args.preset)
    if args.layers and args.layers < cfg.num_hidden_layers:
        cfg = dataclasses.replace(cfg, num_hidden_layers=args.layers, layer_types=cfg.layer_types[:args.layers])
    R = max(args.rows)
    sd = random_state_dict(cfg, 0, dtype=torch.bfloat16, device="cuda")
    model = build_model(cfg, sd, device="cuda", max_seq=args.prompt + 64, num_slots=R, quant=args.quant)
    g = torch.Generator().manual_seed(0)
    nblk = model.max_blocks_per_seq
    tables = [list(range(1 + r * nblk, 1 + (r + 1) * nblk)) for r in range(R)]
    prompts = [torch.randint(0, cfg.vocab_size, (args.prompt - r,), generator=g) for r in range(R)]
    for r, p in enumerate(prompts):
        model.zero_state(r)
        model.prefill(p.cuda(), 0, r, torch.tensor(tables[r], dtype=torch.int32, device="cuda"), want_logits=False)
    snaps = [model.snapshot_state(r) for r in range(R)]
    toks = [int(p[-1]) for p in prompts]
    pos = [len(p) for p in prompts]
    alone = []
    for r in range(R):
        model.set_rows(1, [toks[r]], [pos[r]], [r], [tables[r]])
        alone.append(model.decode(1)[1][0].float().clone())
        model.restore_state(r, snaps[r])
    report = []
    for n in args.rows:
        M = model.bucket_for(n)
        model.set_rows(M, toks[:n], pos[:n], list(range(n)), tables[:n])
        model.decode(M)                                   # warm-up (graph capture)
        for r in range(n):
            model.restore_state(r, snaps[r])
        model.set_rows(M, toks[:n], pos[:n], list(range(n)), tables[:n])
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        _, logits = model.decode(M)
        t1.record()
        torch.cuda.synchronize()
        worst, agree = 0.0, 0
        for r in range(n):
            d = ((logits[r].float() - alone[r]).abs().max() / alone[r].abs().max()).item()
            worst = max(worst, d)
            agree += int(int(logits[r].argmax()) == int(alone[r].argmax()))
            model.restore_state(r, snaps[r])
        report.append({"rows": n, "bucket": M, "step_ms": round(t0.elapsed_time(t1), 3),
                       "max_rel_diff_vs_alone": round(worst, 5), "argmax_agree": f"{agree}/{n}"})
    json.dump(report, sys.stdout, indent=1)
    print()
    return 0


if __name__ == "__main__":
    sys.exit(main())
