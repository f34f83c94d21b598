"""Phase breakdown of the persistent decode kernel: where one decode step spends its time.

    python -m coffin_b200.tools.trace_mega --model qwen35-4b --prompt 2048 --steps 8

CTA 0 stamps ``%globaltimer`` at every phase boundary (prologue, projection, barrier, mixer); the
report sums the spans per phase kind over the layers of the last step.  The stamps are taken inside
the running kernel, so nothing is serialised the way a profiler would.
"""
from __future__ import annotations

import argparse
import dataclasses
import json

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen35-4b")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--rows", type=int, default=1)
    args = ap.parse_args()
    from ..config import preset
    from ..engine.llm import LLM
    from ..ops import kernels as K
    cfg = preset(args.model)
    if args.layers and args.layers < cfg.num_hidden_layers:
        cfg = dataclasses.replace(cfg, num_hidden_layers=args.layers, layer_types=cfg.layer_types[:args.layers])
    llm = LLM.from_random(cfg, seed=0, max_seq=args.prompt + 64, max_num_seqs=max(1, args.rows), max_chunk=args.prompt)
    m = llm.model
    g = torch.Generator().manual_seed(0)
    bt = list(range(m.max_blocks_per_seq))
    for r in range(args.rows):
        m.zero_state(r)
        m.prefill(torch.randint(0, cfg.vocab_size, (args.prompt,), generator=g).cuda(), 0, r,
                  torch.tensor(bt, dtype=torch.int32, device="cuda"), want_logits=False)
    M = m.bucket_for(args.rows)
    mega = m._mega_for(M)
    if mega is None:
        raise SystemExit("this model / bucket does not run on the persistent kernel")
    mega.enable_trace()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(args.steps):
        m.set_rows(M, [1] * args.rows, [args.prompt + i] * args.rows, list(range(args.rows)), [bt] * args.rows)
        if i == args.steps - 1:
            ev0.record()
        m.decode(M, graph=False)
    ev1.record()
    torch.cuda.synchronize()
    K.check_status()
    rep = mega.phase_times()
    rep["event_us"] = ev0.elapsed_time(ev1) * 1e3
    for kind in ("lin", "full", "head"):
        rep[kind] = {k: round(v, 1) for k, v in rep[kind].items()}
    print(json.dumps(rep, indent=1))


if __name__ == "__main__":
    main()
