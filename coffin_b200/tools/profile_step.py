"""Small fixed workload for kernel profiling: a few layers of a named model shape, one prefill
chunk and a few decode steps, no timing.

    python -m coffin_b200.tools.profile_step --model qwen35-4b --layers 4 --prompt 2048 --decode 3

Meant to be run under ``ncu`` (launch list or a per-kernel capture); with ``--layers 4`` the
kernels have the full model's shapes while only ~2 GB is resident.
"""
from __future__ import annotations

import argparse
import dataclasses

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen35-4b")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--decode", type=int, default=3)
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--quant", default="none", choices=["none", "int8", "w4a8"])
    ap.add_argument("--kv-dtype", default="bf16", choices=["bf16", "int8"])
    ap.add_argument("--mega", action="store_true", help="decode through the persistent one-launch kernel")
    ap.add_argument("--tp-force", action="store_true",
                    help="one GPU, world 1, with the tensor-parallel exchange forced on (push epilogues, pull+norm kernel, prefill scatter/reduce)")
    ap.add_argument("--graph", action="store_true")
    ap.add_argument("--no-pdl", action="store_true")
    args = ap.parse_args()
    import os
    if args.mega:
        os.environ["COFFIN_MEGA"] = "1"
    from ..config import preset
    from ..engine.llm import LLM
    from ..ops import kernels as K
    cfg = preset(args.model)
    if args.layers and args.layers < cfg.num_hidden_layers:
        cfg = dataclasses.replace(cfg, num_hidden_layers=args.layers, layer_types=cfg.layer_types[:args.layers])
    if args.tp_force or args.kv_dtype != "bf16":
        from ..models.qwen35.model import Qwen35Model
        from ..weights.init import random_state_dict
        tp = None
        if args.tp_force:
            from ..parallel.tp import TpComm
            tp = TpComm(0, 1, cfg.hidden_size, 8, 2 * cfg.num_hidden_layers + 2, prefill_rows=args.prompt)
        sd = random_state_dict(cfg, 0, dtype=torch.bfloat16, device="cuda")
        model = Qwen35Model(cfg, sd, max_seq=args.prompt + 64, num_slots=max(1, args.rows), max_chunk=args.prompt,
                            pdl=not args.no_pdl, free_source=True, tp=tp, quant=args.quant, kv_dtype=args.kv_dtype)
        model.tp_force = args.tp_force
        llm = LLM(model, graph=args.graph)
    else:
        llm = LLM.from_random(cfg, seed=0, max_seq=args.prompt + 64, max_num_seqs=max(1, args.rows),
                              graph=args.graph, pdl=not args.no_pdl, max_chunk=args.prompt, quant=args.quant)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab_size, (args.prompt,), generator=g).cuda()
    first = llm.device_prefill(prompt)
    torch.cuda.synchronize()
    if args.rows == 1:
        llm.device_decode(first, args.decode)
    else:
        m = llm.model
        M = m.bucket_for(args.rows)
        bt = list(range(m.max_blocks_per_seq))
        for i in range(args.decode):
            m.set_rows(M, [1] * args.rows, [args.prompt + i] * args.rows, list(range(args.rows)), [bt] * args.rows)
            m.decode(M, graph=args.graph)
    torch.cuda.synchronize()
    K.check_status()
    print(f"ok launches={K.LAUNCHES + llm.graph_launches_replayed}")


if __name__ == "__main__":
    main()
