"""On-card probes of the Qwen4-exp decode step.

    python -m coffin_b200.tools.probe_qwen4 batch      --preset tiny-qwen4 --rows 1 2 4 8
    python -m coffin_b200.tools.probe_qwen4 divergence --preset tiny-qwen4 --rows 4
    python -m coffin_b200.tools.probe_qwen4 glue       --preset tiny-qwen4
    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 -m coffin_b200.tools.probe_qwen4 ep --new 16

* ``batch``: step time and aggregate tok/s at each row count, and every row's logits against the
  same sequence decoded alone from the same state - a batched path that computes the wrong thing
  still shows a fine throughput (reference: ``tools/probe_q4_batch_b.py``).
* ``divergence``: where a batched step departs from the single-row step.  The same sequence is put in
  every row: rows that differ from one another mean cross-talk in the batch dimension, rows that agree
  with one another but not with the single-row pass mean a batch-size dependent kernel path.  The
  per-layer residual lanes of both passes are compared (reference: ``tools/probe_q4_batch_divergence.py``).
* ``glue``: what one decode step launches besides the framework's own kernels: every torch operator
  by (name, shapes, dtype) with its call count, next to the count of native launches
  (reference: ``tools/probe_q4_attrib.py``, ``tools/probe_q4_glue.py``).
* ``ep``: expert-parallel generation smoke under ``torchrun``: every rank holds a range of the routed
  experts, the ranks must produce identical tokens, and rank 0 prints prefill and per-token times
  (reference: ``tools/probe_q4_ep4_gen.py``).

``--layers N`` cuts the preset to its first N layers; weights are random (seed 0).
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys
from collections import Counter


def _build(args, num_slots: int, **kw):
    import torch
    from ..models.qwen4exp.config import preset_qwen4
    from ..models.qwen4exp.model import Qwen4ExpModel
    from ..models.qwen4exp.weights import random_state_dict
    cfg = preset_qwen4(args.preset)
    if args.layers and args.layers < cfg.num_hidden_layers:
        cfg = dataclasses.replace(cfg, num_hidden_layers=args.layers, layer_types=cfg.layer_types[:args.layers],
                                  ple_layer_ids=tuple(i for i in cfg.ple_layer_ids if i <= args.layers))
    sd = random_state_dict(cfg, 0, dtype=torch.bfloat16)
    model = Qwen4ExpModel(cfg, sd, max_seq=args.prompt + 64, num_slots=num_slots, quant=args.quant, **kw)
    return cfg, model


def _tables(model, R):
    n = model.max_blocks_per_seq
    return [list(range(1 + r * n, 1 + (r + 1) * n)) for r in range(R)]


def _prefill(model, prompts, tables):
    import torch
    for r, p in enumerate(prompts):
        model.zero_state(r)
        model.prefill(p.cuda(), 0, r, torch.tensor(tables[r], dtype=torch.int32, device="cuda"), want_logits=False)
    return [model.snapshot_state(r) for r in range(len(prompts))]


def _timed_step(model, M, reps: int = 5) -> float:
    """Median device time (ms) of ``decode(M)`` on the rows already staged; the states advance."""
    import torch
    times = []
    for _ in range(reps):
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0.record()
        model.decode(M)
        t1.record()
        torch.cuda.synchronize()
        times.append(t0.elapsed_time(t1))
    return sorted(times)[len(times) // 2]


def probe_batch(args) -> int:
    import torch
    R = max(args.rows)
    cfg, model = _build(args, R)
    g = torch.Generator().manual_seed(0)
    tables = _tables(model, R)
    prompts = [torch.randint(2, cfg.vocab_size, (args.prompt - r,), generator=g) for r in range(R)]
    snaps = _prefill(model, [p[:-1] for p in prompts], tables)
    toks, pos = [int(p[-1]) for p in prompts], [len(p) - 1 for p in prompts]
    alone = []
    for r in range(R):
        model.set_rows(1, [toks[r]], [pos[r]], [r], [tables[r]])
        alone.append(model.decode(1)[1][0].float().clone())
        model.restore_state(r, snaps[r])
    report, base = [], None
    for n in args.rows:
        M = model.bucket_for(n)
        model.set_rows(M, toks[:n], pos[:n], list(range(n)), tables[:n])
        lg = model.decode(M)[1][:n].float().clone()
        worst = max(float((lg[r] - alone[r]).abs().max() / alone[r].abs().max()) for r in range(n))
        same = sum(int(lg[r].argmax() == alone[r].argmax()) for r in range(n))
        ms = _timed_step(model, M)
        for r in range(n):
            model.restore_state(r, snaps[r])
        base = base or ms
        report.append({"rows": n, "step_ms": round(ms, 3), "tok_s": round(n / ms * 1e3, 1), "vs_one_row": round(ms / base, 2),
                       "max_rel_diff_vs_alone": round(worst, 5), "argmax_agree": f"{same}/{n}"})
    print(json.dumps({"probe": "batch", "model": cfg.name, "layers": cfg.num_hidden_layers, "report": report}, indent=1))
    return 0


def probe_divergence(args) -> int:
    import torch
    n = max(args.rows)
    cfg, model = _build(args, n)
    g = torch.Generator().manual_seed(0)
    tables = _tables(model, n)
    prompt = torch.randint(2, cfg.vocab_size, (args.prompt,), generator=g)
    snaps = _prefill(model, [prompt[:-1]] * n, tables)
    tok, pos = int(prompt[-1]), args.prompt - 1
    lanes: dict = {}
    model.layer_hook = lambda li, stream: lanes.setdefault(li, stream.float().clone())
    model.set_rows(1, [tok], [pos], [0], [tables[0]])
    model.decode(1)
    single, lanes = lanes, {}
    model.restore_state(0, snaps[0])
    M = model.bucket_for(n)
    model.set_rows(M, [tok] * n, [pos] * n, list(range(n)), tables)
    model.decode(M)
    model.layer_hook = None
    rows = []
    for li in sorted(single):
        b, s = lanes[li], single[li][0]
        scale = float(s.abs().max()) or 1.0
        rows.append({"layer": li, "kind": cfg.layer_types[li],
                     "row_vs_row": round(float((b[1:] - b[:1]).abs().max()) / scale, 6) if n > 1 else 0.0,
                     "batch_vs_single": round(float((b[0] - s).abs().max()) / scale, 6)})
    first_cross = next((r["layer"] for r in rows if r["row_vs_row"] > 0), None)
    print(json.dumps({"probe": "divergence", "rows": n, "first_layer_with_cross_talk": first_cross,
                      "worst_batch_vs_single": max(r["batch_vs_single"] for r in rows), "layers": rows}, indent=1))
    return 0


def probe_glue(args) -> int:
    import torch
    from torch.utils._python_dispatch import TorchDispatchMode
    from ..ops import kernels as K
    cfg, model = _build(args, 1)
    g = torch.Generator().manual_seed(0)
    tables = _tables(model, 1)
    prompt = torch.randint(2, cfg.vocab_size, (args.prompt,), generator=g)
    _prefill(model, [prompt[:-1]], tables)
    model.set_rows(1, [int(prompt[-1])], [args.prompt - 1], [0], [tables[0]])
    model.decode(1)                                        # warm-up: workspaces exist
    model.advance_rows(1)
    counts: Counter = Counter()

    class Tally(TorchDispatchMode):
        def __torch_dispatch__(self, func, types, a=(), kw=None):
            shapes = tuple(tuple(t.shape) for t in a if isinstance(t, torch.Tensor))
            dt = next((str(t.dtype).replace("torch.", "") for t in a if isinstance(t, torch.Tensor)), "-")
            counts[(func.__name__, shapes, dt)] += 1
            return func(*a, **(kw or {}))

    before = K.LAUNCHES
    with Tally():
        model.decode(1)
    native = K.LAUNCHES - before
    top = [{"op": k[0], "shapes": [list(s) for s in k[1]], "dtype": k[2], "calls": v} for k, v in counts.most_common(args.top)]
    print(json.dumps({"probe": "glue", "layers": cfg.num_hidden_layers, "native_launches": native,
                      "torch_ops": sum(counts.values()), "distinct": len(counts), "top": top}, indent=1))
    return 0


def probe_ep(args) -> int:
    import time
    import torch
    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        dist.init_process_group("nccl")
    from ..parallel.tp import TpComm, make_exchange
    comm = None
    if world > 1:
        from ..models.qwen4exp.config import preset_qwen4
        comm = TpComm(rank, world, preset_qwen4(args.preset).hidden_size, 8, 2, exchange=make_exchange(), prefill_rows=args.prompt + 64)
    cfg, model = _build(args, 1, tp=comm, ep_rank=rank, ep_world=world)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(2, cfg.vocab_size, (args.prompt,), generator=g)
    bt = torch.tensor(_tables(model, 1)[0], dtype=torch.int32, device="cuda")
    model.zero_state(0)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    lg = model.prefill(prompt.cuda(), 0, 0, bt)
    torch.cuda.synchronize()
    t_prefill = time.perf_counter() - t0
    out = [int(lg.argmax())]
    t0 = time.perf_counter()
    for i in range(args.new - 1):
        model.set_rows(1, [out[-1]], [args.prompt + i], [0], [bt.tolist()])
        out.append(int(model.decode(1)[0][0]))
    torch.cuda.synchronize()
    t_decode = time.perf_counter() - t0
    same = True
    if world > 1:
        mine = torch.tensor(out, dtype=torch.int64, device="cuda")
        every = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        same = all(torch.equal(e, every[0]) for e in every)
    model.poll_status()
    torch.cuda.synchronize()
    model.check_status()
    if rank == 0:
        print(json.dumps({"probe": "ep", "world": world, "experts_per_rank": cfg.num_experts // world, "ranks_agree": same,
                          "prefill_ms": round(t_prefill * 1e3, 2), "ms_per_token": round(t_decode / max(args.new - 1, 1) * 1e3, 3),
                          "tokens": out[:8]}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0 if same else 1


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("probe", choices=("batch", "divergence", "glue", "ep"))
    ap.add_argument("--preset", default="tiny-qwen4")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--prompt", type=int, default=96)
    ap.add_argument("--new", type=int, default=16)
    ap.add_argument("--rows", type=int, nargs="+", default=[1, 2, 4, 8])
    ap.add_argument("--quant", default="none")
    ap.add_argument("--top", type=int, default=25)
    args = ap.parse_args(argv)
    return {"batch": probe_batch, "divergence": probe_divergence, "glue": probe_glue, "ep": probe_ep}[args.probe](args)


if __name__ == "__main__":
    sys.exit(main())
