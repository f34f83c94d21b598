#!/usr/bin/env python
"""Headline benchmark: decode & prefill tokens/s of the Qwen3.5-4B-shaped bf16 hybrid model
(prompt 2048 random ids, 256 greedy decode tokens, batch 1, CUDA-graph decode), on N GPUs of one
node (N > 1 = tensor parallel, one rank per GPU under torchrun).

A "step" is one whole request: prefill of the 2048-token prompt, then 256 decode steps.  Both
phases are timed on the device with CUDA events (max over ranks); ``value`` is decode tokens/s,
``prefill_tok_s`` and TTFT/TPOT are reported beside it.  The ``e2e`` figure runs the same request
through the public engine API with the prompt copied from pinned host memory and every generated
token read back to the host, as a serving process does.

``--impl reference`` runs the unmodified reference engine (installed under ``baseline/_ref``) on
the same shape through its own API instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
BASELINE_DECODE_TOK_S = 78.5     # Qwen3.5-4B int8 single-stream decode, Hygon DCU (docs/FACTS-RUNTIME.md:9-16)
BASELINE_PREFILL_TOK_S = 1729.0

MODEL = "qwen35-4b"
PROMPT, NEW = 2048, 256


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.idx = gpu_index
        self.proc = None
        self.path = Path(tempfile.gettempdir()) / f"clocks_{os.getpid()}.csv"

    def start(self) -> None:
        try:
            self.fh = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.idx)], stdout=self.fh, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.fh.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.path.read_text().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        try:
            self.path.unlink()
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args) -> None:
    from baseline.reference_bench import run_reference
    line = run_reference(args)
    if line:                       # ranks other than 0 have nothing to run and print nothing
        print(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default=MODEL)
    ap.add_argument("--prompt", type=int, default=PROMPT)
    ap.add_argument("--new", type=int, default=NEW)
    ap.add_argument("--quant", default="none", choices=["none", "int8", "w4a8"])
    ap.add_argument("--kv-dtype", default="bf16", choices=["bf16", "int8"], help="KV pool storage")
    ap.add_argument("--parallel", default="tp", choices=["tp", "ep"],
                    help="N > 1: tensor parallel (default) or expert parallel (routed-MoE models)")
    ap.add_argument("--rows", type=int, default=1,
                    help="concurrent sequences: > 1 measures batched decode throughput (not the headline config)")
    ap.add_argument("--nccl", action="store_true", help="A/B baseline: all-reduces of prefill and wide decode buckets through NCCL between kernels")
    ap.add_argument("--mega", action="store_true", help="A/B: the persistent one-launch decode step instead of the graph of kernels")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--mma-ctas", type=int, default=0, help="tuning: tensor-core GEMV CTAs per SM")
    ap.add_argument("--gdn-tc", type=int, default=-1, help="tuning: 0 = fp32 SIMT delta-net chunk kernels, 1 = tensor-core (default)")
    ap.add_argument("--mma-stage", type=int, default=-1, help="tuning: GEMV weight batches per warp staged in shared memory before the wait")
    ap.add_argument("--mma-kcta", type=int, default=0, help="tuning: max CTAs sharing one 16-row GEMV block (1 = off)")
    ap.add_argument("--mma-prefetch", type=int, default=-1, help="tuning: GEMV sweep rounds prefetched into L2 before the dependency wait")
    ap.add_argument("--gemv-impl", default="", help="tuning: mma | scalar")
    ap.add_argument("--layers", type=int, default=0, help="Qwen4-exp: cut the geometry to its first N layers")
    ap.add_argument("--no-parity", action="store_true", help="multi-rank runs: skip the comparison with an unsharded copy on rank 0")
    ap.add_argument("--no-stream-gemv", action="store_true", help="tuning: register-staged GEMV for batch 1")
    ap.add_argument("--gemv-ctas", type=int, default=0, help="tuning: GEMV CTAs per SM (0 = library default)")
    ap.add_argument("--gemv-prefetch", type=int, default=-1, help="tuning: GEMV L2 prefetch-ahead (-1 = default)")
    args = ap.parse_args()
    if args.nccl:
        os.environ["COFFIN_TP_NCCL"] = "1"
    if args.mega:
        os.environ["COFFIN_MEGA"] = "1"
    sys.path.insert(0, str(ROOT))
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    import torch.distributed as dist
    from coffin_b200.config import preset
    from coffin_b200.engine.llm import LLM
    from coffin_b200.ops import kernels as K

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    W = max(3, args.warmup)
    if args.no_stream_gemv:
        K.STREAM_GEMV = False
    if args.gemv_impl:
        K.GEMV_IMPL = args.gemv_impl
    if args.gdn_tc >= 0:
        from coffin_b200.ops import _lib as _l5
        _l5.call_nostream("set_gdn_tc", args.gdn_tc)
    if args.mma_stage >= 0:
        from coffin_b200.ops import _lib as _l4
        _l4.call_nostream("set_mma_gemv_stage", args.mma_stage)
    if args.mma_kcta:
        from coffin_b200.ops import _lib as _l3
        _l3.call_nostream("set_mma_gemv_kcta", args.mma_kcta)
    if args.mma_prefetch >= 0:
        from coffin_b200.ops import _lib as _l2
        _l2.call_nostream("set_mma_gemv_prefetch", args.mma_prefetch)
    if args.mma_ctas:
        from coffin_b200.ops import _lib as _l
        _l.call_nostream("set_mma_gemv_opts", args.mma_ctas)
    if args.gemv_ctas or args.gemv_prefetch >= 0:
        from coffin_b200.ops import _lib
        _lib.call_nostream("set_gemv_opts", args.gemv_ctas or 2, 1 if args.gemv_prefetch != 0 else 0)
    cfg = preset(args.model)
    if "qwen4" in args.model:
        return bench_qwen4(args, cfg, W)
    if args.rows > 1:
        return bench_rows(args, cfg, W)
    llm = LLM.from_random(cfg, seed=0, max_seq=args.prompt + args.new + 64, max_num_seqs=1,
                          graph=not args.no_graph, pdl=not args.no_pdl, max_chunk=min(args.prompt, 2048), quant=args.quant,
                          kv_dtype=args.kv_dtype,
                          **({"ep_world": world, "ep_rank": rank} if args.parallel == "ep" and world > 1
                             else {"tp_world": world, "tp_rank": rank}))
    model = llm.model
    g = torch.Generator().manual_seed(1234)
    prompts = [torch.randint(0, cfg.vocab_size, (args.prompt,), generator=g).pin_memory()
               for _ in range(W + args.steps)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------- device-timed kernel path ------------------------------------------
    ev = lambda: torch.cuda.Event(enable_timing=True)
    pre_ms, dec_ms = [], []
    launches = 0
    sampler = ClockSampler(local)
    for i, p in enumerate(prompts):
        timed = i >= W
        if i == W:
            barrier()
            if rank == 0:
                sampler.start()
            l0 = K.LAUNCHES
            r0 = llm.graph_launches_replayed
            t_wall = time.perf_counter()
        e0, e1, e2 = ev(), ev(), ev()
        dev_prompt = p.cuda(non_blocking=True)
        e0.record()
        first = llm.device_prefill(dev_prompt)
        e1.record()
        toks = llm.device_decode(first, args.new)
        e2.record()
        e2.synchronize()
        if i == W:
            # greedy tokens of the first timed prompt: the same value at every N shows that the
            # tensor-parallel output is the single-GPU output
            import zlib
            token_crc = zlib.crc32(torch.cat([first.view(-1), toks.view(-1)]).cpu().numpy().tobytes())
        if timed:
            pre_ms.append(e0.elapsed_time(e1))
            dec_ms.append(e1.elapsed_time(e2))
    barrier()
    wall_s = time.perf_counter() - t_wall
    clocks = sampler.stop() if rank == 0 else {}
    launches = (K.LAUNCHES - l0) + (llm.graph_launches_replayed - r0)
    K.check_status()
    stats = torch.tensor([sum(pre_ms), sum(dec_ms)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    pre_total, dec_total = stats.tolist()
    steps = args.steps
    decode_tok_s = args.new * steps / (dec_total / 1e3)
    prefill_tok_s = args.prompt * steps / (pre_total / 1e3)

    # ---------------- end to end through the public API ---------------------------------
    e2e = None
    if not args.no_e2e:
        e2e_dec, e2e_pre, e2e_steps = [], [], 0
        use = prompts[: max(3, min(W, 3)) + steps]
        for i, p in enumerate(use):
            # args.new + 1 tokens: the first comes out of the prefill, the other args.new are decode steps,
            # so the decode phase covers exactly as many steps as the device-timed figure
            out = llm.generate(p, max_new_tokens=args.new + 1, ignore_eos=True)
            if i >= len(use) - steps:
                e2e_dec.append(out.decode_ms)
                e2e_pre.append(out.prefill_ms)
                e2e_steps += len(out.tokens) - 1
        s2 = torch.tensor([sum(e2e_pre), sum(e2e_dec)], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(s2, op=dist.ReduceOp.MAX)
        e2e = {"value": e2e_steps / (s2[1].item() / 1e3), "unit": "decode tok/s",
               "prefill_tok_s": args.prompt * steps / (s2[0].item() / 1e3),
               "h2d_bytes_per_step": args.prompt * 8 + args.new * 8,
               "d2h_bytes_per_step": (args.new + 1) * 8,
               "timing": "host wall clock around the phases of LLM.generate: prompt copied from pinned host memory, "
                         "every token read back to the host before the next step is staged"}
    wbytes = llm.model.weight_bytes() if hasattr(llm.model, "weight_bytes") else 0
    parity = multi_rank_parity(args, cfg, llm, prompts[W], world, rank) if world > 1 and not args.no_parity else None
    if rank == 0:
        line = {
            "metric": "decode_tok_s", "value": decode_tok_s, "unit": "tok/s", "n_gpus": world,
            "steps": steps, "warmup": W, "ms_per_step": (pre_total + dec_total) / steps,
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": decode_tok_s / BASELINE_DECODE_TOK_S, "dtype": {"none": "bf16", "int8": "int8-w8a8", "w4a8": "int4-w4a8"}.get(args.quant, args.quant), "data": "synthetic",
            "prefill_tok_s": prefill_tok_s, "prefill_vs_baseline": prefill_tok_s / BASELINE_PREFILL_TOK_S,
            "ttft_ms_p50": statistics.median(pre_ms), "tpot_ms_p50": statistics.median(dec_ms) / args.new,
            "config": {"model": args.model, "global_batch": 1, "seq_len": args.prompt, "decode_tokens": args.new,
                       "parallelism": f"{args.parallel}{world}" if world > 1 else "single"},
            "notes": {"cuda_graph": not args.no_graph, "kv_dtype": args.kv_dtype,
                      "cache": f"weights streamed by this rank every decode step ({wbytes / 1e9:.2f} GB; a routed-MoE step reads its dense part plus the selected experts) far exceed the 126 MB L2, no flush needed",
                      "weights": "random-init N(0,0.02)"},
            "token_crc": token_crc, "multi_rank_parity": parity,
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "wall_s": wall_s, "impl": "ours",
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        from coffin_b200.parallel.control import shutdown
        dist.barrier()
        tp = getattr(llm.model, "tp", None)
        llm.model._graphs.clear()
        if tp is not None:
            tp.close()
        shutdown(timeout_s=10.0)


def multi_rank_parity(args, cfg, llm, prompt, world: int, rank: int):
    """Outside the timed region: tie the sharded model's output to the single-GPU model's.  All ranks run
    the prompt of the first timed step and 8 teacher-forced decode steps through the sharded model with
    full logits; rank 0 then builds an UNSHARDED copy of the same random-init model on its own GPU, feeds it
    the same tokens and compares logits (max relative difference on the scale of the largest logit, top-1
    agreement where the single-GPU margin is clear).  Greedy token streams of random-init weights
    diverge at the first near-tie, which is why a CRC of sampled tokens cannot serve as this proof."""
    import torch
    import torch.distributed as dist
    from coffin_b200.engine.llm import LLM
    n_steps = 8
    toks = prompt.cuda()
    g = torch.Generator().manual_seed(77)
    forced = torch.randint(0, cfg.vocab_size, (n_steps,), generator=g).tolist()

    def run(one: LLM):
        m = one.model
        if hasattr(m, "full_logits"):
            m.full_logits = True
        m.zero_state(one._slot)
        T, lg = toks.numel(), None
        for s0 in range(0, T, m.max_chunk):
            s1 = min(T, s0 + m.max_chunk)
            lg = m.prefill(toks[s0:s1], s0, one._slot, one._bt, want_logits=s1 == T)
        out = [lg.float().clone()]
        for i, t in enumerate(forced):
            m.set_rows(1, [t], [T + i], [one._slot], [one._bt.tolist()])
            out.append(m.decode(1, graph=False)[1][0].float().clone())
        return torch.stack(out)

    with torch.no_grad():
        sharded = run(llm)
        dist.barrier()
        res = None
        if rank == 0:
            free = torch.cuda.mem_get_info()[0]
            need = sum(v for v in [llm.model.weight_bytes() * world]) * 2.5
            if free < need:
                res = {"skipped": f"{free / 1e9:.0f} GB free on rank 0, the unsharded copy needs about {need / 1e9:.0f} GB"}
            else:
                single = LLM.from_random(cfg, seed=0, max_seq=args.prompt + args.new + 64, max_num_seqs=1, graph=False,
                                         max_chunk=min(args.prompt, 2048), quant=args.quant, kv_dtype=args.kv_dtype)
                ref = run(single)
                scale = ref.abs().amax(-1, keepdim=True)
                rel = float(((sharded - ref).abs() / scale).max())
                top2 = ref.topk(2, dim=-1).values
                margin = (top2[:, 0] - top2[:, 1]) / scale[:, 0]
                # a top-1 can only be expected to survive where the single-GPU margin exceeds the difference seen
                noise = ((sharded - ref).abs() / scale).amax(-1)
                clear = margin > 2 * noise
                same = bool((sharded.argmax(-1)[clear] == ref.argmax(-1)[clear]).all())
                cos = torch.nn.functional.cosine_similarity(sharded, ref, dim=-1)
                t5s, t5r = sharded.topk(5, dim=-1).indices, ref.topk(5, dim=-1).indices
                overlap = [len(set(a.tolist()) & set(b.tolist())) for a, b in zip(t5s, t5r)]
                res = {"positions": int(ref.shape[0]), "max_rel_logit_diff": round(rel, 5),
                       "min_cosine": round(float(cos.min()), 5),
                       "top1_equal_positions": int((sharded.argmax(-1) == ref.argmax(-1)).sum()),
                       "top5_overlap_min": int(min(overlap)),
                       "median_top2_margin_rel": round(float(margin.median()), 5),
                       "clear_margin_positions": int(clear.sum()), "top1_equal_where_clear": same,
                       "what": f"{args.parallel}{world} logits vs an unsharded copy on rank 0 (prompt + {n_steps} teacher-forced steps); "
                               "random-init logits have top-2 margins of the order of the bf16 difference between the two "
                               "summation orders, so the whole-vector figures (cosine, top-5 overlap) carry the comparison"}
                del single, ref
                torch.cuda.empty_cache()
        dist.barrier()
    return res


def bench_qwen4(args, cfg, W: int) -> None:
    """Qwen4-exp family (hyper-connected lanes, QSA attention, 512-expert MoE): device-timed prefill of one
    prompt and single-sequence decode on one GPU.  The decode step replays as a CUDA graph when the model has no
    n-gram layer (`COFFIN_QWEN4_GRAPH=0`: eager);
    weights are drawn and quantised tensor by tensor (`--quant w4a8` for the full 48-layer geometry, whose
    experts would not fit in bf16); `--layers N` cuts the geometry to its first N layers."""
    import dataclasses
    import statistics
    import torch
    from coffin_b200.models.qwen4exp.model import Qwen4ExpModel
    from coffin_b200.models.qwen4exp.weights import LazyRandomStateDict
    from coffin_b200.ops import kernels as K
    if args.layers and args.layers < cfg.num_hidden_layers:
        cfg = dataclasses.replace(cfg, num_hidden_layers=args.layers, layer_types=cfg.layer_types[:args.layers],
                                  ple_layer_ids=tuple(i for i in cfg.ple_layer_ids if i <= args.layers))
    torch.cuda.set_device(0)
    chunk = min(args.prompt, 2048)
    model = Qwen4ExpModel(cfg, LazyRandomStateDict(cfg, 0), max_seq=args.prompt + args.new + 64, num_slots=1,
                          max_chunk=chunk, quant=args.quant)
    g = torch.Generator().manual_seed(1234)
    prompts = [torch.randint(2, cfg.vocab_size, (args.prompt,), generator=g).pin_memory() for _ in range(W + args.steps)]
    bt = torch.arange(1, model.max_blocks_per_seq + 1, dtype=torch.int32, device="cuda")
    ev = lambda: torch.cuda.Event(enable_timing=True)
    pre_ms, dec_ms = [], []
    sampler = ClockSampler(0)
    l0 = 0
    with torch.no_grad():
        for i, p in enumerate(prompts):
            if i == W:
                torch.cuda.synchronize()
                sampler.start()
                l0 = K.LAUNCHES
            e0, e1, e2 = ev(), ev(), ev()
            dev = p.cuda(non_blocking=True)
            model.zero_state(0)
            e0.record()
            lg = None
            for s0 in range(0, args.prompt, chunk):
                s1 = min(args.prompt, s0 + chunk)
                lg = model.prefill(dev[s0:s1], s0, 0, bt, want_logits=s1 == args.prompt)
            tok = int(lg.argmax())
            e1.record()
            for j in range(args.new):
                model.set_rows(1, [tok], [args.prompt + j], [0], [bt.tolist()])
                tok = int(model.decode(1)[0][0])
            e2.record()
            e2.synchronize()
            if i >= W:
                pre_ms.append(e0.elapsed_time(e1))
                dec_ms.append(e1.elapsed_time(e2))
    clocks = sampler.stop()
    launches = K.LAUNCHES - l0
    K.check_status()
    dec_tok_s = args.new * args.steps / (sum(dec_ms) / 1e3)
    line = {"metric": "decode_tok_s", "value": dec_tok_s, "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": W,
            "ms_per_step": (sum(pre_ms) + sum(dec_ms)) / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": {"none": "bf16", "int8": "int8-w8a8", "w4a8": "int4-w4a8"}.get(args.quant, args.quant),
            "data": "synthetic", "prefill_tok_s": args.prompt * args.steps / (sum(pre_ms) / 1e3),
            "ttft_ms_p50": statistics.median(pre_ms), "tpot_ms_p50": statistics.median(dec_ms) / args.new,
            "config": {"model": args.model, "layers": cfg.num_hidden_layers, "global_batch": 1, "seq_len": args.prompt,
                       "decode_tokens": args.new, "parallelism": "single"},
            "notes": {"cuda_graph": bool(model._graphs), "weights": "random-init, drawn and quantised per tensor",
                      "weight_gb": round(model.weight_bytes() / 1e9, 2),
                      "timing": "CUDA events; the decode loop reads every token back (eager step, host-staged rows)"},
            "clocks": clocks, "gpu_launches": launches, "impl": "ours"}
    print(json.dumps(line), flush=True)


def bench_rows(args, cfg, W: int) -> None:
    """Batched decode throughput: ``--rows`` sequences are prefilled one after the other and then
    advance together, one CUDA-graph step per token (buckets above 8 rows run their projections on the
    tcgen05 GEMM).  On N > 1 GPUs the model is tensor parallel (or expert parallel with ``--parallel
    ep``); ``--nccl`` routes the all-reduces through NCCL between kernels instead of the exchange fused
    into the GEMM epilogue (the A/B baseline).  Device-timed, max over ranks; ``value`` is the
    aggregate decode tok/s."""
    import json
    import statistics
    import torch
    import torch.distributed as dist
    from coffin_b200.engine.llm import LLM
    from coffin_b200.ops import kernels as K
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    R = args.rows
    par = ({"ep_world": world, "ep_rank": rank} if args.parallel == "ep" and world > 1 else {"tp_world": world, "tp_rank": rank})
    llm = LLM.from_random(cfg, seed=0, max_seq=args.prompt + args.new + 64, max_num_seqs=R, max_chunk=min(args.prompt, 2048),
                          quant=args.quant, kv_dtype=args.kv_dtype, **par)
    m = llm.model
    m.full_logits = False
    M = m.bucket_for(R)
    nblk = m.max_blocks_per_seq
    tables = [list(range(r * nblk, (r + 1) * nblk)) for r in range(R)]
    g = torch.Generator().manual_seed(1234)
    ev = lambda: torch.cuda.Event(enable_timing=True)
    pre_ms, dec_ms = [], []
    chunk = m.max_chunk
    for it in range(W + args.steps):
        prompts = [torch.randint(0, cfg.vocab_size, (args.prompt,), generator=g).pin_memory() for _ in range(R)]
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1, e2 = ev(), ev(), ev()
        e0.record()
        firsts = []
        for r in range(R):
            m.zero_state(r)
            dev = prompts[r].cuda(non_blocking=True)
            bt = torch.tensor(tables[r], dtype=torch.int32, device="cuda")
            lg = None
            for s0 in range(0, args.prompt, chunk):
                s1 = min(args.prompt, s0 + chunk)
                lg = m.prefill(dev[s0:s1], s0, r, bt, want_logits=s1 == args.prompt)
            firsts.append(int(lg.argmax()))
        e1.record()
        m.set_rows(M, firsts, [args.prompt] * R, list(range(R)), tables)
        for _ in range(args.new):
            m.decode(M, graph=True, advance=True)
        e2.record()
        e2.synchronize()
        if it >= W:
            pre_ms.append(e0.elapsed_time(e1))
            dec_ms.append(e1.elapsed_time(e2))
    K.check_status()
    stats = torch.tensor([sum(pre_ms), sum(dec_ms)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    pre_total, dec_total = stats.tolist()
    dec_tok_s = R * args.new * len(dec_ms) / (dec_total / 1e3)
    if rank == 0:
        print(json.dumps({"metric": "batched_decode_tok_s", "value": dec_tok_s, "unit": "tok/s", "n_gpus": world,
                          "steps": args.steps, "warmup": W, "higher_is_better": True,
                          "prefill_tok_s": R * args.prompt * len(pre_ms) / (pre_total / 1e3),
                          "step_ms": dec_total / len(dec_ms) / args.new,
                          "dtype": {"none": "bf16", "int8": "int8-w8a8", "w4a8": "int4-w4a8"}[args.quant], "data": "synthetic",
                          "config": {"model": args.model, "global_batch": R, "seq_len": args.prompt, "decode_tokens": args.new,
                                     "parallelism": f"{args.parallel}{world}" if world > 1 else "single"},
                          "notes": {"bucket": M, "cuda_graph": True, "kv_dtype": args.kv_dtype, "exchange": "nccl" if os.environ.get("COFFIN_TP_NCCL") == "1" else "fused peer-memory",
                                    "launches_per_step": m.launches_per_step(M), "weight_gb_per_rank": round(m.weight_bytes() / 1e9, 2)},
                          "impl": "ours"}), flush=True)
    if world > 1:
        from coffin_b200.parallel.control import shutdown
        dist.barrier()
        m._graphs.clear()
        if getattr(m, "tp", None) is not None:
            m.tp.close()
        shutdown(timeout_s=10.0)


if __name__ == "__main__":
    main()
