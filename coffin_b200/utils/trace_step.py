"""In-graph timeline of one decode step (or, with ``--prefill``, of the prefill pass).

    python -m coffin_b200.utils.trace_step --model qwen35-4b --prompt 2048 [--layers 8] [--rows 1] [--prefill]

Every kernel of the library stamps ``%globaltimer`` when its first block enters and when its
programmatic dependency has resolved (``_C/common.cuh``).  This tool installs the trace buffer,
captures the decode graph while recording the kernel names, replays it a few times and prints, for
the last replay, each kernel's *span* (time from its own ready stamp to the next kernel's ready
stamp - what the kernel costs inside the graph, overlap with its neighbours included) and its
*lead* (how long before its dependency resolved it was already resident, i.e. how much prologue
the dependent launch bought).  A serialising profiler cannot show either.  Kernels launched by
torch itself (copies) carry no stamps; their time is folded into the span of the kernel before.
"""
from __future__ import annotations

import argparse
import collections
import ctypes
import dataclasses
import re

import torch

MAX_EVENTS = 8192


class StepTrace:
    """Owns the device trace buffer; ``with StepTrace() as t: ...; t.read()``."""

    def __init__(self, device="cuda") -> None:
        from ..ops import _lib
        self._lib = _lib
        self.buf = torch.zeros(2 + 2 * MAX_EVENTS, dtype=torch.int64, device=device)

    def __enter__(self) -> "StepTrace":
        self._lib.call_nostream("trace_set", self.buf)
        return self

    def __exit__(self, *exc) -> None:
        self._lib.call_nostream("trace_set", None)

    def reset(self) -> None:
        torch.cuda.synchronize()
        self.buf.zero_()
        torch.cuda.synchronize()

    def record_names(self, on: bool) -> None:
        self._lib.call_nostream("trace_record_names", int(on))

    def names(self) -> list[str]:
        lib = self._lib.lib()
        lib.cb_trace_name_count.restype = ctypes.c_int64
        out = []
        raw = ctypes.create_string_buffer(512)
        for i in range(int(lib.cb_trace_name_count())):
            lib.cb_trace_get_name(ctypes.c_int64(i), raw, ctypes.c_int64(512))
            out.append(raw.value.decode())
        return out

    def read(self) -> tuple[list[int], list[int]]:
        torch.cuda.synchronize()
        h = self.buf.cpu().tolist()
        n = min(h[0], h[1], MAX_EVENTS)
        return [h[2 + 2 * i] for i in range(n)], [h[3 + 2 * i] for i in range(n)]


def short_name(mangled: str) -> str:
    """``gemv_mma_kernel<010>`` from the mangled symbol (name found through its length prefix)."""
    end = mangled.find("_kernel")
    base = mangled
    if end >= 0:
        end += len("_kernel")
        for n in range(8, 48):
            if mangled[end - n - len(str(n)):end - n] == str(n):
                base = mangled[end - n:end]
                break
    flags = "".join(re.findall(r"L[bi](\d+)E", mangled[end:] if end >= 0 else mangled))
    return f"{base}<{flags}>" if flags else base


def trace_decode(model, M: int, replays: int = 4):
    """Returns ``[(name, lead_us, span_us)]`` of one replay of bucket ``M``'s decode graph."""
    with StepTrace(model.device) as t:
        model._graphs.pop(model._gkey(M, False), None)
        t.record_names(True)
        model.capture(M, warmup=0)
        t.record_names(False)
        names = t.names()
        t.reset()
        for _ in range(replays):
            model.decode(M, graph=True)
        entry, ready = t.read()
    n = len(names)
    if n == 0 or len(ready) < n * replays:
        raise RuntimeError(f"trace holds {len(ready)} events for {n} kernels x {replays} replays")
    lo = n * (replays - 1)
    rows = []
    for i in range(n):
        end = ready[lo + i + 1] if i + 1 < n else None
        span = (end - ready[lo + i]) / 1e3 if end is not None else float("nan")
        rows.append((short_name(names[i]), (ready[lo + i] - entry[lo + i]) / 1e3, span))
    step_us = (ready[lo + n - 1] - ready[lo]) / 1e3
    prev_us = (ready[lo] - ready[lo - n]) / 1e3 if replays > 1 else float("nan")
    return rows, step_us, prev_us


def trace_prefill(llm, prompt: torch.Tensor):
    """``[(name, lead_us, span_us)]`` of one prefill pass of ``prompt`` (eager launches, same stamps)."""
    with StepTrace(llm.model.device) as t:
        for _ in range(2):
            llm.device_prefill(prompt)
        t.reset()
        t.record_names(True)
        llm.device_prefill(prompt)
        t.record_names(False)
        names = t.names()
        entry, ready = t.read()
    n = min(len(names), len(ready))
    rows = []
    for i in range(n):
        span = (ready[i + 1] - ready[i]) / 1e3 if i + 1 < n else float("nan")
        rows.append((short_name(names[i]), (ready[i] - entry[i]) / 1e3, span))
    return rows, (ready[n - 1] - ready[0]) / 1e3, float("nan")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen35-4b")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--quant", default="none")
    ap.add_argument("--all", action="store_true", help="print every kernel, not only the first layers")
    ap.add_argument("--prefill", action="store_true", help="trace the prefill pass of the prompt instead of a decode step")
    ap.add_argument("--mma-stage", type=int, default=-1, help="tuning: GEMV weight batches per warp staged in shared memory before the wait")
    ap.add_argument("--mma-kcta", type=int, default=0, help="max CTAs sharing one 16-row GEMV block (1 = off)")
    ap.add_argument("--mma-prefetch", type=int, default=-1, help="GEMV sweep rounds prefetched into L2 before the wait")
    args = ap.parse_args()
    from ..config import preset
    from ..engine.llm import LLM
    from ..ops import _lib
    if args.mma_prefetch >= 0:
        _lib.call_nostream("set_mma_gemv_prefetch", args.mma_prefetch)
    if args.mma_kcta:
        _lib.call_nostream("set_mma_gemv_kcta", args.mma_kcta)
    if args.mma_stage >= 0:
        _lib.call_nostream("set_mma_gemv_stage", args.mma_stage)
    cfg = preset(args.model)
    if args.layers and args.layers < cfg.num_hidden_layers:
        cfg = dataclasses.replace(cfg, num_hidden_layers=args.layers, layer_types=cfg.layer_types[:args.layers])
    import os
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:                       # tensor-parallel trace: run under torch.distributed.run
        import torch.distributed as dist
        torch.cuda.set_device(local)
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    llm = LLM.from_random(cfg, seed=0, max_seq=args.prompt + 64, max_num_seqs=max(1, args.rows),
                          max_chunk=min(args.prompt, 2048), quant=args.quant, tp_world=world, tp_rank=rank,
                          device=f"cuda:{local}")
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab_size, (args.prompt,), generator=g).cuda()
    first = llm.device_prefill(prompt)
    m = llm.model
    if args.prefill:
        rows, step_us, prev_us = trace_prefill(llm, prompt)
        if rank == 0:
            _report(rows, step_us, prev_us, args, what="prefill")
        if world > 1:
            import torch.distributed as dist
            from ..parallel.control import shutdown
            dist.barrier()
            m.tp.close()
            shutdown(timeout_s=10.0)
        return
    M = m.bucket_for(args.rows)
    bt = list(range(m.max_blocks_per_seq))
    m.set_rows(M, [int(first[0])] * args.rows, [args.prompt] * args.rows, list(range(args.rows)), [bt] * args.rows)
    for _ in range(3):
        m.decode(M, graph=True)
    rows, step_us, prev_us = trace_decode(m, M)
    if world > 1:
        from ..parallel.control import shutdown
        import torch.distributed as dist
        dist.barrier()
    if rank == 0:
        _report(rows, step_us, prev_us, args)
    if world > 1:
        m._graphs.clear()
        m.tp.close()
        shutdown(timeout_s=10.0)


def _report(rows, step_us, prev_us, args, what: str = "decode step") -> None:
    print(f"{what} (first ready -> last ready): {step_us:.1f} us; replay period {prev_us:.1f} us; {len(rows)} kernels")
    agg = collections.OrderedDict()
    for name, lead, span in rows:
        a = agg.setdefault(name, [0, 0.0, 0.0])
        a[0] += 1
        a[1] += lead
        a[2] += 0.0 if span != span else span
    print(f"{'kernel':44s} {'n':>4s} {'span us':>9s} {'avg':>7s} {'avg lead':>9s}")
    for name, (n, lead, span) in agg.items():
        print(f"{name:44s} {n:4d} {span:9.1f} {span / n:7.2f} {lead / n:9.2f}")
    limit = len(rows) if args.all else min(len(rows), 14)
    print("-- per kernel, in order --")
    for name, lead, span in rows[:limit]:
        print(f"{span:8.2f} us  lead {lead:6.2f}  {name}")


if __name__ == "__main__":
    main()
