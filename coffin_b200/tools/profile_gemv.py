"""Stand-alone decode-projection workload for profiling and bandwidth measurement.

    python -m coffin_b200.tools.profile_gemv --n 151936 --k 2560 --variant stream --iters 5

Runs one single-row projection shape several times (a buffer larger than L2 is rewritten between
iterations so that every run reads the weights from HBM) and prints the CUDA-event time and the
achieved bandwidth per iteration.  Under ``ncu`` use ``-k regex:gemv -s <warm-up> -c 1``.
"""
from __future__ import annotations

import argparse

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--n", type=int, default=151936)
    ap.add_argument("--k", type=int, default=2560)
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--variant", default="mma", choices=["mma", "stream", "reg"])
    ap.add_argument("--swiglu", action="store_true")
    ap.add_argument("--norm", action="store_true")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    args = ap.parse_args()
    from ..ops import kernels as K
    K.GEMV_IMPL = "mma" if args.variant == "mma" else "scalar"
    K.STREAM_GEMV = args.variant == "stream"
    dev = "cuda"
    rows = args.n * (2 if args.swiglu else 1)
    W = (torch.randn(rows, args.k, device=dev) * 0.02).to(torch.bfloat16)
    x = torch.randn(args.rows, args.k, device=dev).to(torch.bfloat16)
    gain = torch.ones(args.k, device=dev)
    out = torch.empty(args.rows, args.n, dtype=torch.bfloat16, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    norm = (x, None, gain, None, 1e-6) if args.norm else None
    nbytes = W.numel() * 2
    for i in range(args.warmup + args.iters):
        if not args.no_flush:
            flush.fill_(i & 0xff)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        K.gemv(W, None if args.norm else x, out, swiglu=args.swiglu, norm=norm)
        e1.record()
        e1.synchronize()
        if i >= args.warmup:
            ms = e0.elapsed_time(e1)
            print(f"{args.variant} n={args.n} k={args.k} rows={args.rows}: {ms * 1e3:.1f} us  {nbytes / ms / 1e6:.0f} GB/s")


if __name__ == "__main__":
    main()
