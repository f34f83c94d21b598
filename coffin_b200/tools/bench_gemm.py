"""Prefill-GEMM timing on one GPU: the tcgen05 kernels of this package against ``torch.matmul`` (cuBLAS).

    python -m coffin_b200.tools.bench_gemm [--rows 2048] [--int8]

For every projection shape of the named model (and its two-rank tensor-parallel shards) the product is timed
with CUDA events after warm-up, the weights rotating through four copies so that they come from HBM, not
from L2: the one-CTA kernel (``gemm_tc.cu``), the CTA-pair kernel (``gemm_tc2.cu``) with each tile width, the
width the library would choose, and ``torch.matmul``.  Each result is first checked against an fp32 product.
"""
from __future__ import annotations

import argparse


def _time(fn, n: int = 20) -> float:
    import torch
    for _ in range(3):
        fn(0)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n * 1e3


def main(argv=None) -> int:
    import torch
    from ..config import preset
    from ..ops import kernels as K
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="qwen35-4b")
    ap.add_argument("--rows", type=int, default=2048)
    ap.add_argument("--int8", action="store_true", help="W8A8 products (kind::i8) instead of bf16")
    args = ap.parse_args(argv)
    c, dev, M = preset(args.model), "cuda", args.rows
    H, I = c.hidden_size, c.intermediate_size
    lin_in = 2 * c.linear_num_key_heads * c.linear_key_head_dim + 2 * c.linear_num_value_heads * c.linear_value_head_dim \
        + 2 * c.linear_num_value_heads
    lin_in = (lin_in + 7) // 8 * 8
    lin_out = c.linear_num_value_heads * c.linear_value_head_dim
    shapes = [("delta-net in", lin_in, H), ("delta-net out", H, lin_out), ("gate|up", 2 * I, H), ("down", H, I),
              ("tp2 gate|up", I, H), ("tp2 down", H, I // 2)]
    hints = (("one-cta", -1), ("pair256", 1256), ("pair288", 1288), ("pair320", 1320), ("chosen", 0))
    for name, N, Kd in shapes:
        fl = 2.0 * M * N * Kd
        row = [f"{name} {M}x{N}x{Kd}"]
        out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        if args.int8:
            A = torch.randint(-127, 128, (M, Kd), device=dev, dtype=torch.int8)
            Ws = [torch.randint(-127, 128, (N, Kd), device=dev, dtype=torch.int8) for _ in range(4)]
            sa, sw = torch.rand(M, device=dev) * 0.01 + 1e-3, torch.rand(N, device=dev) * 0.01 + 1e-3
            ref = (A[:256].double() @ Ws[0].double().t()) * sa[:256].double()[:, None] * sw.double()[None, :]
            run = lambda i, bn: K.gemm_i8(A, sa, Ws[i % 4], sw, out=out, bn=bn)
        else:
            A = (torch.randn(M, Kd, device=dev) * 0.5).bfloat16()
            Ws = [(torch.randn(N, Kd, device=dev) * 0.05).bfloat16() for _ in range(4)]
            ref = (A[:256].float() @ Ws[0].float().t()).double()
            run = lambda i, bn: K.gemm(A, Ws[i % 4], out=out, bn=bn)
        for label, bn in hints:
            K.call("set_gemm_pair", 0 if bn == -1 else 1)
            bnv = 0 if bn == -1 else bn
            run(0, bnv)
            torch.cuda.synchronize()
            K.check_status()
            err = float((out[:256].double() - ref).abs().max() / ref.abs().max())
            assert err < 2e-2, f"{name} {label}: relative error {err:.3g}"
            us = _time(lambda i: run(i, bnv))
            row.append(f"{label} {us:.1f} us ({fl / us / 1e6:.0f} T/s)")
        K.call("set_gemm_pair", 1)
        if not args.int8:
            us = _time(lambda i: torch.matmul(A, Ws[i % 4].t(), out=out))
            row.append(f"torch.matmul {us:.1f} us ({fl / us / 1e6:.0f} T/s)")
        print(" | ".join(row), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
