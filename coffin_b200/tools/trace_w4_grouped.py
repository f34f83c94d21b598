"""Per-k-block timeline of the int4 grouped expert GEMM (``_C/gemm_w4_tc.cu``) on one GPU.

    python -m coffin_b200.tools.trace_w4_grouped [--tokens 2048] [--experts 256] [--topk 8] [--hidden 2048] [--inter 512]

CTA 0 stamps ``%globaltimer`` for its first k-blocks: when a dequant group starts on a k-block, when its
bf16 rows are written, when the proxy fence has passed, and when the MMA thread issues that k-block's
products.  The gaps show what paces the kernel (expansion, hand-off, tensor core / shared-memory bandwidth).
Also prints the CUDA-event time of the gate|up (+SwiGLU) and down products of one routed-MoE layer shape.
"""
from __future__ import annotations

import argparse


def main(argv=None) -> int:
    import torch
    from ..ops import kernels as K
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--inter", type=int, default=512)
    ap.add_argument("--rows", type=int, default=40, help="k-blocks to print")
    a = ap.parse_args(argv)
    dev, T, k, E, H, I = "cuda", a.tokens, a.topk, a.experts, a.hidden, a.inter
    g = torch.Generator().manual_seed(0)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).int()
    x = (torch.randn(T, H, generator=g) * 0.5).bfloat16().to(dev)
    gq = torch.randint(0, 256, (E, 2 * I, H // 2), dtype=torch.uint8, device=dev)
    gs = torch.rand(E, 2 * I, H // 128, device=dev) * 0.01
    dq = torch.randint(0, 256, (E, H, I // 2), dtype=torch.uint8, device=dev)
    ds = torch.rand(E, H, I // 128, device=dev) * 0.01
    d = K.moe_dispatch(idx.to(dev), E)
    xs = x.index_select(0, d["src_tok"])
    inter = torch.empty(T * k, I, dtype=torch.bfloat16, device=dev)
    y = torch.empty(T * k, H, dtype=torch.bfloat16, device=dev)

    def timed(fn) -> float:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 5 * 1e3

    print(f"gate|up + SwiGLU [{T * k} x {2 * I} x {H}]: {timed(lambda: K.gemm_w4_grouped(xs, gq, gs, d, swiglu=True, out=inter)):.1f} us")
    print(f"down             [{T * k} x {H} x {I}]: {timed(lambda: K.gemm_w4_grouped(inter, dq, ds, d, out=y)):.1f} us")
    tr = torch.zeros(96 * 4, dtype=torch.int64, device=dev)
    K.gemm_w4_grouped(xs, gq, gs, d, swiglu=True, out=inter, trace=tr)
    torch.cuda.synchronize()
    K.check_status()
    t = tr.cpu().reshape(96, 4)
    t0 = int(t[0, 0])
    print("k-block  start  rows-written  fenced  mma-issued   (ns after the first start)   expand  hand-off")
    for i in range(min(a.rows, 96)):
        s, w, f, m = (int(v) - t0 for v in t[i])
        print(f"{i:7d} {s:6d} {w:13d} {f:7d} {m:11d}   {w - s:32d} {m - f:9d}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
