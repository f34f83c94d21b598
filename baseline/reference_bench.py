"""Reference arm of ``bench.py``: the unmodified reference engine, installed under
``baseline/_ref``, on the same shape (Qwen3.5-4B-shaped bf16, prompt 2048, 256 greedy decode
tokens), through its own public API and stock code path.

The reference ships no NVIDIA backend; its ``reference`` backend pins ``device="cpu"``
(``backends/reference/__init__.py:59-72``), so this arm measures the reference's own torch path on
the host CPUs of the box.  A random-init checkpoint of the named shape is written to a temporary
directory in the HF safetensors layout the reference loads (``engine_api.create_model``), then
``engine.prefix_engine.PrefixCacheEngine`` (its paged single-stream engine) prefills and decodes.
Timing is host wall clock (the reference has no device timing on this backend).

Because a CPU step of this size takes tens of seconds, the warm-up steps use a short request
(64-token prompt, 4 tokens) to warm code paths, and a wall-clock budget counted from process start
(``COFFIN_REF_BUDGET_S``, default 600 s) ends the timed loop early; the JSON line reports the steps
actually completed (``steps``) beside the number asked for (``requested_steps``).  Under
``torch.distributed.run`` the launcher sets ``OMP_NUM_THREADS=1``; rank 0 restores a thread count of
half the host's cores, the other ranks have nothing to run and print nothing.  The reference's
figure is host wall clock around its own ``prefill`` / ``decode`` calls with token ids going in and
coming out as host lists, so it is already an end-to-end number and is reported as ``e2e`` too.
"""
from __future__ import annotations

import json
import os
import shutil
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"


def _line(**kw) -> dict:
    base = {"impl": "reference", "metric": "decode_tok_s", "unit": "tok/s", "higher_is_better": True,
            "scaling": "strong", "dtype": "bf16", "data": "synthetic"}
    base.update(kw)
    return base


def run_reference(args) -> dict:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not (REF / "engine_api.py").exists():
        return {"impl": "reference", "unavailable": "baseline/_ref is missing: the reference is not installed on this box"}
    if rank != 0:
        return {}        # nothing to run on this rank: the reference's only offline backend is the host CPU of rank 0
    import torch
    # the launcher pins OMP_NUM_THREADS=1 for multi-rank runs; this arm is one CPU process
    threads = int(os.environ.get("COFFIN_REF_THREADS", "0")) or max(1, (os.cpu_count() or 2) // 2)
    torch.set_num_threads(threads)
    sys.path.insert(0, str(ROOT))
    from coffin_b200.config import preset
    from coffin_b200.weights.init import random_state_dict, save_checkpoint
    budget = float(os.environ.get("COFFIN_REF_BUDGET_S", "600"))
    t_start = time.time()
    cfg = preset(args.model)
    tmp = Path(tempfile.mkdtemp(prefix="coffin_ref_ckpt_"))
    try:
        keep = ("A_log", "dt_bias")
        sd = random_state_dict(cfg, 0, dtype=torch.bfloat16, device="cpu")
        save_checkpoint(cfg, sd, tmp)
        del sd
        os.environ["COFFIN_BACKEND"] = "reference"
        sys.path.insert(0, str(REF))
        import engine_api                                   # the reference's public model API
        from engine.prefix_engine import PrefixCacheEngine  # its single-stream paged engine
        max_seq = args.prompt + args.new + 64
        nblk = (max_seq + 63) // 64 + 2
        with torch.inference_mode():
            model = engine_api.create_model(str(tmp), max_seq=max_seq, bench=False, paged=True)
            eng = PrefixCacheEngine(model, num_blocks=nblk, block_size=64, graph=False)
            g = torch.Generator().manual_seed(1234)
            W = max(3, args.warmup)
            for _ in range(W):                               # short warm-up requests
                p = torch.randint(0, cfg.vocab_size, (64,), generator=g).tolist()
                eng.radix.clear()
                lg = eng.prefill(p)
                eng.decode(lg, 4)
            pre_s, dec_s, done = [], [], 0
            for _ in range(args.steps):
                p = torch.randint(0, cfg.vocab_size, (args.prompt,), generator=g).tolist()
                eng.radix.clear()
                t0 = time.perf_counter()
                lg = eng.prefill(p)
                t1 = time.perf_counter()
                out = eng.decode(lg, args.new)
                t2 = time.perf_counter()
                pre_s.append(t1 - t0)
                dec_s.append(t2 - t1)
                done += 1
                if time.time() - t_start > budget:
                    break
        n_new = args.new
        dec_tok_s = n_new * done / sum(dec_s)
        pre_tok_s = args.prompt * done / sum(pre_s)
        return _line(value=dec_tok_s, prefill_tok_s=pre_tok_s, n_gpus=world, steps=done, warmup=W,
                     requested_steps=args.steps,
                     ms_per_step=(sum(pre_s) + sum(dec_s)) / done * 1e3, vs_baseline=dec_tok_s / 78.5,
                     ttft_ms_p50=sorted(pre_s)[len(pre_s) // 2] * 1e3,
                     tpot_ms_p50=sorted(dec_s)[len(dec_s) // 2] / n_new * 1e3,
                     config={"model": args.model, "global_batch": 1, "seq_len": args.prompt, "decode_tokens": n_new},
                     e2e={"value": dec_tok_s, "unit": "decode tok/s", "prefill_tok_s": pre_tok_s,
                          "h2d_bytes_per_step": args.prompt * 8, "d2h_bytes_per_step": n_new * 8,
                          "timing": "host wall clock around the reference's prefill/decode calls; token ids enter and "
                                    "leave as host lists (its backend computes on the host CPU, so no device copy exists)"},
                     notes={"parallelism": "single process: the reference's only offline backend is torch on the host CPU",
                            "cuda_graph": False, "warmup_kind": "short requests (64-token prompt, 4 tokens)",
                            "threads": threads, "budget_s": budget},
                     gpu_launches=0, device="cpu", timing="host wall clock")
    except Exception as exc:      # noqa: BLE001 - report instead of failing the driver
        return {"impl": "reference", "unavailable": f"reference run failed: {type(exc).__name__}: {str(exc)[:200]}"}
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny")
    ap.add_argument("--prompt", type=int, default=64)
    ap.add_argument("--new", type=int, default=8)
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=3)
    line = run_reference(ap.parse_args())
    if line:
        print(json.dumps(line))
