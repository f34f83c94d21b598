"""Run one function as ``world`` rank processes with a hard time limit.

Each rank's stdout/stderr goes to a log file; a rank that is still alive at the deadline is ended
by its PID and the test fails with the tail of every log (and the Python stacks that
``faulthandler`` dumped), so a stuck collective shows where it is stuck instead of running into the
suite's timeout.
"""
from __future__ import annotations

import faulthandler
import multiprocessing as mp
import os
import sys
import tempfile
import time
from pathlib import Path


def _entry(target, rank, world, args, log_path, env, dump_after):
    os.environ.update(env)
    log = open(log_path, "w", buffering=1)
    os.dup2(log.fileno(), 1)
    os.dup2(log.fileno(), 2)
    sys.stdout = sys.stderr = log
    faulthandler.enable(file=log)
    faulthandler.dump_traceback_later(dump_after, repeat=False, file=log)
    target(rank, world, *args)
    faulthandler.cancel_dump_traceback_later()


def run_ranks(target, world: int, args=(), timeout: float = 150.0, env: dict | None = None) -> None:
    ctx = mp.get_context("spawn")
    out_dir = Path(os.environ.get("COFFIN_RANK_LOG_DIR") or tempfile.mkdtemp(prefix="ranks_"))
    out_dir.mkdir(parents=True, exist_ok=True)
    stamp = f"{target.__name__}_{int(time.time())}"
    logs = [out_dir / f"{stamp}_rank{r}.log" for r in range(world)]
    env = {k: str(v) for k, v in (env or {}).items()}
    procs = [ctx.Process(target=_entry, args=(target, r, world, args, str(logs[r]), env, max(5.0, timeout - 20.0)))
             for r in range(world)]
    for p in procs:
        p.start()
    deadline = time.monotonic() + timeout
    for p in procs:
        p.join(max(0.1, deadline - time.monotonic()))
    stuck = [r for r, p in enumerate(procs) if p.is_alive()]
    for p in procs:
        if p.is_alive():
            p.terminate()
    for p in procs:
        p.join(10)
        if p.is_alive():
            p.kill()
    bad = [r for r, p in enumerate(procs) if p.exitcode != 0]
    if stuck or bad:
        tails = []
        for r, lp in enumerate(logs):
            text = lp.read_text(errors="replace") if lp.exists() else ""
            tails.append(f"--- rank {r} (exit {procs[r].exitcode}) ---\n{text[-3000:]}")
        raise AssertionError(f"ranks stuck={stuck} failed={bad} after {timeout:.0f}s\n" + "\n".join(tails))
