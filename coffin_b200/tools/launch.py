"""Start a multi-rank engine on one node, check it, and tear it down cleanly.

    python -m coffin_b200.tools.launch --parallel tp --gpus 4 --preset qwen35-4b --sock /tmp/coffin.sock
    python -m coffin_b200.tools.launch --parallel ep --gpus 8 --model /ckpt/moe-w4a8 --smoke "Hello"

Steps (each with its own time limit, as in the reference's launch recipes,
``tools/launch_occamy_ep.sh:51-131``): probe every GPU with a tiny matmul in a child process, start
one engine process per GPU (``RANK`` / ``LOCAL_RANK`` / ``WORLD_SIZE`` / ``MASTER_ADDR`` /
``MASTER_PORT`` / ``COFFIN_PARALLEL`` set; every rank sees all GPUs because the kernels reach their
peers' memory), wait until rank 0 answers ``ping`` on the socket, optionally send a smoke request,
then either stay attached (``--hold``) or stop the ranks.  Ranks are ended by their own PIDs.
"""
from __future__ import annotations

import argparse
import os
import signal
import socket
import subprocess
import sys
import time

PROBE = ("import torch,sys;d=int(sys.argv[1]);torch.cuda.set_device(d);"
         "a=torch.ones(8,8,device='cuda');print(float((a@a).sum()));torch.cuda.synchronize()")


def probe_gpu(index: int, timeout: float = 60.0) -> tuple[bool, str]:
    """An 8 x 8 matmul on GPU ``index`` in a child process; ``(ok, message)``."""
    try:
        out = subprocess.run([sys.executable, "-c", PROBE, str(index)], capture_output=True, text=True, timeout=timeout)
    except subprocess.TimeoutExpired:
        return False, f"gpu {index}: no answer within {timeout:.0f}s"
    if out.returncode != 0 or out.stdout.strip() != "512.0":
        return False, f"gpu {index}: exit {out.returncode}: {out.stderr.strip()[-200:]}"
    return True, f"gpu {index}: ok"


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def rank_env(rank: int, world: int, port: int, parallel: str, base: dict | None = None) -> dict:
    env = dict(base if base is not None else os.environ)
    env.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
               MASTER_PORT=str(port), COFFIN_PARALLEL=parallel)
    return env


def engine_argv(args, extra: list[str]) -> list[str]:
    argv = [sys.executable, "-m", "coffin_b200.entrypoints.cli.runtime", "--serve", "--sock", args.sock]
    if args.model:
        argv += ["--model", args.model]
    if args.preset:
        argv += ["--preset", args.preset]
    return argv + extra


def wait_ping(sock: str, timeout: float, procs: list | None = None) -> bool:
    """Poll ``ping`` until rank 0 answers.  Gives up early when a rank process has already exited: the
    others would wait in their first collective until the start limit runs out."""
    from ..serving.transport import call
    deadline = time.monotonic() + timeout
    while time.monotonic() < deadline:
        dead = [i for i, p in enumerate(procs or []) if p.poll() is not None]
        if dead:
            print(f"rank(s) {dead} exited during start-up (codes {[procs[i].returncode for i in dead]})", file=sys.stderr)
            return False
        try:
            if call(sock, {"op": "ping"}, timeout=5).get("ok"):
                return True
        except OSError:
            pass
        time.sleep(0.5)
    return False


def stop(procs: list[subprocess.Popen], grace: float = 10.0) -> None:
    for p in procs:
        if p.poll() is None:
            p.send_signal(signal.SIGTERM)
    deadline = time.monotonic() + grace
    for p in procs:
        try:
            p.wait(max(0.1, deadline - time.monotonic()))
        except subprocess.TimeoutExpired:
            p.kill()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--parallel", choices=("tp", "pp", "ep"), default="tp")
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--model")
    ap.add_argument("--preset")
    ap.add_argument("--sock", default="/tmp/coffin_b200.sock")
    ap.add_argument("--smoke", help="send this prompt through `generate` once the engine answers")
    ap.add_argument("--start-timeout", type=float, default=600.0)
    ap.add_argument("--hold", action="store_true", help="stay attached until interrupted")
    ap.add_argument("--skip-probe", action="store_true")
    args, extra = ap.parse_known_args(argv)
    if not args.skip_probe:
        for i in range(args.gpus):
            ok, msg = probe_gpu(i)
            print(msg, flush=True)
            if not ok:
                return 2
    port = free_port()
    procs = [subprocess.Popen(engine_argv(args, extra), env=rank_env(r, args.gpus, port, args.parallel))
             for r in range(args.gpus)]
    try:
        if not wait_ping(args.sock, args.start_timeout, procs):
            print("engine did not answer ping", file=sys.stderr)
            return 3
        print(f"engine up: {args.gpus} ranks, {args.parallel}, socket {args.sock}", flush=True)
        if args.smoke:
            from ..serving.transport import call
            rep = call(args.sock, {"op": "generate", "prompt": args.smoke, "max_new": 16}, timeout=300)
            print(rep, flush=True)
            if not rep.get("ok"):
                return 4
        if args.hold:
            while all(p.poll() is None for p in procs):
                time.sleep(1.0)
        return 0
    finally:
        try:
            from ..serving.transport import call
            call(args.sock, {"op": "stop"}, timeout=5)
        except Exception:              # noqa: BLE001
            pass
        stop(procs)


if __name__ == "__main__":
    sys.exit(main())
