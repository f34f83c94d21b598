"""CPU control plane of a multi-rank engine: bootstrap, request fan-out, heartbeats.

Data moves between GPUs inside the kernels (``parallel/tp.py``) or through NCCL; everything else
- which request to run, whether every rank is still alive - travels over a gloo process group on
the host, so that a failure is noticed on the CPU before the next kernel is launched and never
has to be inferred from a hung GPU.

* ``init_control_plane`` creates the default process group (NCCL for device collectives when CUDA
  is present) plus a gloo group for control traffic (reference: ``_init_tensor_parallel``,
  ``serving/runtime_transport.py:33-55``).
* ``make_fanout`` / ``worker_loop``: rank 0 broadcasts every request dict; the other ranks replay it
  on their ``Server`` so that all ranks issue the same kernels (reference ``_tp_worker``, l.99-135).
* ``Heartbeat``: every rank stamps a counter in the shared store; ``check()`` reports ranks whose
  stamp is older than the timeout.  The serving loop calls it between steps; on a dead peer the
  engine fails the requests in flight and the launcher restarts the group (no elastic re-ranking,
  as in the reference).
* ``agree_tokens``: rank 0's sampled tokens are broadcast so that a numerical divergence between
  ranks can never fork the sequences (reference ``ModelRunner.sample``, ``engine/model_runner.py:900-924``).
"""
from __future__ import annotations

import datetime
import os
import threading
import time

import torch
import torch.distributed as dist

_CONTROL = None


def init_control_plane(backend: str | None = None, timeout_s: float = 120.0):
    """Initialise ``torch.distributed`` from the environment (``RANK``, ``WORLD_SIZE``,
    ``MASTER_ADDR``, ``MASTER_PORT``) and return the gloo control group."""
    global _CONTROL
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kw = {}
        if backend == "nccl":
            local = int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", "0")))
            torch.cuda.set_device(local)
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend, timeout=datetime.timedelta(seconds=timeout_s), **kw)
    if _CONTROL is None:
        _CONTROL = (dist.group.WORLD if dist.get_backend() == "gloo"
                    else dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s)))
    return _CONTROL


def control_group():
    return _CONTROL


def make_fanout(group=None):
    """Rank 0 side: returns ``fanout(req)`` that broadcasts the request to the workers.
    A lock serialises fan-outs so that the workers see requests in one order."""
    group = group or _CONTROL
    lock = threading.Lock()

    def fanout(req: dict) -> None:
        with lock:
            dist.broadcast_object_list([req], src=0, group=group)
    return fanout


def worker_loop(srv, group=None) -> None:
    """Ranks > 0: replay every request rank 0 received until a ``stop`` arrives."""
    group = group or _CONTROL
    srv.start()
    while True:
        box = [None]
        dist.broadcast_object_list(box, src=0, group=group)
        req = box[0] or {}
        if req.get("op") == "chat_stream":
            for _ in srv.stream_chat(req):
                pass
        else:
            rep = srv.handle(req)
            if rep.get("stopping"):
                srv.stop()
                return


def agree_tokens(tokens: list[int], group=None) -> list[int]:
    """Every rank returns rank 0's tokens."""
    group = group or _CONTROL
    if group is None or dist.get_world_size(group) == 1:
        return tokens
    t = torch.tensor(tokens, dtype=torch.int64)
    dist.broadcast(t, src=0, group=group)
    return t.tolist()


class Heartbeat:
    """Liveness through the process group's key-value store (host only)."""

    def __init__(self, store, rank: int, world: int, interval_s: float = 0.5, timeout_s: float = 5.0) -> None:
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.timeout_s = interval_s, timeout_s
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._seen: dict[int, tuple[int, float]] = {}

    def start(self) -> None:
        self._beat()
        self._thread = threading.Thread(target=self._run, name="heartbeat", daemon=True)
        self._thread.start()

    def _beat(self) -> None:
        self.store.add(f"hb/{self.rank}", 1)

    def _run(self) -> None:
        while not self._stop.wait(self.interval_s):
            try:
                self._beat()
            except Exception:      # noqa: BLE001 - the store went away with rank 0
                return

    def stop(self) -> None:
        self._stop.set()

    def check(self) -> list[int]:
        """Ranks whose counter has not advanced for ``timeout_s`` seconds."""
        now, dead = time.monotonic(), []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                v = int(self.store.add(f"hb/{r}", 0))
            except Exception:      # noqa: BLE001
                dead.append(r)
                continue
            last = self._seen.get(r)
            if last is None or v != last[0]:
                self._seen[r] = (v, now)
            elif now - last[1] > self.timeout_s:
                dead.append(r)
        return dead


def shutdown(timeout_s: float = 10.0, hard_exit: bool = True) -> bool:
    """Leave the process group at the end of a rank process.

    ``destroy_process_group`` has been seen to block for minutes when the ranks hold CUDA-IPC
    mappings of each other's memory (the peer communicator), although every collective had
    completed.  So the ranks synchronise, the teardown runs in a helper thread, and when it has not
    returned after ``timeout_s`` the process ends itself with ``os._exit(0)`` (all results have been
    written by then; the driver reaps the child).  Returns whether the teardown finished."""
    import sys
    done = threading.Event()

    def run() -> None:
        try:
            dist.destroy_process_group()
        finally:
            done.set()

    if not dist.is_initialized():
        return True
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    t = threading.Thread(target=run, name="pg-teardown", daemon=True)
    t.start()
    ok = done.wait(timeout_s)
    if not ok and hard_exit:
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    return ok
