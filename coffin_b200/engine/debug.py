"""Opt-in consistency checks and traces of the engine (all off by default, switched by environment
variables read once at import):

* ``COFFIN_KV_TRACE=1``      before every forward, print each live sequence's block table head and
  verify that no block a sequence is about to WRITE is referenced by another live sequence (shared
  prefix blocks are legal, a shared write block means two sequences overwrite each other's KV).
* ``COFFIN_PREFILL_TRACE=1`` per-chunk prefill timing (host clock around the launches + a device sync).
* ``COFFIN_PC_TRACE=1``      prefix-cache decisions at admission (tokens matched, blocks adopted).
* ``COFFIN_EP_TRACE=1``      accumulated device time of the expert-parallel / prefill all-reduce, printed at exit.
* ``COFFIN_MOE_CHECK=1``     after every device-side expert dispatch, check on the host that the sorted
  order is a permutation of the routed slots and that the tile list covers exactly the local slots.
* ``COFFIN_MOE_SHAPE=1``     print every distinct shape the grouped expert projections run at (rows, local
  experts, output width, depth, storage), once per shape.
* ``COFFIN_WQ_TRACE=1``      print the shape and the caller's stack whenever a whole int4 expert stack is
  expanded to bf16 (1.6 GB per layer on the 35B model: the line tells who reached it).
* ``COFFIN_DEBUG_STEP=1``    every 50th engine step, one line with the scheduler's queues and the free
  blocks (read in ``engine/llm_engine.py``); the serving loop also prints one line per submitted request.
* ``COFFIN_PD_TRACE`` / ``COFFIN_PD_VERIFY``  one line per adopted sequence / a read-back comparison of what
  the adopt wrote (read in ``engine/pd.py``).

Reference switches of the same names: ``engine/model_runner.py:312,438,634,777-827``,
``engine/prefix_engine.py:131``, ``models/qwen35/ep.py:45-48``, ``models/qwen4exp/moe.py:57-69``,
``int8_weights.py:172``, ``engine/llm_engine.py:27-32``, ``serving/runtime_parts.py:1341-1342``.
"""
from __future__ import annotations

import atexit
import os
import time

_env = os.environ
KV_TRACE = _env.get("COFFIN_KV_TRACE") == "1"
PREFILL_TRACE = _env.get("COFFIN_PREFILL_TRACE") == "1"
PC_TRACE = bool(_env.get("COFFIN_PC_TRACE"))
EP_TRACE = _env.get("COFFIN_EP_TRACE", "").strip() == "1"
MOE_CHECK = bool(_env.get("COFFIN_MOE_CHECK"))
MOE_SHAPE = bool(_env.get("COFFIN_MOE_SHAPE"))
WQ_TRACE = _env.get("COFFIN_WQ_TRACE") == "1"
_shapes_seen: set = set()


def moe_shape(tag: str, rows: int, experts: int, n: int, k: int, storage: str) -> bool:
    """Print a grouped-projection shape the first time it is seen; True when it printed."""
    key = (tag, rows, experts, n, k, storage)
    if key in _shapes_seen:
        return False
    _shapes_seen.add(key)
    print(f"[moe-shape] {tag} rows={rows} experts={experts} n={n} k={k} weights={storage}", flush=True)
    return True


def wq_expand(shape: tuple, kept: bool) -> None:
    """Report a whole-stack int4 -> bf16 expansion with the last frames of the caller's stack."""
    import traceback
    print(f"[wq-expand] {tuple(shape)} kept={kept}", flush=True)
    print("".join(traceback.format_stack()[-6:-1]), flush=True)


class BlockAliasError(RuntimeError):
    pass


def check_block_alias(seqs, block_size: int, where: str, n_new: dict | None = None, verbose: bool = False) -> None:
    """Raise when a block that one sequence is about to write (the blocks from its write position on) is
    also in another live sequence's table.  ``n_new[seq_id]`` = tokens the forward will write (default 1)."""
    owner: dict[int, int] = {}
    tables = {}
    for s in seqs:
        if s.blocks is None:
            continue
        tables[s.seq_id] = list(s.blocks.table)
        if verbose:
            print(f"[blktrace] {where} seq={s.seq_id} slot={s.slot} computed={s.num_computed} cached={s.cached_tokens} "
                  f"nblocks={len(tables[s.seq_id])} head={tables[s.seq_id][:3]}", flush=True)
    for s in seqs:
        if s.seq_id not in tables:
            continue
        first = s.num_computed // block_size
        n = (n_new or {}).get(s.seq_id, 1)
        last = (s.num_computed + max(1, n) - 1) // block_size
        for b in tables[s.seq_id][first:last + 1]:
            if b in owner and owner[b] != s.seq_id:
                raise BlockAliasError(f"{where}: block {b} is written by sequences {owner[b]} and {s.seq_id}")
            owner[b] = s.seq_id
    for s in seqs:
        for b in tables.get(s.seq_id, ()):
            if b in owner and owner[b] != s.seq_id:
                raise BlockAliasError(f"{where}: block {b} written by sequence {owner[b]} is in the table of {s.seq_id}")


class _Stopwatch:
    """Accumulates device time between CUDA events; printed once at exit."""

    def __init__(self, label: str) -> None:
        self.label, self.pairs, self.total_ms, self.n = label, [], 0.0, 0
        atexit.register(self.report)

    def span(self):
        import torch
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        self.pairs.append((a, b))
        return b

    def drain(self) -> None:
        keep = []
        for a, b in self.pairs:
            if b.query():
                self.total_ms += a.elapsed_time(b)
                self.n += 1
            else:
                keep.append((a, b))
        self.pairs = keep

    def report(self) -> None:
        try:
            import torch
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            self.drain()
        except Exception:       # noqa: BLE001 - interpreter shutdown
            pass
        if self.n:
            print(f"[{self.label}] {self.n} spans, {self.total_ms:.2f} ms on the device, {self.total_ms / self.n * 1e3:.1f} us each",
                  flush=True)


_ep_watch: _Stopwatch | None = None


def ep_span():
    """Start a device-time span of an expert-parallel / prefill all-reduce; call ``.record()`` on the
    returned event when it ends (``None`` when the trace is off)."""
    global _ep_watch
    if not EP_TRACE:
        return None
    if _ep_watch is None:
        _ep_watch = _Stopwatch("eptrace")
    _ep_watch.drain()
    return _ep_watch.span()


def check_moe_dispatch(idx, disp: dict, n_local: int) -> None:
    """Host check of a device-side dispatch: ``pos`` is a bijection from the local routed slots onto the
    sorted rows, ``src_tok`` inverts it, and the tile list covers exactly those rows, expert by expert."""
    import torch
    T, k = idx.shape
    flat = idx.reshape(-1).cpu()
    pos, src = disp["pos"].cpu(), disp["src_tok"].cpu()
    local = (flat >= 0) & (flat < n_local)
    n = int(local.sum())
    p = pos[local]
    if sorted(p.tolist()) != list(range(n)) or bool((pos[~local] >= 0).any()):
        raise RuntimeError("moe dispatch: sorted rows are not a permutation of the local slots")
    slots = torch.nonzero(local).flatten()
    if not torch.equal(src[p.long()], (slots // k).to(src.dtype)):
        raise RuntimeError("moe dispatch: src_tok does not invert pos")
    cnt = int(disp["count"][0])
    rows = disp["rows"][:cnt].cpu().tolist()
    row0 = disp["row0"][:cnt].cpu().tolist()
    exp = disp["expert"][:cnt].cpu().tolist()
    covered = sorted((r0 + i, e) for r0, n_r, e in zip(row0, rows, exp) for i in range(n_r))
    want = sorted((int(pp), int(flat[s])) for pp, s in zip(p.tolist(), slots.tolist()))
    if covered != want:
        raise RuntimeError("moe dispatch: the tile list does not cover the sorted rows expert by expert")


def prefill_trace(seq, start: int, end: int, t0: float, device) -> None:
    import torch
    if device is not None and device.type == "cuda":
        torch.cuda.synchronize(device)
    print(f"[prefill] seq={seq.seq_id} slot={seq.slot} tokens {start}..{end} of {seq.num_tokens} "
          f"{(time.perf_counter() - t0) * 1e3:.2f} ms", flush=True)
