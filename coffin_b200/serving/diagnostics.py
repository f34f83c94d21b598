"""Diagnostic ops of the engine socket: ``bench``, ``profile``, ``ops``, ``spec``, ``verify`` and the
prefill/decode disaggregation hand-off (``pd_prefill`` / ``pd_decode`` / ``pd_decode_batch``).

They run on the engine thread while the engine is idle and use engine slot 0 directly.
Reference: ``serving/runtime_parts.py:1044-1130`` (spec/bench/profile/ops), ``:1135-1466`` (PD),
``:1514-1743`` (verify A/B).
"""
from __future__ import annotations

import time
from pathlib import Path

import torch


def _tokens(srv, req: dict) -> list[int]:
    if req.get("tokens"):
        return [int(t) for t in req["tokens"]]
    return srv.tok.encode(req.get("prompt") or "Hello")


def _sync(srv) -> None:
    dev = getattr(srv.model, "device", None)
    if dev is not None and dev.type == "cuda":
        torch.cuda.synchronize(dev)


class DiagError(ValueError):
    """A diagnostic request the engine refuses (answered as ``{"ok": false, "error": ...}``)."""


def _room(srv, n_prompt: int) -> int:
    """Tokens that a solo run can decode after a prompt of ``n_prompt`` tokens: bounded by the private
    block table of ``_solo`` and by the model's window, with a margin for a verify pass of 8."""
    m = srv.model
    nblk = min((n_prompt + 64 + 4096) // 64 + 1, m.num_blocks - 1, getattr(m, "max_blocks_per_seq", 1 << 30))
    return min(nblk * 64, getattr(m, "max_seq", 1 << 30)) - n_prompt - 8


def _bounded(srv, prompt: list[int], n: int, what: str = "n") -> int:
    """Validate a client-supplied step count against the room of the solo table; the kernels index
    block tables and rotary tables with these positions and do not check them."""
    room = _room(srv, len(prompt))
    if n < 1 or n > room:
        raise DiagError(f"{what}={n} outside 1..{max(room, 0)} for a prompt of {len(prompt)} tokens "
                        f"(block table / context window)")
    return n


def _solo(srv, prompt: list[int]):
    """Prefill ``prompt`` into slot 0 with a private block table; returns (table, logits)."""
    m = srv.model
    srv.engine.reset()
    if _room(srv, len(prompt)) < 1:
        raise DiagError(f"a prompt of {len(prompt)} tokens leaves no room to decode")
    nblk = (len(prompt) + 64 + 4096) // 64 + 1
    nblk = min(nblk, m.num_blocks - 1, getattr(m, "max_blocks_per_seq", 1 << 30))
    table = list(range(1, 1 + nblk))
    m.zero_state(0)
    bt = torch.tensor(table, dtype=torch.int32, device=m.device)
    logits = None
    for s in range(0, len(prompt), m.max_chunk):
        e = min(len(prompt), s + m.max_chunk)
        toks = torch.tensor(prompt[s:e], dtype=torch.int64, device=m.device)
        logits = m.prefill(toks, s, 0, bt, want_logits=e == len(prompt))
    return table, logits


def _decode_loop(srv, table, tok: int, pos: int, n: int, graph: bool) -> list[int]:
    m, out = srv.model, []
    for _ in range(n):
        m.set_rows(1, [tok], [pos], [0], [table])
        nxt, _ = m.decode(1, graph=graph)
        tok = int(nxt[0])
        out.append(tok)
        pos += 1
    return out


def bench(srv, req: dict) -> dict:
    """Host-timed decode after three warm-up steps, device synchronised on both sides."""
    prompt = _tokens(srv, req)
    n = _bounded(srv, prompt, int(req.get("n", 32)) + 3) - 3
    table, logits = _solo(srv, prompt)
    tok = int(logits.argmax())
    _decode_loop(srv, table, tok, len(prompt), 3, srv.cfg.graph)
    _sync(srv)
    t0 = time.perf_counter()
    _decode_loop(srv, table, tok, len(prompt) + 3, n, srv.cfg.graph)
    _sync(srv)
    dt = time.perf_counter() - t0
    return {"ok": True, "n": n, "ms_per_step": round(dt / n * 1e3, 4), "decode_tok_s": round(n / dt, 2)}


def _profile(srv, req: dict, by_op: bool) -> dict:
    from torch.profiler import ProfilerActivity, profile as tprofile
    prompt = _tokens(srv, req)
    n = _bounded(srv, prompt, int(req.get("n", 8)) + 2) - 2
    table, logits = _solo(srv, prompt)
    tok = int(logits.argmax())
    _decode_loop(srv, table, tok, len(prompt), 2, False)
    _sync(srv)
    acts = [ProfilerActivity.CPU]
    if getattr(srv.model, "device", torch.device("cpu")).type == "cuda":
        acts.append(ProfilerActivity.CUDA)
    with tprofile(activities=acts) as prof:
        _decode_loop(srv, table, tok, len(prompt) + 2, n, False)
        _sync(srv)
    rows, total, launches = [], 0.0, 0
    for ev in prof.key_averages():
        us = float(getattr(ev, "self_device_time_total", 0.0) or getattr(ev, "self_cuda_time_total", 0.0) or 0.0)
        if ev.key in ("cudaLaunchKernel", "cudaLaunchKernelExC"):
            launches += ev.count
        if us <= 0 and not by_op:
            continue
        if by_op:
            us = us or float(ev.self_cpu_time_total)
        rows.append({"kernel" if not by_op else "op": ev.key[:80], "calls": ev.count, "us": round(us, 1)})
        total += us
    rows.sort(key=lambda r: -r["us"])
    for r in rows:
        r["pct"] = round(100 * r["us"] / total, 2) if total else 0.0
    out = {"ok": True, "n": n, "total_us": round(total, 1), "rows": rows[:18]}
    if not by_op:
        out.update({"launches": launches // max(1, n), "listed": min(18, len(rows)), "all": len(rows)})
    return out


def profile(srv, req: dict) -> dict:
    return _profile(srv, req, by_op=False)


def ops(srv, req: dict) -> dict:
    return _profile(srv, req, by_op=True)


def spec(srv, req: dict) -> dict:
    """Plain vs speculative greedy decode on the same prompt: speed-up, exactness, accept rate."""
    from ..engine.speculative import SpeculativeDecoder
    k = int(req.get("spec_k", 3))
    prompt = _tokens(srv, req)
    n = _bounded(srv, prompt, int(req.get("n", 32)))
    table, logits = _solo(srv, prompt)
    tok = int(logits.argmax())
    _sync(srv)
    t0 = time.perf_counter()
    plain = [tok] + _decode_loop(srv, table, tok, len(prompt), n - 1, srv.cfg.graph)
    _sync(srv)
    t_plain = time.perf_counter() - t0
    table, logits = _solo(srv, prompt)
    sd = SpeculativeDecoder(srv.model, k=k)
    _sync(srv)
    t0 = time.perf_counter()
    spec_toks = sd.generate(prompt, table, logits, n)
    _sync(srv)
    t_spec = time.perf_counter() - t0
    return {"ok": True, "plain_tok_s": round(n / t_plain, 2), "spec_tok_s": round(n / t_spec, 2),
            "speedup": round(t_plain / t_spec, 3), "exact": spec_toks[:n] == plain[:n], "accept": sd.stats()}


def verify(srv, req: dict) -> dict:
    """A/B timing of c-token verification against c single steps (same tokens)."""
    from ..engine.speculative import SpeculativeDecoder
    c = int(req.get("c", 4))
    if c not in (2, 4, 8):
        raise DiagError("c must be 2, 4 or 8")
    prompt = _tokens(srv, req)
    n = int(req.get("n", 8))
    _bounded(srv, prompt, c * n, "c*n")
    table, logits = _solo(srv, prompt)
    tok = int(logits.argmax())
    seq = [tok] + _decode_loop(srv, table, tok, len(prompt), c * n, False)
    table, logits = _solo(srv, prompt)
    sd = SpeculativeDecoder(srv.model, k=c - 1)
    _sync(srv)
    t0 = time.perf_counter()
    for i in range(n):
        sd.verify_only(table, seq[i * c:(i + 1) * c], len(prompt) + i * c)
    _sync(srv)
    t_verify = time.perf_counter() - t0
    table, logits = _solo(srv, prompt)
    _sync(srv)
    t0 = time.perf_counter()
    _decode_loop(srv, table, tok, len(prompt), c * n, False)
    _sync(srv)
    t_step = time.perf_counter() - t0
    return {"ok": True, "c": c, "n": n, "verify_ms": round(t_verify / n * 1e3, 3),
            "steps_ms": round(t_step / n * 1e3, 3), "ratio": round(t_step / t_verify, 3)}


# ---------------------------------------------------------------------------- PD hand-off
def pd_prefill(srv, req: dict) -> dict:
    """Prefill a prompt and export the sequence state (KV blocks + delta-net state + logits) to
    ``out_dir`` for a decode instance to adopt."""
    from ..engine.pd import export_state, export_state_device
    prompt = _tokens(srv, req)
    out_dir = Path(req["out_dir"])
    transport = req.get("transport", "file")
    if transport not in ("file", "device"):
        raise DiagError("transport must be 'file' or 'device'")
    if transport == "device" and getattr(getattr(srv.model, "device", None), "type", "cpu") != "cuda":
        raise DiagError("the device transport needs a CUDA engine")
    t0 = time.perf_counter()
    table, logits = _solo(srv, prompt)
    _sync(srv)
    ms = (time.perf_counter() - t0) * 1e3
    t1 = time.perf_counter()
    if transport == "device":
        # one device buffer + its CUDA IPC handle: the decode instance copies device to device
        nbytes = export_state_device(srv.model, 0, table, prompt, logits, out_dir, token=str(req.get("token", "default")))
    else:
        stale = out_dir / "state.json"
        if stale.exists():
            stale.unlink()
        nbytes = export_state(srv.model, 0, table, prompt, logits, out_dir)
    return {"ok": True, "n_prompt": len(prompt), "prefill_ms": round(ms, 2), "bytes": nbytes, "out_dir": str(out_dir),
            "transport": transport, "export_ms": round((time.perf_counter() - t1) * 1e3, 2)}


def pd_release(srv, req: dict) -> dict:
    """Free the device buffer a ``pd_prefill`` with the device transport published (after the adopter copied it)."""
    from ..engine.pd import release_export
    return {"ok": True, "released": release_export(str(req.get("token", "default")))}


def pd_decode(srv, req: dict) -> dict:
    from ..engine.pd import adopt_any
    srv.engine.reset()
    n = int(req.get("max_new", 32))
    table, prompt, logits = adopt_any(srv.model, 0, Path(req["out_dir"]), max_new=n)
    if n < 1 or len(prompt) + n > min(len(table) * 64, getattr(srv.model, "max_seq", 1 << 30)):
        raise DiagError(f"max_new={n} does not fit the adopted sequence's block table / window")
    tok = int(logits.argmax())
    _sync(srv)
    t0 = time.perf_counter()
    out = [tok] + _decode_loop(srv, table, tok, len(prompt), n - 1, srv.cfg.graph)
    _sync(srv)
    dt = time.perf_counter() - t0
    return {"ok": True, "tokens": out, "text": srv.tok.decode(out, skip_special_tokens=True), "n_prompt": len(prompt),
            "n_new": len(out), "decode_tok_s": round(len(out) / dt, 2)}


def pd_decode_batch(srv, req: dict) -> dict:
    """Adopt several exported sequences into batch rows and decode them together."""
    from ..engine.pd import adopt_any as adopt_state
    srv.engine.reset()
    items = req.get("items") or []
    m = srv.model
    if len(items) > m.num_slots:
        return {"ok": False, "error": f"{len(items)} items exceed {m.num_slots} rows"}
    rows, base = [], 1
    for slot, it in enumerate(items):
        mx = int(it.get("max_new", req.get("max_new", 32)))
        table, prompt, logits = adopt_state(m, slot, Path(it["dir"]), first_block=base, max_new=mx)
        if mx < 1 or len(prompt) + mx > min(len(table) * 64, getattr(m, "max_seq", 1 << 30)):
            raise DiagError(f"max_new={mx} does not fit the adopted sequence's block table / window")
        base += len(table)
        rows.append({"table": table, "pos": len(prompt), "tok": int(logits.argmax()), "out": [], "max_new": mx})
    _sync(srv)
    t0 = time.perf_counter()
    live = list(range(len(rows)))
    for r in rows:
        r["out"].append(r["tok"])
    while live:
        M = m.bucket_for(len(live))
        m.set_rows(M, [rows[i]["tok"] for i in live], [rows[i]["pos"] for i in live], live,
                   [rows[i]["table"] for i in live])
        nxt, _ = m.decode(M, graph=srv.cfg.graph)
        nxt = nxt.tolist()
        for j, i in enumerate(list(live)):
            r = rows[i]
            r["tok"] = int(nxt[j])
            r["pos"] += 1
            r["out"].append(r["tok"])
            if len(r["out"]) >= r["max_new"]:
                live.remove(i)
    _sync(srv)
    dt = time.perf_counter() - t0
    total = sum(len(r["out"]) for r in rows)
    return {"ok": True, "items": [{"tokens": r["out"], "text": srv.tok.decode(r["out"], skip_special_tokens=True)} for r in rows],
            "decode_tok_s": round(total / dt, 2)}
