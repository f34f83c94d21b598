"""Open-loop load generator for the OpenAI-compatible HTTP front.

    # against a running front (engine + `python -m coffin_b200.entrypoints.cli.openai`)
    python -m coffin_b200.tools.bench_serving --port 18080 --requests 512 --rate 8

    # or let the tool start one engine process per replica and the HTTP front itself
    python -m coffin_b200.tools.bench_serving --spawn --preset qwen35-4b --replicas 1 \
        --requests 128 --rate 8 --prefix-tokens 1024 --suffix-tokens 64 --max-tokens 128

Requests arrive as a Poisson process of ``--rate`` per second (open loop: arrivals do not wait for
completions), every prompt is a shared prefix followed by a unique suffix (so the radix prefix cache
is exercised), responses are streamed over SSE, and a fraction ``--image-frac`` of the requests
carries one synthetic ``--image-size`` square PNG as a base64 ``image_url``.  Per request the tool
records the time to the first streamed token, the mean gap between the following tokens and the total
latency; it prints one JSON object with percentiles and the aggregate request and token rates.

This is the measuring instrument for the serving configuration of the benchmark plan (512 requests,
8 requests/s, shared 1024-token prefix, SSE, 10 % image requests); the reference has no load
generator of its own, its serving numbers are single-request (``docs/FACTS-RUNTIME.md``).
"""
from __future__ import annotations

import argparse
import base64
import http.client
import io
import json
import os
import random
import subprocess
import sys
import tempfile
import threading
import time

WORDS = ("alpha beta gamma delta epsilon zeta eta theta iota kappa lambda mu nu xi omicron pi rho sigma tau "
         "upsilon phi chi psi omega").split()


def make_text(n_tokens: int, seed: int, chars_per_token: float) -> str:
    """Deterministic filler of roughly ``n_tokens`` tokens."""
    rng = random.Random(seed)
    out, n = [], 0
    target = int(n_tokens * chars_per_token)
    while n < target:
        w = rng.choice(WORDS)
        out.append(w)
        n += len(w) + 1
    return " ".join(out)[:target]


def make_png(size: int, seed: int) -> str:
    from PIL import Image
    rng = random.Random(seed)
    img = Image.new("RGB", (size, size))
    px = img.load()
    c0 = (rng.randrange(256), rng.randrange(256), rng.randrange(256))
    for y in range(0, size, 16):
        for x in range(0, size, 16):
            col = ((c0[0] + x) % 256, (c0[1] + y) % 256, (c0[2] + x + y) % 256)
            for yy in range(y, min(size, y + 16)):
                for xx in range(x, min(size, x + 16)):
                    px[xx, yy] = col
    buf = io.BytesIO()
    img.save(buf, format="PNG")
    return base64.b64encode(buf.getvalue()).decode()


class Result:
    __slots__ = ("ok", "status", "t_send", "t_first", "t_done", "n_out", "prompt_tokens", "image", "error",
                 "srv_ttft_ms", "srv_decode_ms", "cached")

    def __init__(self) -> None:
        self.ok = False
        self.status = 0
        self.t_send = self.t_first = self.t_done = 0.0
        self.n_out = 0
        self.prompt_tokens = 0
        self.image = False
        self.error = ""
        self.srv_ttft_ms = self.srv_decode_ms = None
        self.cached = 0


def one_request(host: str, port: int, body: dict, res: Result, timeout: float) -> None:
    res.t_send = time.perf_counter()
    try:
        c = http.client.HTTPConnection(host, port, timeout=timeout)
        c.request("POST", "/v1/chat/completions", json.dumps(body),
                  {"Content-Type": "application/json", "Connection": "close"})
        r = c.getresponse()
        res.status = r.status
        if r.status != 200:
            res.error = r.read().decode(errors="replace")[:200]
            c.close()
            return
        while True:
            line = r.readline()
            if not line:
                break
            line = line.strip()
            if not line.startswith(b"data: "):
                continue
            payload = line[6:]
            if payload == b"[DONE]":
                break
            ev = json.loads(payload)
            if ev.get("usage"):
                res.prompt_tokens = int(ev["usage"].get("prompt_tokens", 0))
                res.n_out = max(res.n_out, int(ev["usage"].get("completion_tokens", 0)))
                res.cached = int((ev["usage"].get("prompt_tokens_details") or {}).get("cached_tokens", 0))
                tm = ev["usage"].get("timing") or {}
                res.srv_ttft_ms, res.srv_decode_ms = tm.get("ttft_ms"), tm.get("decode_ms")
            for ch in ev.get("choices", []):
                d = ch.get("delta", {})
                if d.get("content") or d.get("reasoning_content") or d.get("tool_calls"):
                    if not res.t_first:
                        res.t_first = time.perf_counter()
        res.t_done = time.perf_counter()
        res.ok = True
        c.close()
    except Exception as exc:      # noqa: BLE001 - a failed request is a data point, not a crash
        res.error = f"{type(exc).__name__}: {exc}"
        res.t_done = time.perf_counter()


def pct(xs: list[float], q: float) -> float | None:
    if not xs:
        return None
    xs = sorted(xs)
    i = min(len(xs) - 1, max(0, int(round(q * (len(xs) - 1)))))
    return xs[i]


def run_load(host: str, port: int, args) -> dict:
    rng = random.Random(args.seed)
    prefix = make_text(args.prefix_tokens, 1, args.chars_per_token)
    image_b64 = make_png(args.image_size, 7) if args.image_frac > 0 else None
    results = [Result() for _ in range(args.requests)]
    threads = []
    t0 = time.perf_counter()
    t_next = t0
    for i in range(args.requests):
        now = time.perf_counter()
        if t_next > now:
            time.sleep(t_next - now)
        t_next += rng.expovariate(args.rate) if args.rate > 0 else 0.0
        text = prefix + " " + make_text(args.suffix_tokens, 1000 + i, args.chars_per_token)
        with_image = image_b64 is not None and rng.random() < args.image_frac
        if with_image:
            content = [{"type": "image_url", "image_url": {"url": "data:image/png;base64," + image_b64}},
                       {"type": "text", "text": text}]
        else:
            content = text
        body = {"model": args.model, "stream": True, "max_tokens": args.max_tokens, "temperature": 0,
                "stream_options": {"include_usage": True}, "messages": [{"role": "user", "content": content}]}
        results[i].image = with_image
        th = threading.Thread(target=one_request, args=(host, port, body, results[i], args.timeout), daemon=True)
        th.start()
        threads.append(th)
    for th in threads:
        th.join(args.timeout)
    t1 = time.perf_counter()
    ok = [r for r in results if r.ok]
    # TTFT / TPOT come from the engine's own clock (submit -> first token -> last token, scheduling queue
    # included) reported in the usage chunk: a random-init model emits tokens that often decode to no
    # text, so "first text seen by the client" says when the detokeniser first had something to show,
    # not when the first token existed.  The client's first-text clock is reported next to it.
    srv = [r for r in ok if r.srv_ttft_ms is not None]
    ttft = [float(r.srv_ttft_ms) for r in srv] or [(r.t_first - r.t_send) * 1e3 for r in ok if r.t_first]
    tpot = [float(r.srv_decode_ms) / (r.n_out - 1) for r in srv if r.srv_decode_ms is not None and r.n_out > 1] or \
           [(r.t_done - r.t_first) * 1e3 / (r.n_out - 1) for r in ok if r.t_first and r.n_out > 1]
    first_text = [(r.t_first - r.t_send) * 1e3 for r in ok if r.t_first]
    lat = [(r.t_done - r.t_send) * 1e3 for r in ok]
    out_tokens = sum(r.n_out for r in ok)
    rnd = lambda v: None if v is None else round(v, 2)   # noqa: E731
    rep = {"requests": args.requests, "completed": len(ok), "failed": len(results) - len(ok),
           "rate_req_s": args.rate, "wall_s": round(t1 - t0, 2),
           "throughput_req_s": round(len(ok) / (t1 - t0), 3),
           "output_tok_s": round(out_tokens / (t1 - t0), 1),
           "prompt_tokens_p50": pct([float(r.prompt_tokens) for r in ok], 0.5),
           "cached_prompt_tokens_p50": pct([float(r.cached) for r in ok], 0.5),
           "timing_source": "engine" if srv else "client",
           "client_first_text_ms": {"p50": rnd(pct(first_text, 0.5)), "p99": rnd(pct(first_text, 0.99)), "n": len(first_text)},
           "output_tokens_total": out_tokens, "image_requests": sum(1 for r in results if r.image),
           "ttft_ms": {"p50": rnd(pct(ttft, 0.5)), "p90": rnd(pct(ttft, 0.9)), "p99": rnd(pct(ttft, 0.99))},
           "tpot_ms": {"p50": rnd(pct(tpot, 0.5)), "p90": rnd(pct(tpot, 0.9)), "p99": rnd(pct(tpot, 0.99))},
           "latency_ms": {"p50": rnd(pct(lat, 0.5)), "p99": rnd(pct(lat, 0.99))}}
    errs = sorted({r.error for r in results if r.error})
    if errs:
        rep["errors"] = errs[:5]
    return rep


def spawn_stack(args):
    """One engine process per replica plus the HTTP front in this process.  Returns (port, cleanup)."""
    from ..entrypoints.openai import app as oa
    from ..entrypoints.openai.client import EngineClient
    tmp = tempfile.mkdtemp(prefix="coffin_bench_")
    procs, socks = [], []
    for r in range(args.replicas):
        sock = os.path.join(tmp, f"engine{r}.sock")
        cmd = [sys.executable, "-m", "coffin_b200.entrypoints.cli.runtime", "--serve", "--sock", sock,
               "--max-seq", str(args.max_seq), "--max-num-seqs", str(args.max_num_seqs)]
        cmd += ["--model", args.model_dir] if args.model_dir else ["--preset", args.preset]
        if args.quant != "none":
            cmd += ["--quant", args.quant]
        if args.snapshot_interval:
            cmd += ["--snapshot-interval", str(args.snapshot_interval), "--snapshots", str(args.snapshots)]
        if args.image_frac > 0:
            cmd += ["--vision", args.vision]
        if args.device:
            cmd += ["--device", args.device]
        env = dict(os.environ)
        if args.replicas > 1 and not args.device:
            env["CUDA_VISIBLE_DEVICES"] = str(r)
        log = open(os.path.join(tmp, f"engine{r}.log"), "w")
        procs.append((subprocess.Popen(cmd, env=env, stdout=log, stderr=subprocess.STDOUT), log))
        socks.append(sock)

    def cleanup() -> None:
        for s in socks:
            try:
                EngineClient(s, 10).call({"op": "stop"})
            except OSError:
                pass
        for p, log in procs:
            try:
                p.wait(20)
            except subprocess.TimeoutExpired:
                p.kill()
            log.close()

    deadline = time.time() + args.startup_timeout
    for s, (p, _) in zip(socks, procs):
        while True:
            if p.poll() is not None:
                cleanup()
                raise RuntimeError(f"engine exited with code {p.returncode}; log in {tmp}")
            try:
                if os.path.exists(s) and EngineClient(s, 5).ping().get("ok"):
                    break
            except OSError:
                pass
            if time.time() > deadline:
                cleanup()
                raise RuntimeError(f"engine did not answer within {args.startup_timeout}s; log in {tmp}")
            time.sleep(0.5)
    oa.configure(oa.ReplicaRouter([EngineClient(s, args.timeout) for s in socks]), served_model_name=args.model,
                 default_max_tokens=args.max_tokens)
    srv = oa.make_server("127.0.0.1", 0)
    threading.Thread(target=srv.serve_forever, daemon=True).start()

    def stop_all() -> None:
        srv.shutdown()
        cleanup()

    return srv.server_address[1], stop_all


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=18080)
    ap.add_argument("--model", default="coffin")
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--rate", type=float, default=8.0, help="mean arrivals per second (0 = all at once)")
    ap.add_argument("--prefix-tokens", type=int, default=1024)
    ap.add_argument("--suffix-tokens", type=int, default=64)
    ap.add_argument("--chars-per-token", type=float, default=1.0,
                    help="filler characters per token (1 for the byte-level fallback tokenizer, ~5 for a BPE vocabulary)")
    ap.add_argument("--max-tokens", type=int, default=128)
    ap.add_argument("--image-frac", type=float, default=0.0)
    ap.add_argument("--image-size", type=int, default=1024)
    ap.add_argument("--timeout", type=float, default=600.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--spawn", action="store_true", help="start the engine process(es) and the HTTP front here")
    ap.add_argument("--preset", default="qwen35-4b")
    ap.add_argument("--model-dir", default=None)
    ap.add_argument("--quant", default="none")
    ap.add_argument("--replicas", type=int, default=1)
    ap.add_argument("--vision", default="default")
    ap.add_argument("--device", default=None)
    ap.add_argument("--max-seq", type=int, default=4096)
    ap.add_argument("--max-num-seqs", type=int, default=64)
    ap.add_argument("--snapshot-interval", type=int, default=0,
                    help="tokens between delta-net state snapshots (a shared prefix is reusable up to the last snapshot inside it)")
    ap.add_argument("--snapshots", type=int, default=32)
    ap.add_argument("--startup-timeout", type=float, default=600.0)
    args = ap.parse_args(argv)
    stop = None
    port = args.port
    if args.spawn:
        port, stop = spawn_stack(args)
    try:
        rep = run_load(args.host, port, args)
    finally:
        if stop is not None:
            stop()
    rep["config"] = {k: getattr(args, k) for k in ("preset", "quant", "replicas", "prefix_tokens", "suffix_tokens",
                                                   "max_tokens", "image_frac", "image_size", "max_num_seqs", "snapshot_interval")}
    print(json.dumps(rep))
    return 0 if rep["failed"] == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
