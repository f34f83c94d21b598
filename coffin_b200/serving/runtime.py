"""The resident engine process: model + tokenizer + engine thread behind a JSON-lines protocol.

``Server`` owns the model, the ``LLMEngine`` and one *engine thread*, the only thread that touches
either.  Connection threads translate a request dict into a submission (a sequence, or a
diagnostic job that needs the engine idle) and read results from a per-request queue, so any
number of clients stream concurrently while the engine batches their decode steps.
A failing step fails the requests in flight, resets the engine and keeps the service up.

Wire protocol (one JSON object per line in, one or more lines out) and reply fields follow the
reference: ops ``ping tokenize generate chat chat_stream bench profile ops spec verify
pd_prefill pd_decode pd_decode_batch pd_release reload reset stop`` (``serving/runtime_parts.py:925-1133``),
stream events ``start / token / done / error`` (``:769-869``), engine loop and failure path
(``:196-245``).
"""
from __future__ import annotations

import dataclasses
import os
import queue
import threading
import time
import traceback
from pathlib import Path
from typing import Any, Callable, Iterator

import torch

from ..config import ModelConfig
from ..engine.config import EngineConfig
from ..engine.llm_engine import LLMEngine
from ..engine.sequence import SamplingParams, Sequence
from ..utils.tokenizer import IncrementalDecoder, load_tokenizer
from ..utils.tool_call import parse_tool_calls, split_thinking

DIAGNOSTIC_OPS = {"reload", "reset", "bench", "profile", "ops", "spec", "verify", "pd_prefill", "pd_decode",
                  "pd_decode_batch", "pd_release"}


class MMError(Exception):
    """A multimodal request the engine refuses; ``status`` is the HTTP status the adapter returns."""

    def __init__(self, message: str, status: int = 400) -> None:
        super().__init__(message)
        self.status = status


@dataclasses.dataclass
class _Ticket:
    seq: Sequence
    out: "queue.Queue[tuple[str, Any]]"
    t_submit: float


SPEC_BATCH_MIN_FREE = int(1.5 * 2 ** 30)


def free_bytes(device) -> int:
    """Free device memory in bytes, or -1 when the device has no such notion (the CPU twin)."""
    dev = torch.device(device)
    if dev.type != "cuda" or not torch.cuda.is_available():
        return -1
    return int(torch.cuda.mem_get_info(dev)[0])


def guard_spec_batch(cfg: EngineConfig, free: int) -> EngineConfig:
    """Batched speculation keeps roll-back snapshots and the drafter's rows next to the weights; with less
    than 1.5 GiB free it is switched off (with a line on the log) rather than left to run out of memory in the
    middle of a step (reference: ``serving/runtime_service.py:186-198``)."""
    if cfg.spec_batch and 0 <= free < SPEC_BATCH_MIN_FREE:
        print(f"[serve] spec_batch disabled: only {free / 2 ** 30:.2f} GiB free (batched speculation needs ~1.5 GiB)", flush=True)
        return dataclasses.replace(cfg, spec_batch=False)
    return cfg


class Server:
    def __init__(self, model, cfg: EngineConfig | None = None, tokenizer=None, model_path: str = "",
                 model_name: str = "", builder: Callable[[], Any] | None = None) -> None:
        """``builder`` rebuilds the model for the ``reload`` op (weights stay resident in the
        caller's closure)."""
        self.model = model
        self.model_cfg: ModelConfig = model.cfg
        self.cfg = cfg or EngineConfig()
        self.tok = tokenizer or load_tokenizer(model_path or None, self.model_cfg.vocab_size)
        self.model_path = model_path
        self.model_name = model_name or Path(model_path or self.model_cfg.name).name
        self.builder = builder
        t0 = time.time()
        self.cfg = guard_spec_batch(self.cfg, free_bytes(getattr(model, "device", "cpu")))
        self.engine = LLMEngine(model, self.cfg)
        self.warmup_s = round(self.engine.warmup(), 3) if self.cfg.warmup else 0.0
        self.build_s = round(time.time() - t0, 3)
        self.load_s = 0.0
        self.eos = tuple(i for i in self.tok.eos_ids if i < self.model_cfg.vocab_size)
        self.n_req = self.n_reload = self.n_image_req = 0
        self.vision = getattr(model, "vision", None)
        self.processor = None                    # image recipe, loaded by the first image request (serving/processor.py)
        self._processor_failed: str | None = None
        self._inbox: "queue.Queue[Any]" = queue.Queue()
        self._tickets: dict[int, _Ticket] = {}
        self._wake = threading.Condition()
        self._running = False
        self._thread: threading.Thread | None = None
        self._stopping = threading.Event()
        self.last_error: str | None = None
        # multi-rank engines: an object with ``check() -> list[int]`` (``parallel.control.Heartbeat``);
        # the loop asks it between steps, before the next kernels are launched
        self.heartbeat = None
        self.dead_ranks: list[int] = []

    def attach_heartbeat(self, hb) -> None:
        self.heartbeat = hb

    # ------------------------------------------------------------------ lifecycle
    def start(self) -> None:
        if self._running:
            return
        self._running = True
        self._thread = threading.Thread(target=self._engine_loop, name="engine", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._running = False
        self._stopping.set()
        with self._wake:
            self._wake.notify_all()
        if self._thread is not None and self._thread is not threading.current_thread():
            self._thread.join(timeout=10)

    @property
    def stopping(self) -> bool:
        return self._stopping.is_set()

    def _engine_loop(self) -> None:
        dev = getattr(self.model, "device", None)
        if dev is not None and dev.type == "cuda":
            torch.cuda.set_device(dev)
        while self._running:
            self._drain_inbox()
            if not self.engine.has_work():
                with self._wake:
                    if self._inbox.empty() and self._running:
                        self._wake.wait(timeout=0.05)
                continue
            if self.heartbeat is not None:
                dead = self.heartbeat.check()
                if dead:
                    # a peer is gone: nothing more is launched for this group; the requests in flight
                    # fail on the host and the launcher restarts the ranks (no elastic re-ranking)
                    self.dead_ranks = dead
                    self._fail(RuntimeError(f"rank(s) {dead} stopped answering the heartbeat"))
                    self._running = False
                    self._stopping.set()
                    break
            try:
                outs = self.engine.step()
            except Exception as exc:            # noqa: BLE001 - the service must survive a bad step
                self._fail(exc)
                continue
            for o in outs:
                t = self._tickets.get(o.seq.seq_id)
                if t is None:
                    continue
                if o.token is not None:
                    t.out.put(("token", o.token))
                if o.finished:
                    t.out.put(("done", o.seq.finish_reason))
                    self._tickets.pop(o.seq.seq_id, None)

    def _drain_inbox(self) -> None:
        while True:
            try:
                item = self._inbox.get_nowait()
            except queue.Empty:
                return
            kind = item[0]
            if kind == "submit":
                _, prompt, params, mm, outq = item
                try:
                    seq = self.engine.add_request(prompt, params, mm)
                    self._tickets[seq.seq_id] = _Ticket(seq, outq, time.monotonic())
                    if os.environ.get("COFFIN_DEBUG_STEP"):
                        sch = self.engine.scheduler
                        print(f"[req] t={time.time():.3f} seq={seq.seq_id} waiting={len(sch.waiting)} "
                              f"running={len(sch.running)}", flush=True)
                    outq.put(("seq", seq))
                except Exception as exc:        # noqa: BLE001
                    outq.put(("error", str(exc)))
            elif kind == "abort":
                seq = item[1]
                self.engine.abort(seq)
                t = self._tickets.pop(seq.seq_id, None)
                if t:
                    t.out.put(("done", "abort"))
            elif kind == "job":
                _, fn, outq = item
                if self.engine.has_work():
                    outq.put(("error", "engine busy: diagnostic ops need an idle engine"))
                    continue
                try:
                    outq.put(("result", fn()))
                except Exception as exc:        # noqa: BLE001
                    outq.put(("error", f"{type(exc).__name__}: {exc}"))

    def _fail(self, exc: Exception) -> None:
        self.last_error = "".join(traceback.format_exception_only(type(exc), exc)).strip()
        print(f"[serve] engine step failed: {self.last_error}", flush=True)
        for t in list(self._tickets.values()):
            t.out.put(("error", f"engine step failed: {self.last_error}"))
        self._tickets.clear()
        try:
            self.engine.reset()
        except Exception as exc2:               # noqa: BLE001
            print(f"[serve] reset after failure failed: {exc2}", flush=True)

    # ------------------------------------------------------------------ submission helpers
    def _submit(self, prompt: list[int], params: SamplingParams, mm=None) -> tuple[Sequence, "queue.Queue"]:
        outq: "queue.Queue[tuple[str, Any]]" = queue.Queue()
        self._inbox.put(("submit", prompt, params, mm, outq))
        with self._wake:
            self._wake.notify_all()
        kind, val = outq.get(timeout=60)
        if kind == "error":
            raise ValueError(val)
        return val, outq

    def _job(self, fn: Callable[[], dict], timeout: float = 600) -> dict:
        outq: "queue.Queue[tuple[str, Any]]" = queue.Queue()
        self._inbox.put(("job", fn, outq))
        with self._wake:
            self._wake.notify_all()
        kind, val = outq.get(timeout=timeout)
        if kind == "error":
            rep = {"ok": False, "error": val}
            if str(val).startswith(("DiagError", "ValueError")):
                rep["status"] = 400
            return rep
        return val

    def _sampling(self, req: dict) -> SamplingParams:
        max_new = int(req.get("max_new", 256))
        secs = float(req.get("max_seconds", 0) or 0)
        return SamplingParams(temperature=float(req.get("temperature", 0.0) or 0.0), max_tokens=max(1, max_new),
                              eos=self.eos, ignore_eos=bool(req.get("ignore_eos", False)),
                              deadline=time.monotonic() + secs if secs > 0 else None,
                              seed=req.get("seed"),
                              spec_k=int(req["spec_k"]) if req.get("spec_k") is not None else -1)

    def _collect(self, seq: Sequence, outq: "queue.Queue", on_token=None) -> str:
        while True:
            kind, val = outq.get(timeout=3600)
            if kind == "token":
                if on_token:
                    on_token(val)
            elif kind == "done":
                return val
            elif kind == "error":
                raise RuntimeError(val)

    def _result(self, seq: Sequence, t0: float, max_new: int) -> dict:
        first = seq.first_token_time or time.monotonic()
        end = seq.finish_time or time.monotonic()
        prefill_ms = (first - t0) * 1e3
        decode_ms = max(0.0, (end - first) * 1e3)
        n_new = len(seq.output)
        return {"tokens": list(seq.output), "n_prompt": len(seq.prompt), "n_new": n_new, "max_new": max_new,
                "window_full": seq.finish_reason == "window", "cached_tokens": seq.cached_tokens,
                "prefill_ms": round(prefill_ms, 2), "decode_ms": round(decode_ms, 2),
                "decode_tok_s": round((n_new - 1) / (decode_ms / 1e3), 2) if decode_ms > 0 and n_new > 1 else 0.0,
                "stopped": seq.finish_reason,
                "spec_k": self.engine.runner.spec_k_of(seq) if seq.params.temperature <= 0 else 0,
                "spec": ({"steps": seq.spec_steps, "drafted": seq.spec_drafted, "accepted": seq.spec_accepted,
                          "accept_rate": round(seq.spec_accepted / seq.spec_drafted, 4) if seq.spec_drafted else 0.0}
                         if seq.spec_steps else None)}

    # ------------------------------------------------------------------ chat rendering
    def _render(self, req: dict) -> tuple[list[int], bool, str | None]:
        """Prompt ids for a chat request, whether the prompt ends inside ``<think>``, and the
        forced tool-call opener (if the adapter asked for one)."""
        msgs = req.get("messages") or []
        thinking = bool(req.get("enable_thinking", True))
        text = self.tok.apply_chat_template(msgs, tools=req.get("tools") or None, tokenize=False,
                                            add_generation_prompt=True, enable_thinking=thinking)
        forced = req.get("tool_prefix") or None
        if forced:
            if text.rstrip().endswith("<think>"):
                text = text.rstrip()[: -len("<think>")] + "<think>\n\n</think>\n\n"
            text += forced
        opens = text.rstrip().endswith("<think>")
        return self.tok.encode(text), opens, forced

    def _prepare_mm(self, req: dict, prompt: list[int]):
        images = req.get("images") or []
        if not images:
            return None, prompt
        if self.vision is None or not self.cfg.vision:
            raise MMError("this engine was started without a vision tower", 503)
        if len(images) > self.cfg.max_images:
            raise MMError(f"too many images: {len(images)} > {self.cfg.max_images}", 400)
        from .multimodal import build_mm_input
        self.n_image_req += 1
        return build_mm_input(self, images, prompt)

    # ------------------------------------------------------------------ streaming chat
    def stream_chat(self, req: dict) -> Iterator[dict]:
        try:
            prompt, opens, forced = self._render(req)
            mm, prompt = self._prepare_mm(req, prompt)
            params = self._sampling(req)
            t0 = time.monotonic()
            seq, outq = self._submit(prompt, params, mm)
        except MMError as exc:
            yield {"type": "error", "error": str(exc), "status": exc.status}
            return
        except Exception as exc:                # noqa: BLE001
            yield {"type": "error", "error": str(exc), "status": 400}
            return
        self.n_req += 1
        yield {"type": "start", "n_prompt": len(prompt), "prompt_opens_think": opens, "forced_tool": forced}
        dec = IncrementalDecoder(self.tok)
        waited = 0.0
        try:
            while True:
                # {"type": "tick"} lines are not part of the protocol: they hand control to the transport while
                # nothing printable is produced (a long prefill, tokens that complete no character), so that it can
                # notice a client that went away and close this generator, which aborts the sequence
                try:
                    kind, val = outq.get(timeout=0.5)
                except queue.Empty:
                    waited += 0.5
                    if waited > 3600:
                        raise
                    yield {"type": "tick"}
                    continue
                waited = 0.0
                if kind == "token":
                    piece = dec.push(val)
                    yield {"type": "token", "text": piece} if piece else {"type": "tick"}
                elif kind == "done":
                    break
                elif kind == "error":
                    yield {"type": "error", "error": val, "status": 500}
                    return
        except GeneratorExit:
            self._inbox.put(("abort", seq))
            raise
        tail = dec.flush()
        if tail:
            yield {"type": "token", "text": tail}
        done = self._chat_reply(seq, t0, params.max_tokens, opens, forced, mm)
        done["type"] = "done"
        yield done

    def _chat_reply(self, seq: Sequence, t0: float, max_new: int, opens: bool, forced: str | None, mm) -> dict:
        rep = self._result(seq, t0, max_new)
        raw = self.tok.decode(seq.output, skip_special_tokens=True)
        full = (forced or "") + raw
        thinking, answer = split_thinking(full, prompt_opens_think=opens and not forced)
        content, calls = parse_tool_calls(answer)
        rep.update({"ok": True, "text": content, "thinking": thinking, "raw": raw,
                    "tool_calls": [c.to_openai_dict() for c in calls], "forced_tool": forced,
                    "n_images": len(mm.spans) if mm is not None else 0,
                    "image_tokens": sum(e - s for s, e in mm.spans) if mm is not None else 0})
        rep.pop("tokens", None)
        return rep

    # ------------------------------------------------------------------ request dispatch
    def handle(self, req: dict) -> dict:
        op = req.get("op", "ping")
        if op in DIAGNOSTIC_OPS and (self._tickets or self.engine.has_work()):
            return {"ok": False, "error": f"op {op!r} is refused while requests are in flight", "status": 409}
        try:
            return self._handle_impl(op, req)
        except MMError as exc:
            return {"ok": False, "error": str(exc), "status": exc.status}
        except Exception as exc:                # noqa: BLE001
            return {"ok": False, "error": f"{type(exc).__name__}: {exc}"}

    def _handle_impl(self, op: str, req: dict) -> dict:
        if op == "ping":
            return self._ping()
        if op == "tokenize":
            return {"ok": True, "tokens": self.tok.encode(req.get("prompt", ""))}
        if op == "stop":
            return {"ok": True, "stopping": True}
        if op == "reset":
            return self._job(lambda: (self.engine.reset(), {"ok": True})[1])
        if op == "reload":
            return self._job(self._reload)
        if op == "generate":
            prompt = req.get("tokens") or self.tok.encode(req.get("prompt", ""))
            params = self._sampling(req)
            t0 = time.monotonic()
            seq, outq = self._submit([int(t) for t in prompt], params)
            self.n_req += 1
            self._collect(seq, outq)
            rep = self._result(seq, t0, params.max_tokens)
            rep.update({"ok": True, "text": self.tok.decode(seq.output, skip_special_tokens=True)})
            return rep
        if op == "chat":
            prompt, opens, forced = self._render(req)
            mm, prompt = self._prepare_mm(req, prompt)
            params = self._sampling(req)
            t0 = time.monotonic()
            seq, outq = self._submit(prompt, params, mm)
            self.n_req += 1
            self._collect(seq, outq)
            return self._chat_reply(seq, t0, params.max_tokens, opens, forced, mm)
        if op in ("bench", "profile", "ops", "spec", "verify", "pd_prefill", "pd_decode", "pd_decode_batch", "pd_release"):
            from . import diagnostics
            return self._job(lambda: getattr(diagnostics, op)(self, req))
        return {"ok": False, "error": f"unknown op {op!r}", "status": 400}

    def _reload(self) -> dict:
        if self.builder is None:
            return {"ok": False, "error": "this server was started without a model builder"}
        t0 = time.time()
        self.engine.reset()
        self.model = self.builder()
        self.vision = getattr(self.model, "vision", None)       # the rebuilt model brings its own tower ...
        self.processor, self._processor_failed = None, None    # ... and the image recipe is read again
        self.engine = LLMEngine(self.model, self.cfg)
        self.warmup_s = round(self.engine.warmup(), 3) if self.cfg.warmup else 0.0
        self.n_reload += 1
        self.build_s = round(time.time() - t0, 3)
        return {"ok": True, "build_s": self.build_s, "n_reload": self.n_reload, "backend": "sm_100a", "reason": "reload"}

    def _ping(self) -> dict:
        dev = getattr(self.model, "device", torch.device("cpu"))
        vram = 0.0
        if dev.type == "cuda":
            vram = round(torch.cuda.memory_allocated(dev) / 2 ** 30, 2)
        st = self.engine.stats()
        from ..ops import _lib
        return {"ok": True, "model": self.model_name, "model_path": self.model_path,
                "arch": self.model_cfg.architecture, "graph": self.cfg.graph, "max_seq": self.engine.max_seq,
                "load_s": self.load_s, "build_s": self.build_s, "warmup_s": getattr(self, "warmup_s", 0.0), "n_req": self.n_req, "n_reload": self.n_reload,
                "backend": "sm_100a" if dev.type == "cuda" else "oracle-cpu", "device": str(dev),
                "native_ops": len(_lib.exported()) if dev.type == "cuda" and _lib.available() else 0,
                "total_ops": len(_lib.exported()) if _lib.available() else 0,
                "int8": self.cfg.quant != "none", "vram_gib": vram, "batch": self.cfg.max_num_seqs > 1,
                "decode_capacity": self.cfg.max_num_seqs, "vision": self.vision is not None, "vision_int8": False,
                "image_max_pixels": self.cfg.image_max_pixels, "image_min_pixels": self.cfg.image_min_pixels,
                "max_images": self.cfg.max_images, "n_image_req": self.n_image_req,
                "processor": (None if self.vision is None else "failed: " + self._processor_failed if self._processor_failed
                              else self.processor.source if self.processor is not None else "not loaded"),
                "queue": {"waiting": st["queue"]["waiting"], "running": st["queue"]["running"] + st["queue"]["prefilling"]},
                "prefix": st["blocks"]["prefix"], "last_error": self.last_error}
