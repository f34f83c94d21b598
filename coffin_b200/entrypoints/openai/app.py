"""OpenAI-compatible HTTP adapter in front of the engine socket.

Endpoints: ``GET /health`` and ``/healthz`` (engine ping passthrough), ``GET /v1/models``,
``POST /v1/chat/completions`` (JSON or SSE), ``OPTIONS`` for CORS.  The adapter holds no model:
it validates and normalises the request, forwards it over the unix socket, and shapes the reply
(``chat.completion`` / ``chat.completion.chunk`` with ``tool_calls``, ``reasoning_content``,
``usage.prompt_tokens_details.cached_tokens``).  Several adapters (or one adapter with several
engine sockets) give data-parallel replicas: ``ReplicaRouter`` picks the engine with the fewest
requests in flight.  Reference: ``entrypoints/openai/app.py:162-510``.
"""
from __future__ import annotations

import json
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Any

from ...utils.tool_call import TC_OPEN
from .client import EngineClient
from .request import RequestError, build_engine_request, include_usage
from .stream import AnswerFilter, ToolStream


class ReplicaRouter:
    """Least-loaded choice among engine replicas (each an ``EngineClient``)."""

    def __init__(self, clients: list[EngineClient]) -> None:
        if not clients:
            raise ValueError("need at least one engine")
        self.clients = clients
        self.inflight = [0] * len(clients)
        self.served = [0] * len(clients)
        self._lock = threading.Lock()

    def acquire(self) -> int:
        with self._lock:
            i = min(range(len(self.clients)), key=lambda j: (self.inflight[j], self.served[j]))
            self.inflight[i] += 1
            self.served[i] += 1
            return i

    def release(self, i: int) -> None:
        with self._lock:
            self.inflight[i] -= 1

    def call(self, req: dict) -> dict:
        i = self.acquire()
        try:
            return self.clients[i].call(req)
        finally:
            self.release(i)

    def stream(self, req: dict):
        i = self.acquire()
        try:
            yield from self.clients[i].stream(req)
        finally:
            self.release(i)

    def ping(self) -> dict:
        return self.clients[0].ping()


STATE: dict[str, Any] = {
    "engine": None, "served_model_name": "coffin-b200", "default_max_tokens": 8192, "enable_thinking": True,
    "max_decode_seconds": 180.0, "max_images": 4, "max_image_bytes": 10 << 20, "max_image_total_bytes": 32 << 20,
    "vision": True,      # False when the engine reported no vision tower (``--no-vision``): image requests answer 503 here
}


def configure(engine, **kw) -> None:
    STATE["engine"] = engine
    for k, v in kw.items():
        if v is not None:
            STATE[k] = v


def finish_reason(out: dict) -> str:
    if out.get("tool_calls"):
        return "tool_calls"
    if out.get("stopped") in ("timeout", "deadline"):
        return "length"
    n_new, n_max = int(out.get("n_new") or 0), int(out.get("max_new") or 0)
    return "length" if n_max > 0 and n_new >= n_max else "stop"


def usage(out: dict) -> dict:
    pt, ct = int(out.get("n_prompt") or 0), int(out.get("n_new") or 0)
    u = {"prompt_tokens": pt, "completion_tokens": ct, "total_tokens": pt + ct,
         "prompt_tokens_details": {"cached_tokens": int(out.get("cached_tokens") or 0)}}
    if "prefill_ms" in out:     # engine-side clock: submit -> first token, first -> last token (an extension field)
        u["timing"] = {"ttft_ms": out.get("prefill_ms"), "decode_ms": out.get("decode_ms")}
    return u


class Handler(BaseHTTPRequestHandler):
    protocol_version = "HTTP/1.1"
    server_version = "coffin-b200"

    def log_message(self, fmt, *args) -> None:  # quiet by default; requests are logged explicitly
        pass

    # ------------------------------------------------------------------ plumbing
    def _cors(self) -> None:
        self.send_header("Access-Control-Allow-Origin", "*")
        self.send_header("Access-Control-Allow-Headers", "*")
        self.send_header("Access-Control-Allow-Methods", "GET, POST, OPTIONS")

    def _json(self, status: int, obj: dict) -> None:
        body = json.dumps(obj, ensure_ascii=False).encode()
        self.send_response(status)
        self.send_header("Content-Type", "application/json")
        self.send_header("Content-Length", str(len(body)))
        self._cors()
        self.end_headers()
        self.wfile.write(body)

    def _error(self, status: int, message: str, etype: str | None = None, code: str | None = None) -> None:
        etype = etype or ("invalid_request_error" if status < 500 else "server_error")
        self._json(status, {"error": {"message": message, "type": etype, "code": code}})

    def do_OPTIONS(self) -> None:
        self.send_response(204)
        self._cors()
        self.send_header("Content-Length", "0")
        self.end_headers()

    def do_GET(self) -> None:
        path = self.path.split("?", 1)[0]
        if path in ("/health", "/healthz"):
            try:
                p = STATE["engine"].ping()
            except OSError as exc:
                self._json(503, {"status": "engine unreachable", "error": str(exc)})
                return
            p.update({"status": "ok" if p.get("ok") else "error", "served_model_name": STATE["served_model_name"]})
            self._json(200 if p.get("ok") else 503, p)
        elif path == "/v1/models":
            self._json(200, {"object": "list", "data": [{"id": STATE["served_model_name"], "object": "model",
                                                         "created": int(time.time()), "owned_by": "coffin-b200"}]})
        else:
            self._error(404, f"no route {path}", code="not_found")

    def do_POST(self) -> None:
        path = self.path.split("?", 1)[0]
        if path != "/v1/chat/completions":
            self._error(404, f"no route {path}", code="not_found")
            return
        try:
            n = int(self.headers.get("Content-Length") or 0)
            body = json.loads(self.rfile.read(n).decode() or "{}")
            if not isinstance(body, dict):
                raise ValueError("body must be a JSON object")
        except (ValueError, UnicodeDecodeError) as exc:
            self._error(400, f"invalid JSON body: {exc}")
            return
        self._chat(body)

    # ------------------------------------------------------------------ chat
    def _chat(self, body: dict) -> None:
        stream = bool(body.get("stream"))
        try:
            req, single = build_engine_request(
                body, default_max_tokens=STATE["default_max_tokens"], default_thinking=STATE["enable_thinking"],
                max_decode_seconds=STATE["max_decode_seconds"], max_images=STATE["max_images"],
                max_image_bytes=STATE["max_image_bytes"], max_image_total_bytes=STATE["max_image_total_bytes"],
                stream=stream)
        except RequestError as exc:
            self._error(exc.status, str(exc), code=exc.code)
            return
        if req.get("images") and STATE.get("vision") is False:
            self._error(503, "this server's engine was started with --no-vision: image inputs are disabled", "server_error")
            return
        cid = "chatcmpl-" + uuid.uuid4().hex[:24]
        created = int(time.time())
        model = body.get("model") or STATE["served_model_name"]
        t0 = time.time()
        try:
            if stream:
                self._chat_stream(req, cid, created, model, single, include_usage(body))
            else:
                self._chat_once(req, cid, created, model, single)
        except OSError as exc:
            try:
                self._error(503, f"engine unreachable: {exc}", "server_error")
            except OSError:
                pass
        print(f"[http] chat stream={stream} {round((time.time() - t0) * 1e3)}ms", flush=True)

    def _chat_once(self, req: dict, cid: str, created: int, model: str, single: bool) -> None:
        out = STATE["engine"].call(req)
        if not out.get("ok", True):
            status = int(out.get("status") or 500)
            self._error(status, f"engine: {out.get('error')}")
            return
        calls = out.get("tool_calls") or []
        if single and len(calls) > 1:
            calls = calls[:1]
        text = out.get("text") or ""
        if calls:
            text = text.split(TC_OPEN, 1)[0].strip()
        message: dict = {"role": "assistant", "content": text or None}
        if calls:
            message["tool_calls"] = calls
        if out.get("thinking"):
            message["reasoning_content"] = out["thinking"]
        self._json(200, {"id": cid, "object": "chat.completion", "created": created, "model": model,
                         "choices": [{"index": 0, "message": message,
                                      "finish_reason": finish_reason({**out, "tool_calls": calls})}],
                         "usage": usage(out)})

    def _sse(self, obj: dict | str) -> None:
        data = obj if isinstance(obj, str) else json.dumps(obj, ensure_ascii=False)
        chunk = f"data: {data}\n\n".encode()
        self.wfile.write(f"{len(chunk):x}\r\n".encode() + chunk + b"\r\n")
        self.wfile.flush()

    def _chat_stream(self, req: dict, cid: str, created: int, model: str, single: bool, want_usage: bool) -> None:
        lines = STATE["engine"].stream(req)
        try:
            self._relay_stream(lines, cid, created, model, single, want_usage)
        finally:
            lines.close()      # closes the engine connection: an HTTP client that went away ends its sequence there

    def _relay_stream(self, lines, cid: str, created: int, model: str, single: bool, want_usage: bool) -> None:
        first = next(lines, None)
        if first is None:
            self._error(503, "engine closed the stream", "server_error")
            return
        if first.get("type") == "error":
            self._error(int(first.get("status") or 500), f"engine: {first.get('error')}")
            return
        self.send_response(200)
        self.send_header("Content-Type", "text/event-stream")
        self.send_header("Cache-Control", "no-cache")
        self.send_header("Transfer-Encoding", "chunked")
        self._cors()
        self.end_headers()

        def chunk(delta: dict, finish: str | None = None, **extra) -> dict:
            return {"id": cid, "object": "chat.completion.chunk", "created": created, "model": model,
                    "choices": [{"index": 0, "delta": delta, "finish_reason": finish}], **extra}

        self._sse(chunk({"role": "assistant", "content": ""}))
        forced = first.get("forced_tool")
        filt = AnswerFilter(in_think=bool(first.get("prompt_opens_think")) and not forced, in_tool=False)
        tools = ToolStream()
        n_calls = 0
        done: dict | None = None

        def emit(events) -> None:
            nonlocal n_calls
            for kind, text in events:
                if kind == "content":
                    self._sse(chunk({"content": text}))
                elif kind == "reasoning":
                    self._sse(chunk({"reasoning_content": text}))
                else:
                    for d in tools.feed(kind, text):
                        if single and d["index"] > 0:
                            continue
                        if "id" in d:
                            n_calls += 1
                        self._sse(chunk({"tool_calls": [d]}))

        if forced:
            emit(filt.feed(forced))
        for line in lines:
            t = line.get("type")
            if t == "token":
                emit(filt.feed(line.get("text", "")))
            elif t == "done":
                done = line
                break
            elif t == "error":
                self._sse({"error": {"message": f"engine: {line.get('error')}", "type": "server_error", "code": None}})
                break
        emit(filt.flush())
        for d in tools.finish():
            if not (single and d["index"] > 0):
                self._sse(chunk({"tool_calls": [d]}))
        if done is not None:
            fr = finish_reason({**done, "tool_calls": n_calls > 0})
            self._sse(chunk({}, fr))
            if want_usage:
                u = chunk({}, None, usage=usage(done))
                u["choices"] = []
                self._sse(u)
        self._sse("[DONE]")
        self.wfile.write(b"0\r\n\r\n")
        self.wfile.flush()


def make_server(host: str, port: int) -> ThreadingHTTPServer:
    srv = ThreadingHTTPServer((host, port), Handler)
    srv.daemon_threads = True
    return srv
