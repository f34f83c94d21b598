"""Unix-socket JSON-lines transport of the engine process, and its client call.

One request per connection: the client writes one JSON object and a newline; the server answers
with one line (``chat_stream``: one line per stream event) and closes.  Replies carry ``ok`` and
``wall_ms``.  Under tensor parallelism rank 0 owns the socket and fans every request out to the
worker ranks over the CPU process group before handling it, so that all ranks replay the same op
(reference: ``serving/runtime_transport.py:99-135`` worker loop, ``:146-250`` serve, ``:253-340``
connection handler, ``:343-371`` client).
"""
from __future__ import annotations

import json
import os
import select
import socket
import threading
import time
from typing import Iterator

DEFAULT_SOCK = os.environ.get("ENGINE_SOCK", "/tmp/coffin_b200.sock")


def banner(srv) -> str:
    p = srv._ping()
    return (f"[serve] backend={p['backend']} device={p['device']} native={p['native_ops']}/{p['total_ops']} "
            f"graph={p['graph']}\n[serve] model={p['model']} arch={p['arch']} max_seq={p['max_seq']} "
            f"rows={p['decode_capacity']} vram={p['vram_gib']}GiB")


def _recv_line(conn: socket.socket) -> bytes:
    buf = b""
    while not buf.endswith(b"\n"):
        chunk = conn.recv(65536)
        if not chunk:
            break
        buf += chunk
    return buf


def _peer_closed(conn: socket.socket) -> bool:
    """True when the other end of a stream connection has closed it (an orderly shutdown reads as b"")."""
    try:
        readable, _, _ = select.select([conn], [], [], 0)
        return bool(readable) and conn.recv(1, socket.MSG_PEEK | socket.MSG_DONTWAIT) == b""
    except (BlockingIOError, InterruptedError):
        return False
    except (OSError, ValueError):       # ValueError: the descriptor is already closed on this side
        return True


def _serve_connection(srv, conn: socket.socket, fanout=None) -> None:
    try:
        req = json.loads(_recv_line(conn).decode() or "{}")
        t0 = time.time()
        if fanout is not None:
            fanout(req)
        if req.get("op") == "chat_stream":
            lines = srv.stream_chat(req)
            try:
                gone = False
                for line in lines:
                    if line.get("type") == "tick":       # nothing to send: see whether the client is still there
                        if fanout is None and _peer_closed(conn):
                            print("[serve] chat_stream: client went away, sequence aborted", flush=True)
                            return
                        continue
                    if gone:
                        continue
                    try:
                        conn.sendall((json.dumps(line, ensure_ascii=False) + "\n").encode())
                    except (BrokenPipeError, ConnectionResetError):
                        if fanout is None:
                            raise
                        gone = True      # the other ranks replay this request step for step: finish it, send nothing
            finally:
                lines.close()        # a client that went away mid-stream: the generator aborts its sequence
            print(f"[serve] chat_stream -> {round((time.time() - t0) * 1000, 1)}ms", flush=True)
            return
        rep = srv.handle(req)
        rep["wall_ms"] = round((time.time() - t0) * 1000, 1)
        conn.sendall((json.dumps(rep, ensure_ascii=False) + "\n").encode())
        print(f"[serve] {req.get('op')} -> {rep.get('wall_ms')}ms", flush=True)
        if rep.get("stopping"):
            srv.stop()
    except (BrokenPipeError, ConnectionResetError):
        pass
    except Exception as exc:        # noqa: BLE001 - a bad request must not take the server down
        rep = {"ok": False, "error": str(exc)}
        status = getattr(exc, "status", None)
        if status:
            rep["status"] = status
        try:
            conn.sendall((json.dumps(rep) + "\n").encode())
        except OSError:
            pass
        print(f"[serve] error: {exc}", flush=True)
    finally:
        conn.close()


def serve(srv, sock_path: str = DEFAULT_SOCK, fanout=None, ready: threading.Event | None = None) -> None:
    """Listen until the server is stopped.  One thread per connection."""
    if os.path.exists(sock_path):
        os.unlink(sock_path)
    srv.start()
    print(banner(srv), flush=True)
    lst = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    lst.bind(sock_path)
    lst.listen(64)
    lst.settimeout(0.5)
    print(f"[serve] listening on {sock_path}", flush=True)
    if ready is not None:
        ready.set()
    try:
        while not srv.stopping:
            try:
                conn, _ = lst.accept()
            except socket.timeout:
                continue
            threading.Thread(target=_serve_connection, args=(srv, conn, fanout), daemon=True).start()
    finally:
        lst.close()
        try:
            os.unlink(sock_path)
        except OSError:
            pass
        srv.stop()


def call(sock_path: str, req: dict, timeout: float | None = None) -> dict:
    """Send one request, return the one-line reply (which may carry ``ok: false``)."""
    s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    s.settimeout(timeout)
    s.connect(sock_path)
    s.sendall((json.dumps(req) + "\n").encode())
    buf = _recv_line(s)
    s.close()
    return json.loads(buf.decode())


def stream(sock_path: str, req: dict, timeout: float | None = None) -> Iterator[dict]:
    """Send a ``chat_stream`` request and yield its event lines."""
    s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    s.settimeout(timeout)
    s.connect(sock_path)
    s.sendall((json.dumps(req) + "\n").encode())
    fh = s.makefile("rb")
    try:
        for line in fh:
            if line.strip():
                yield json.loads(line.decode())
    finally:
        fh.close()
        s.close()
