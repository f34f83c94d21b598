"""Client of the engine socket used by the HTTP adapter: one connection per request.

``call`` returns the single reply line, ``stream`` yields the event lines of a ``chat_stream``
request.  ``_open`` is the one place that creates the connection (tests point it at a TCP fake).
Reference: ``entrypoints/openai/client.py:16-116``.
"""
from __future__ import annotations

import json
import socket
from typing import Iterator


class EngineClient:
    def __init__(self, sock_path: str, timeout: float = 900.0) -> None:
        self.sock_path = sock_path
        self.timeout = timeout

    def _open(self) -> socket.socket:
        s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        s.settimeout(self.timeout)
        s.connect(self.sock_path)
        return s

    def call(self, req: dict) -> dict:
        s = self._open()
        try:
            s.sendall((json.dumps(req) + "\n").encode())
            with s.makefile("rb") as fh:
                line = fh.readline()
            if not line:
                return {"ok": False, "error": "engine closed the connection", "status": 503}
            return json.loads(line.decode())
        finally:
            s.close()

    def stream(self, req: dict) -> Iterator[dict]:
        s = self._open()
        try:
            s.sendall((json.dumps(req) + "\n").encode())
            with s.makefile("rb") as fh:
                for line in fh:
                    if line.strip():
                        yield json.loads(line.decode())
        finally:
            s.close()

    def ping(self) -> dict:
        return self.call({"op": "ping"})
