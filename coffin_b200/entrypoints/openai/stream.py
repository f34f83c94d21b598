"""Incremental filters that turn the engine's raw token text into OpenAI stream deltas.

``AnswerFilter`` splits reasoning (``<think>...</think>``) from the answer and holds back any
suffix that could still turn into ``<tool_call>``, so that markup never leaks into ``content``.
``ToolStream`` consumes what follows ``<tool_call>`` and emits OpenAI ``tool_calls`` deltas as the
call is parsed: first the name (with id), then the arguments as JSON text fragments whose
concatenation equals ``json.dumps(arguments)`` of the non-streaming reply.
Reference: ``entrypoints/openai/stream.py:29-131`` (AnswerFilter), ``:184-441`` (ToolStream).
"""
from __future__ import annotations

import json
import uuid
from typing import Any

from ...utils.tool_call import TC_CLOSE, TC_OPEN, coerce

THINK_OPEN, THINK_CLOSE = "<think>", "</think>"


def _held_suffix(text: str, markers: tuple[str, ...]) -> int:
    """Length of the longest suffix of ``text`` that is a proper prefix of a marker."""
    best = 0
    for m in markers:
        for n in range(min(len(m) - 1, len(text)), 0, -1):
            if text.endswith(m[:n]):
                best = max(best, n)
                break
    return best


class AnswerFilter:
    """Feed text pieces; each ``feed`` returns a list of ``(kind, text)`` with kind in
    ``reasoning`` / ``content`` / ``tool`` (raw text inside tool-call markup)."""

    def __init__(self, in_think: bool = False, emit_reasoning: bool = True, in_tool: bool = False) -> None:
        self.buf = ""
        self.state = "tool" if in_tool else ("think" if in_think else "answer")
        self.emit_reasoning = emit_reasoning
        self.seen_tool = in_tool
        self._answer_started = False

    def feed(self, piece: str) -> list[tuple[str, str]]:
        self.buf += piece
        out: list[tuple[str, str]] = []
        while True:
            if self.state == "think":
                i = self.buf.find(THINK_CLOSE)
                if i >= 0:
                    self._emit(out, "reasoning", self.buf[:i])
                    self.buf = self.buf[i + len(THINK_CLOSE):]
                    self.state = "answer"
                    continue
                hold = _held_suffix(self.buf, (THINK_CLOSE,))
                self._emit(out, "reasoning", self.buf[:len(self.buf) - hold])
                self.buf = self.buf[len(self.buf) - hold:]
                return out
            if self.state == "answer":
                i_t, i_c = self.buf.find(THINK_OPEN), self.buf.find(TC_OPEN)
                if i_t >= 0 and (i_c < 0 or i_t < i_c):
                    self._emit(out, "content", self.buf[:i_t])
                    self.buf = self.buf[i_t + len(THINK_OPEN):]
                    self.state = "think"
                    continue
                if i_c >= 0:
                    self._emit(out, "content", self.buf[:i_c])
                    self.buf = self.buf[i_c + len(TC_OPEN):]
                    self.state = "tool"
                    self.seen_tool = True
                    out.append(("tool_open", ""))
                    continue
                hold = _held_suffix(self.buf, (THINK_OPEN, TC_OPEN))
                self._emit(out, "content", self.buf[:len(self.buf) - hold])
                self.buf = self.buf[len(self.buf) - hold:]
                return out
            # inside <tool_call> ... </tool_call>
            i = self.buf.find(TC_CLOSE)
            if i >= 0:
                if self.buf[:i]:
                    out.append(("tool", self.buf[:i]))
                out.append(("tool_close", ""))
                self.buf = self.buf[i + len(TC_CLOSE):]
                self.state = "answer"
                continue
            hold = _held_suffix(self.buf, (TC_CLOSE,))
            if self.buf[:len(self.buf) - hold]:
                out.append(("tool", self.buf[:len(self.buf) - hold]))
            self.buf = self.buf[len(self.buf) - hold:]
            return out

    def _emit(self, out: list, kind: str, text: str) -> None:
        if not text:
            return
        if kind == "reasoning" and not self.emit_reasoning:
            return
        if kind == "content":
            if not self._answer_started:
                text = text.lstrip("\n")
                if not text:
                    return
                self._answer_started = True
            if self.seen_tool and not text.strip():
                return
        out.append((kind, text))

    def flush(self) -> list[tuple[str, str]]:
        out: list[tuple[str, str]] = []
        if self.buf:
            if self.state == "think":
                self._emit(out, "reasoning", self.buf)
            elif self.state == "answer":
                self._emit(out, "content", self.buf)
            else:
                out.append(("tool", self.buf))
        self.buf = ""
        return out


class ToolStream:
    """Incremental parser of the body of ``<tool_call>`` blocks.

    ``feed(kind, text)`` takes the ``tool_open`` / ``tool`` / ``tool_close`` events of
    ``AnswerFilter`` and returns OpenAI ``tool_calls`` delta entries.  A parameter is emitted once
    its closing tag has been seen (its value is needed whole to decide between a JSON literal and a
    string), as ``"key": <json>`` fragments between ``{`` and ``}``.
    """

    def __init__(self, first_index: int = 0) -> None:
        self.index = first_index - 1
        self.buf = ""
        self.open = False          # inside <function=...>
        self.n_params = 0
        self.calls: list[dict[str, Any]] = []
        self._args: dict[str, Any] = {}
        self._json_mode = False

    def feed(self, kind: str, text: str = "") -> list[dict]:
        out: list[dict] = []
        if kind == "tool_open":
            self.buf = ""
            self._json_mode = False
            return out
        if kind == "tool":
            self.buf += text
            self._drain(out)
            return out
        if kind == "tool_close":
            self._drain(out, final=True)
            self.buf = ""
        return out

    def _start_call(self, name: str, out: list[dict]) -> None:
        self.index += 1
        self.open = True
        self.n_params = 0
        self._args = {}
        call_id = "call_" + uuid.uuid4().hex[:24]
        self.calls.append({"id": call_id, "name": name, "arguments": self._args})
        out.append({"index": self.index, "id": call_id, "type": "function",
                    "function": {"name": name, "arguments": ""}})
        out.append({"index": self.index, "function": {"arguments": "{"}})

    def _end_call(self, out: list[dict]) -> None:
        if self.open:
            out.append({"index": self.index, "function": {"arguments": "}"}})
            self.open = False

    def _param(self, key: str, raw: str, out: list[dict]) -> None:
        val = coerce(raw)
        self._args[key] = val
        frag = ("" if self.n_params == 0 else ", ") + json.dumps(key, ensure_ascii=False) + ": " + \
            json.dumps(val, ensure_ascii=False)
        self.n_params += 1
        out.append({"index": self.index, "function": {"arguments": frag}})

    def _drain(self, out: list[dict], final: bool = False) -> None:
        while True:
            b = self.buf.lstrip() if not self.open else self.buf
            if not self.open:
                if b.startswith("{"):
                    self._json_mode = True
                if self._json_mode:
                    if final:
                        self._json_call(b, out)
                        self.buf = ""
                    return
                i = b.find("<function=")
                if i < 0:
                    return
                j = b.find(">", i)
                if j < 0:
                    return
                self._start_call(b[i + len("<function="):j].strip(), out)
                self.buf = b[j + 1:]
                continue
            i_p, i_e = self.buf.find("<parameter="), self.buf.find("</function>")
            if i_e >= 0 and (i_p < 0 or i_e < i_p):
                self._end_call(out)
                self.buf = self.buf[i_e + len("</function>"):]
                continue
            if i_p >= 0:
                j = self.buf.find(">", i_p)
                k = self.buf.find("</parameter>", j + 1) if j >= 0 else -1
                if j >= 0 and k >= 0:
                    self._param(self.buf[i_p + len("<parameter="):j].strip(), self.buf[j + 1:k], out)
                    self.buf = self.buf[k + len("</parameter>"):]
                    continue
            if final:
                self._end_call(out)
            return

    def _json_call(self, body: str, out: list[dict]) -> None:
        try:
            obj = json.loads(body.strip())
        except ValueError:
            return
        if not isinstance(obj, dict) or not isinstance(obj.get("name"), str):
            return
        args = obj.get("arguments", {})
        if isinstance(args, str):
            try:
                args = json.loads(args)
            except ValueError:
                args = {}
        self.index += 1
        call_id = "call_" + uuid.uuid4().hex[:24]
        self.calls.append({"id": call_id, "name": obj["name"], "arguments": args})
        out.append({"index": self.index, "id": call_id, "type": "function",
                    "function": {"name": obj["name"], "arguments": ""}})
        out.append({"index": self.index, "function": {"arguments": json.dumps(args, ensure_ascii=False)}})

    def finish(self) -> list[dict]:
        out: list[dict] = []
        self._drain(out, final=True)
        return out
