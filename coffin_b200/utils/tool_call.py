"""Qwen3.5 tool-call wire format: parsing and serialisation (standard library only).

The chat template teaches the model to answer a tool request with

    <tool_call>
    <function=get_weather>
    <parameter=city>
    Beijing
    </parameter>
    </function>
    </tool_call>

(several ``<function=...>`` blocks per call and several ``<parameter=...>`` blocks per function
are allowed; a JSON body ``{"name": ..., "arguments": {...}}`` inside ``<tool_call>`` is accepted
too).  Parameter values are raw text: a value that parses as a JSON literal is unwrapped, anything
else stays a string.  Reasoning arrives in ``<think>...</think>`` before the answer.  Parsing never
raises on malformed or truncated text — it yields fewer calls — because it runs on degraded
generations and on partial streams.  Reference: ``utils/tool_call.py`` (whole file).
"""
from __future__ import annotations

import dataclasses
import json
import re
import uuid
from typing import Any

TC_OPEN, TC_CLOSE = "<tool_call>", "</tool_call>"
_TC = re.compile(r"<tool_call>(.*?)</tool_call>", re.DOTALL)
_FN = re.compile(r"<function=([^>\n]+)>(.*?)</function>", re.DOTALL)
_FN_OPEN = re.compile(r"<function=([^>\n]+)>(.*)", re.DOTALL)
_PARAM = re.compile(r"<parameter=([^>\n]+)>(.*?)</parameter>", re.DOTALL)
_THINK = re.compile(r"<think>(.*?)</think>", re.DOTALL)


@dataclasses.dataclass
class ToolCall:
    name: str
    arguments: dict[str, Any] = dataclasses.field(default_factory=dict)
    id: str = ""
    raw: str = ""

    def __post_init__(self) -> None:
        if not self.id:
            self.id = "call_" + uuid.uuid4().hex[:24]

    def to_openai_dict(self) -> dict[str, Any]:
        return {"id": self.id, "type": "function",
                "function": {"name": self.name, "arguments": json.dumps(self.arguments, ensure_ascii=False)}}

    def to_template_dict(self) -> dict[str, Any]:
        return {"id": self.id, "type": "function", "function": {"name": self.name, "arguments": dict(self.arguments)}}


def coerce(text: str) -> Any:
    """A parameter value: JSON literal if it is one (numbers, booleans, null, objects, arrays,
    quoted strings), else the stripped text itself.  Leading-zero integers stay strings."""
    v = text.strip("\n")
    s = v.strip()
    if not s:
        return v
    if re.fullmatch(r"-?0\d+", s):
        return s
    try:
        return json.loads(s)
    except (ValueError, TypeError):
        return v.strip() if "\n" not in v.strip() else v


def split_thinking(text: str, prompt_opens_think: bool = False) -> tuple[str, str]:
    """``(thinking, answer)``.  With ``prompt_opens_think`` the prompt already ended in
    ``<think>`` so the text starts inside the reasoning block."""
    if prompt_opens_think:
        if "</think>" in text:
            t, a = text.split("</think>", 1)
            return t.strip(), a.lstrip("\n")
        return text.strip(), ""
    m = _THINK.search(text)
    if m:
        return m.group(1).strip(), (text[:m.start()] + text[m.end():]).lstrip("\n")
    if text.lstrip().startswith("<think>"):      # unterminated
        return text.lstrip()[len("<think>"):].strip(), ""
    return "", text


def _parse_block(body: str) -> list[ToolCall]:
    calls = []
    fns = _FN.findall(body)
    if not fns:
        m = _FN_OPEN.search(body)                   # truncated: function never closed
        if m and _PARAM.search(m.group(2)):
            fns = [(m.group(1), m.group(2))]
    for name, inner in fns:
        args = {k.strip(): coerce(v) for k, v in _PARAM.findall(inner)}
        calls.append(ToolCall(name.strip(), args, raw=body))
    if calls:
        return calls
    s = body.strip()
    if s.startswith("{"):
        try:
            obj = json.loads(s)
        except ValueError:
            return []
        if isinstance(obj, dict) and isinstance(obj.get("name"), str):
            args = obj.get("arguments", obj.get("parameters", {}))
            if isinstance(args, str):
                try:
                    args = json.loads(args)
                except ValueError:
                    args = {"_raw": args}
            return [ToolCall(obj["name"], args if isinstance(args, dict) else {}, raw=body)]
    return []


def parse_tool_calls(text: str) -> tuple[str, list[ToolCall]]:
    """``(content_without_calls, calls)``; a trailing unterminated ``<tool_call>`` is parsed as
    far as it goes and never leaks into the content."""
    calls: list[ToolCall] = []
    for body in _TC.findall(text):
        calls.extend(_parse_block(body))
    content = _TC.sub("", text)
    i = content.find(TC_OPEN)
    if i >= 0:
        calls.extend(_parse_block(content[i + len(TC_OPEN):]))
        content = content[:i]
    return content.strip(), calls


def tool_result_message(call_id: str, name: str, result: Any) -> dict[str, Any]:
    body = result if isinstance(result, str) else json.dumps(result, ensure_ascii=False)
    return {"role": "tool", "tool_call_id": call_id, "name": name, "content": body}


def render_call(name: str, arguments: dict[str, Any]) -> str:
    """Serialise a call in the native format (used for forced openers and by tests)."""
    lines = [TC_OPEN, f"<function={name}>"]
    for k, v in arguments.items():
        val = v if isinstance(v, str) else json.dumps(v, ensure_ascii=False)
        lines += [f"<parameter={k}>", val, "</parameter>"]
    lines += ["</function>", TC_CLOSE]
    return "\n".join(lines)
