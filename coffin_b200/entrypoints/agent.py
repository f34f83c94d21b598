"""Tool-calling agent loop over the engine socket.

Sends the conversation with a tools array, executes the calls the model makes (built-in demo tools
or a user module with ``execute(name, arguments) -> result``), appends the results as ``tool``
messages and repeats until the model answers in plain text or the round limit is hit.
Reference: ``agent.py:40-135``; demo tools: ``tools_demo.json``.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import sys
from typing import Any, Callable

from ..serving.transport import call
from ..utils.tool_call import tool_result_message

DEMO_TOOLS = [
    {"type": "function", "function": {"name": "get_weather", "description": "Current weather of a city",
                                      "parameters": {"type": "object", "properties": {"city": {"type": "string"}},
                                                     "required": ["city"]}}},
    {"type": "function", "function": {"name": "multiply", "description": "Multiply two numbers",
                                      "parameters": {"type": "object", "properties": {"a": {"type": "number"},
                                                                                      "b": {"type": "number"}},
                                                     "required": ["a", "b"]}}},
]


def builtin(name: str, args: dict[str, Any]) -> Any:
    if name == "get_weather":
        return {"city": args.get("city"), "temperature_c": 21, "condition": "clear"}
    if name == "multiply":
        return {"result": float(args.get("a", 0)) * float(args.get("b", 0))}
    return {"error": f"unknown tool {name!r}"}


def load_executor(path: str | None) -> Callable[[str, dict], Any]:
    if not path:
        return builtin
    spec = importlib.util.spec_from_file_location("agent_tools", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.execute


def run(sock: str, prompt: str, tools: list[dict], execute: Callable[[str, dict], Any], rounds: int = 4,
        max_new: int = 512, system: str = "") -> list[dict]:
    msgs: list[dict] = ([{"role": "system", "content": system}] if system else []) + [{"role": "user", "content": prompt}]
    for _ in range(rounds):
        rep = call(sock, {"op": "chat", "messages": msgs, "tools": tools, "max_new": max_new})
        if not rep.get("ok"):
            raise RuntimeError(rep.get("error"))
        calls = rep.get("tool_calls") or []
        assistant: dict = {"role": "assistant", "content": rep.get("text") or ""}
        if calls:
            assistant["tool_calls"] = [{"id": c["id"], "type": "function",
                                        "function": {"name": c["function"]["name"],
                                                     "arguments": json.loads(c["function"]["arguments"] or "{}")}}
                                       for c in calls]
        msgs.append(assistant)
        if not calls:
            break
        for c in calls:
            args = json.loads(c["function"]["arguments"] or "{}")
            msgs.append(tool_result_message(c["id"], c["function"]["name"], execute(c["function"]["name"], args)))
    return msgs


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("prompt")
    ap.add_argument("--sock", default=os.environ.get("ENGINE_SOCK", "/tmp/coffin_b200.sock"))
    ap.add_argument("--tools", default="")
    ap.add_argument("--executor", default="")
    ap.add_argument("--rounds", type=int, default=4)
    args = ap.parse_args(argv)
    tools = json.load(open(args.tools)) if args.tools else DEMO_TOOLS
    for m in run(args.sock, args.prompt, tools, load_executor(args.executor or None), args.rounds):
        print(json.dumps(m, ensure_ascii=False))
    return 0


if __name__ == "__main__":
    sys.exit(main())
