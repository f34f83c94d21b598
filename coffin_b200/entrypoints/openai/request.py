"""OpenAI request -> engine request: message normalisation, image extraction, token budgets,
thinking switch and tool plan.  Pure functions, no I/O.

Reference: ``entrypoints/openai/request.py`` (``_decode_data_url`` l.43-96, ``_split_messages``
l.99-229, ``_norm_messages`` l.302-366, ``_max_tokens`` l.369-394, ``_thinking_flag`` l.397-433,
``_tool_plan`` l.436-494, ``_include_usage`` l.497-508).
"""
from __future__ import annotations

import base64
import binascii
import json
import re
from typing import Any

IMAGE_MIMES = {"image/png", "image/jpeg", "image/jpg", "image/webp", "image/gif", "image/bmp"}
_DATA_URL = re.compile(r"^data:([\w/+.-]+);base64,(.*)$", re.DOTALL)


class RequestError(Exception):
    def __init__(self, message: str, status: int = 400, code: str | None = None) -> None:
        super().__init__(message)
        self.status = status
        self.code = code


def decode_data_url(url: str, max_bytes: int) -> dict:
    """``data:`` URLs only (the engine never fetches from the network)."""
    if not isinstance(url, str) or not url.startswith("data:"):
        raise RequestError("image_url must be a base64 data: URL; remote URLs are not fetched", 400, "invalid_image_url")
    m = _DATA_URL.match(url)
    if not m:
        raise RequestError("malformed data: URL (expected data:<mime>;base64,<payload>)", 400, "invalid_image_url")
    mime, payload = m.group(1).lower(), m.group(2)
    if mime not in IMAGE_MIMES:
        raise RequestError(f"unsupported image type {mime!r}", 400, "unsupported_image_type")
    if len(payload) * 3 // 4 > max_bytes:
        raise RequestError(f"image larger than {max_bytes} bytes", 413, "image_too_large")
    try:
        raw = base64.b64decode(payload, validate=True)
    except (binascii.Error, ValueError):
        raise RequestError("image payload is not valid base64", 400, "invalid_image_url") from None
    if not raw:
        raise RequestError("image payload is empty", 400, "invalid_image_url")
    if len(raw) > max_bytes:
        raise RequestError(f"image larger than {max_bytes} bytes", 413, "image_too_large")
    return {"b64": payload, "mime": mime, "bytes": len(raw)}


def split_messages(messages: list[dict], max_images: int, max_image_bytes: int, max_total_bytes: int
                   ) -> tuple[list[dict], list[dict]]:
    """Pull images out of the content parts.  Returns the messages, and the images in prompt order.  A message
    with at least one image keeps a parts array in which every image is the template's ``{"type": "image"}``
    marker at its place (text and images stay interleaved as the client wrote them); a parts array of text
    only is flattened to the plain string it spells, so a text request reaches the template exactly as it would
    without vision.  User and tool messages may carry images (a screenshot returned by a tool is the common
    case); a system message may not (the chat template rejects it) and an assistant turn may not (the template
    never renders media there), each with a message that says where the image belongs
    (reference: ``entrypoints/openai/request.py:99-229, 232-300``)."""
    out, images, total = [], [], 0
    for m in messages:
        content = m.get("content")
        if not isinstance(content, list):
            out.append(dict(m))
            continue
        role = str(m.get("role") or "user").lower()
        parts, n_img = [], 0
        for p in content:
            if isinstance(p, str):
                parts.append({"type": "text", "text": p})
                continue
            if not isinstance(p, dict):
                raise RequestError(f"content part must be an object, got {type(p).__name__}", 400)
            t = p.get("type")
            if t in (None, "text"):
                parts.append({"type": "text", "text": str(p.get("text") or "")})
            elif t in ("image_url", "image"):
                if role in ("system", "developer"):
                    raise RequestError("a system message cannot contain images: the chat template rejects it; "
                                       "put the image in a user turn", 400)
                if role == "assistant":
                    raise RequestError("an assistant message cannot carry images; put the image in a user or tool message", 400)
                url = p.get("image_url")
                url = url.get("url") if isinstance(url, dict) else url
                if url is None and t == "image":
                    url = p.get("image")
                    url = url.get("url") if isinstance(url, dict) else url
                if url is None:
                    raise RequestError(f"`{t}` part has no `image_url.url`; send "
                                       '{"type": "image_url", "image_url": {"url": "data:image/png;base64,..."}}', 400)
                if len(images) + 1 > max_images:
                    raise RequestError(f"too many images (max {max_images})", 400, "too_many_images")
                img = decode_data_url(url, max_image_bytes)
                total += img["bytes"]
                if total > max_total_bytes:
                    raise RequestError(f"images exceed {max_total_bytes} bytes in total", 413, "images_too_large")
                images.append({"b64": img["b64"], "mime": img["mime"]})
                parts.append({"type": "image"})
                n_img += 1
            elif t in ("video_url", "video", "input_video"):
                raise RequestError("video input is not supported: frame count -> token count is not bounded by this "
                                   "build's image limits", 400, "unsupported_content")
            elif t in ("input_audio", "audio_url"):
                raise RequestError("audio input is not supported by this model", 400, "unsupported_content")
            else:
                raise RequestError(f"unknown content part type {t!r}", 400)
        nm = dict(m)
        nm["content"] = parts if n_img else "".join(x["text"] for x in parts)
        out.append(nm)
    return out, images


def norm_messages(messages: Any) -> list[dict]:
    """developer -> system, function -> tool, tool-call arguments str -> dict, system turns
    merged in front, at least one user turn."""
    if isinstance(messages, str):
        messages = [{"role": "user", "content": messages}]
    if not isinstance(messages, list) or not messages:
        raise RequestError("messages must be a non-empty array", 400)
    out, systems = [], []
    for m in messages:
        if not isinstance(m, dict) or "role" not in m:
            raise RequestError("every message needs a role", 400)
        role = {"developer": "system", "function": "tool"}.get(m["role"], m["role"])
        if role not in ("system", "user", "assistant", "tool"):
            raise RequestError(f"unknown role {m['role']!r}", 400)
        nm = {k: v for k, v in m.items() if k != "role"}
        nm["role"] = role
        if nm.get("content") is None:
            nm["content"] = ""
        calls = nm.get("tool_calls")
        if calls:
            fixed = []
            for c in calls:
                fn = dict(c.get("function") or {})
                args = fn.get("arguments", {})
                if isinstance(args, str):
                    try:
                        args = json.loads(args) if args.strip() else {}
                    except ValueError:
                        args = {"_raw": args}
                fn["arguments"] = args
                fixed.append({**c, "function": fn})
            nm["tool_calls"] = fixed
        if role == "system":
            systems.append(nm)
        else:
            out.append(nm)
    if systems:
        if all(isinstance(s["content"], str) for s in systems):
            merged = {"role": "system", "content": "\n\n".join(s["content"] for s in systems if s["content"])}
        else:
            parts = []
            for s in systems:
                c = s["content"]
                parts.extend(c if isinstance(c, list) else [{"type": "text", "text": c}])
            merged = {"role": "system", "content": parts}
        out.insert(0, merged)
    if not any(m["role"] == "user" for m in out):
        out.append({"role": "user", "content": ""})
    return out


def max_tokens(body: dict, default: int) -> int:
    for key in ("max_completion_tokens", "max_tokens", "max_new_tokens"):
        v = body.get(key)
        if v is not None:
            try:
                n = int(v)
            except (TypeError, ValueError):
                raise RequestError(f"{key} must be an integer", 400) from None
            if n < 1:
                raise RequestError(f"{key} must be >= 1", 400)
            return n
    return default


def thinking_flag(body: dict, default: bool) -> bool:
    kw = body.get("chat_template_kwargs")
    if isinstance(kw, dict) and "enable_thinking" in kw:
        return bool(kw["enable_thinking"])
    for key in ("enable_thinking", "thinking"):
        if key in body:
            v = body[key]
            if isinstance(v, dict):
                return v.get("type", "enabled") != "disabled"
            return bool(v)
    eff = body.get("reasoning_effort")
    if isinstance(eff, str):
        return eff.lower() not in ("none", "off", "minimal")
    return default


def tool_plan(body: dict) -> tuple[list[dict] | None, str | None, bool]:
    """``(tools, forced_prefix, single_call)``.

    ``tool_choice``: ``none`` drops the tools; ``auto`` leaves the model free; ``required`` forces
    the reply to open with ``<tool_call>``; a named function forces ``<tool_call>\\n<function=X>``.
    Legacy ``functions`` / ``function_call`` are mapped onto the same plan.
    """
    tools = body.get("tools")
    if not tools and body.get("functions"):
        tools = [{"type": "function", "function": f} for f in body["functions"]]
    choice = body.get("tool_choice")
    if choice is None and "function_call" in body:
        fc = body["function_call"]
        choice = fc if isinstance(fc, str) else {"type": "function", "function": {"name": fc.get("name")}}
    single = body.get("parallel_tool_calls") is False
    if not tools:
        if isinstance(choice, dict) or choice == "required":
            raise RequestError("tool_choice requires tools", 400)
        return None, None, single
    for t in tools:
        if not isinstance(t, dict) or not isinstance(t.get("function"), dict) or not t["function"].get("name"):
            raise RequestError("every tool needs function.name", 400)
    if choice in (None, "auto"):
        return tools, None, single
    if choice == "none":
        return None, None, single
    if choice == "required":
        return tools, "<tool_call>\n", single
    if isinstance(choice, dict):
        name = (choice.get("function") or {}).get("name") or choice.get("name")
        if not name or name not in {t["function"]["name"] for t in tools}:
            raise RequestError(f"tool_choice names an unknown function {name!r}", 400)
        return tools, f"<tool_call>\n<function={name}>\n", single
    raise RequestError(f"unsupported tool_choice {choice!r}", 400)


def include_usage(body: dict) -> bool:
    so = body.get("stream_options")
    return bool(isinstance(so, dict) and so.get("include_usage"))


def build_engine_request(body: dict, *, default_max_tokens: int, default_thinking: bool, max_decode_seconds: float,
                         max_images: int, max_image_bytes: int, max_image_total_bytes: int, stream: bool) -> tuple[dict, bool]:
    msgs = norm_messages(body.get("messages"))
    msgs, images = split_messages(msgs, max_images, max_image_bytes, max_image_total_bytes)
    tools, prefix, single = tool_plan(body)
    temp = body.get("temperature")
    req = {"op": "chat_stream" if stream else "chat", "messages": msgs, "tools": tools, "tool_prefix": prefix,
           "enable_thinking": thinking_flag(body, default_thinking), "max_new": max_tokens(body, default_max_tokens),
           "temperature": float(temp) if temp is not None else 0.0, "max_seconds": max_decode_seconds}
    if images:
        req["images"] = images
    if body.get("seed") is not None:
        req["seed"] = int(body["seed"])
    return req, single
