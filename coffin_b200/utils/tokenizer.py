"""Tokenizer access for the serving layer.

``load_tokenizer(model_dir)`` returns the checkpoint's HF tokenizer when its files are present
(``AutoTokenizer``, as the reference does in ``serving/runtime_service.py:41-200``); otherwise a
self-contained ``ByteTokenizer`` (UTF-8 bytes + ChatML control tokens), so that a random-init
model can be served and benchmarked without any tokenizer files.  Both expose ``encode``,
``decode``, ``apply_chat_template`` and ``eos_ids``.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Sequence


class ByteTokenizer:
    """256 byte tokens followed by the ChatML control tokens. ids stay below 512."""

    SPECIAL = ["<|im_start|>", "<|im_end|>", "<|endoftext|>", "<think>", "</think>", "<tool_call>", "</tool_call>",
               "<|vision_start|>", "<|vision_end|>", "<|image_pad|>"]

    def __init__(self, vocab_size: int = 512, image_token_id: int | None = None) -> None:
        self.vocab_size = vocab_size
        self.special = {s: 256 + i for i, s in enumerate(self.SPECIAL)}
        if image_token_id is not None:
            self.special["<|image_pad|>"] = image_token_id
        self.inv = {v: k for k, v in self.special.items()}
        self.eos_token_id = self.special["<|im_end|>"]
        self.name_or_path = "byte-tokenizer"

    @property
    def eos_ids(self) -> tuple[int, ...]:
        return (self.special["<|im_end|>"], self.special["<|endoftext|>"])

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        out: list[int] = []
        i = 0
        while i < len(text):
            if text[i] == "<":
                for s, tid in self.special.items():
                    if text.startswith(s, i):
                        out.append(tid)
                        i += len(s)
                        break
                else:
                    out.extend(text[i].encode("utf-8"))
                    i += 1
            else:
                out.extend(text[i].encode("utf-8"))
                i += 1
        return out

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = False) -> str:
        parts: list[str] = []
        buf = bytearray()
        for t in ids:
            t = int(t)
            if t < 256:
                buf.append(t)
                continue
            if buf:
                parts.append(buf.decode("utf-8", errors="replace"))
                buf = bytearray()
            if t in self.inv:
                if not skip_special_tokens or self.inv[t] in ("<think>", "</think>", "<tool_call>", "</tool_call>"):
                    parts.append(self.inv[t])
            # ids beyond the byte + control range (a model with a larger vocabulary) print nothing
        if buf:
            parts.append(buf.decode("utf-8", errors="replace"))
        return "".join(parts)

    def apply_chat_template(self, messages: list[dict], tools: list[dict] | None = None, tokenize: bool = False,
                            add_generation_prompt: bool = True, enable_thinking: bool = True, **_: Any):
        """ChatML rendering with the Qwen conventions: tools listed in the system turn, tool
        results as ``<tool_response>`` user turns, assistant tool calls in the native format."""
        from .tool_call import render_call
        out = []
        msgs = list(messages)
        sys_text = ""
        if msgs and msgs[0].get("role") == "system":
            sys_text = _text(msgs.pop(0).get("content"))
        if tools:
            sys_text += ("\n\n" if sys_text else "") + "# Tools\n\nYou may call one or more functions.\n<tools>\n" + \
                "\n".join(json.dumps(t, ensure_ascii=False) for t in tools) + "\n</tools>"
        if sys_text:
            out.append(f"<|im_start|>system\n{sys_text}<|im_end|>\n")
        for m in msgs:
            role, content = m.get("role"), _text(m.get("content"))
            if role == "tool":
                out.append(f"<|im_start|>user\n<tool_response>\n{content}\n</tool_response><|im_end|>\n")
                continue
            body = content
            for tc in m.get("tool_calls") or []:
                fn = tc.get("function", tc)
                args = fn.get("arguments", {})
                if isinstance(args, str):
                    try:
                        args = json.loads(args)
                    except ValueError:
                        args = {}
                body += ("\n" if body else "") + render_call(fn.get("name", ""), args)
            out.append(f"<|im_start|>{role}\n{body}<|im_end|>\n")
        if add_generation_prompt:
            out.append("<|im_start|>assistant\n" + ("<think>\n" if enable_thinking else "<think>\n\n</think>\n\n"))
        text = "".join(out)
        return self.encode(text) if tokenize else text


def _text(content) -> str:
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    parts = []
    for p in content:
        if isinstance(p, dict):
            if p.get("type") == "text":
                parts.append(p.get("text", ""))
            elif p.get("type") in ("image", "image_url"):
                parts.append("<|vision_start|><|image_pad|><|vision_end|>")
    return "".join(parts)


class HFTokenizer:
    """Thin adapter so that HF tokenizers and ``ByteTokenizer`` look alike."""

    def __init__(self, tok) -> None:
        self.tok = tok
        self.vocab_size = len(tok)
        self.name_or_path = getattr(tok, "name_or_path", "hf")

    @property
    def eos_ids(self) -> tuple[int, ...]:
        ids = set()
        for name in ("<|im_end|>", "<|endoftext|>"):
            t = self.tok.convert_tokens_to_ids(name)
            if isinstance(t, int) and t >= 0:
                ids.add(t)
        if self.tok.eos_token_id is not None:
            ids.add(int(self.tok.eos_token_id))
        return tuple(sorted(ids))

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        return self.tok.encode(text, add_special_tokens=add_special_tokens)

    def decode(self, ids, skip_special_tokens: bool = False) -> str:
        return self.tok.decode(list(ids), skip_special_tokens=skip_special_tokens)

    def apply_chat_template(self, messages, tools=None, tokenize=False, add_generation_prompt=True,
                            enable_thinking=True, **kw):
        return self.tok.apply_chat_template(messages, tools=tools, tokenize=tokenize,
                                            add_generation_prompt=add_generation_prompt,
                                            enable_thinking=enable_thinking, **kw)


def load_tokenizer(model_dir: str | Path | None, vocab_size: int = 512, image_token_id: int | None = None):
    if model_dir is not None:
        p = Path(model_dir)
        if (p / "tokenizer.json").exists() or (p / "tokenizer_config.json").exists():
            from transformers import AutoTokenizer
            return HFTokenizer(AutoTokenizer.from_pretrained(str(p)))
    return ByteTokenizer(vocab_size, image_token_id)


class IncrementalDecoder:
    """Token-by-token text decoding that never emits half a UTF-8 character: text is released
    only up to the last complete character (the reference streams the same way,
    ``serving/runtime_parts.py:769-869``)."""

    def __init__(self, tok) -> None:
        self.tok = tok
        self.ids: list[int] = []
        self.sent = 0

    def push(self, token: int) -> str:
        self.ids.append(int(token))
        text = self.tok.decode(self.ids, skip_special_tokens=True)
        if text.endswith("�"):
            return ""
        new = text[self.sent:]
        self.sent = len(text)
        return new

    def flush(self) -> str:
        text = self.tok.decode(self.ids, skip_special_tokens=True)
        new = text[self.sent:]
        self.sent = len(text)
        return new
