"""OpenAI adapter wire format against a fake engine that speaks the real line protocol with
canned replies (no model): health/models, finish reasons, SSE framing, reasoning split,
tool-call parsing and non-leak, fragment accumulation == non-stream arguments, tool_choice
variants, legacy functions, parallel_tool_calls, include_usage, image parts and budgets."""
import base64
import http.client
import json
import os
import socket
import tempfile
import threading

import pytest

from coffin_b200.entrypoints.openai import app as oa
from coffin_b200.entrypoints.openai.client import EngineClient
from coffin_b200.utils.tool_call import parse_tool_calls, split_thinking

CALL = ("<tool_call>\n<function=get_weather>\n<parameter=city>\nBeijing\n</parameter>\n<parameter=days>\n3\n"
        "</parameter>\n</function>\n</tool_call>")
TWO = CALL + "\n<tool_call>\n<function=multiply>\n<parameter=a>\n2\n</parameter>\n<parameter=b>\n4.5\n</parameter>\n</function>\n</tool_call>"


class FakeEngine:
    """Unix-socket engine double: the reply text is chosen by the last user message."""

    def __init__(self):
        self.path = os.path.join(tempfile.mkdtemp(), "fake.sock")
        self.requests = []
        self.lst = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        self.lst.bind(self.path)
        self.lst.listen(16)
        self.alive = True
        threading.Thread(target=self._loop, daemon=True).start()

    def _script(self, req):
        last = ""
        for m in req.get("messages", []):
            if m["role"] == "user":
                c = m["content"]
                last = c if isinstance(c, str) else "".join(p.get("text", "") for p in c if p.get("type") == "text")
        forced = req.get("tool_prefix") or ""
        if forced:
            body = CALL[len(forced):] if CALL.startswith(forced) else CALL[len("<tool_call>\n"):]
            return forced, body, False
        if last == "tool":
            return "", "plan it</think>\n\nLet me check.\n" + CALL, True
        if last == "two":
            return "", "</think>\n\n" + TWO, True
        if last == "long":
            return "", "</think>\n\n" + "word " * 8, True
        if last == "err":
            return None, None, None
        return "", "thinking hard</think>\n\nHello there!", True

    def _reply(self, req, raw, forced, opens, n_max):
        full = (forced or "") + raw
        thinking, answer = split_thinking(full, prompt_opens_think=opens and not forced)
        content, calls = parse_tool_calls(answer)
        n_new = len(raw.split())
        return {"ok": True, "text": content, "thinking": thinking, "raw": raw,
                "tool_calls": [c.to_openai_dict() for c in calls], "forced_tool": forced or None,
                "n_prompt": 11, "n_new": min(n_new, n_max), "max_new": n_max, "cached_tokens": 4,
                "stopped": "stop", "n_images": len(req.get("images") or [])}

    def _loop(self):
        while self.alive:
            try:
                conn, _ = self.lst.accept()
            except OSError:
                return
            threading.Thread(target=self._serve, args=(conn,), daemon=True).start()

    def _serve(self, conn):
        with conn, conn.makefile("rwb") as fh:
            req = json.loads(fh.readline().decode())
            self.requests.append(req)
            op = req.get("op")
            send = lambda o: (fh.write((json.dumps(o) + "\n").encode()), fh.flush())
            if op == "ping":
                send({"ok": True, "model": "fake", "backend": "fake", "queue": {"waiting": 0, "running": 0}})
                return
            forced, raw, opens = self._script(req)
            n_max = int(req.get("max_new", 100))
            if forced is None:
                if op == "chat_stream":
                    send({"type": "error", "error": "image too large", "status": 413})
                else:
                    send({"ok": False, "error": "image too large", "status": 413})
                return
            if op == "chat":
                send(self._reply(req, raw, forced, opens, n_max))
                return
            send({"type": "start", "n_prompt": 11, "prompt_opens_think": opens, "forced_tool": forced or None})
            for i in range(0, len(raw), 5):         # five characters per "token" splits every marker
                send({"type": "token", "text": raw[i:i + 5]})
            done = self._reply(req, raw, forced, opens, n_max)
            done["type"] = "done"
            send(done)


@pytest.fixture(scope="module")
def server():
    eng = FakeEngine()
    oa.configure(oa.ReplicaRouter([EngineClient(eng.path, 10)]), served_model_name="fake-model",
                 default_max_tokens=64, max_images=2, max_image_bytes=2000, max_image_total_bytes=3000)
    srv = oa.make_server("127.0.0.1", 0)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    yield eng, srv.server_address[1]
    srv.shutdown()
    eng.alive = False
    eng.lst.close()


def post(port, body):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=10)
    c.request("POST", "/v1/chat/completions", json.dumps(body), {"Content-Type": "application/json"})
    r = c.getresponse()
    data = r.read().decode()
    c.close()
    return r.status, data


def get(port, path):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=10)
    c.request("GET", path)
    r = c.getresponse()
    data = json.loads(r.read().decode())
    c.close()
    return r.status, data


def sse(data):
    events = [l[6:] for l in data.split("\n") if l.startswith("data: ")]
    assert events[-1] == "[DONE]"
    return [json.loads(e) for e in events[:-1]]


def user(text):
    return [{"role": "user", "content": text}]


TOOLS = [{"type": "function", "function": {"name": "get_weather", "parameters": {}}},
         {"type": "function", "function": {"name": "multiply", "parameters": {}}}]


def test_health_models_and_404(server):
    _, port = server
    st, h = get(port, "/health")
    assert st == 200 and h["status"] == "ok" and h["served_model_name"] == "fake-model"
    st, m = get(port, "/v1/models")
    assert m["data"][0]["id"] == "fake-model"
    assert get(port, "/nope")[0] == 404


def test_plain_completion_and_usage(server):
    _, port = server
    st, data = post(port, {"messages": user("hi")})
    out = json.loads(data)
    msg = out["choices"][0]["message"]
    assert st == 200 and msg["content"] == "Hello there!" and msg["reasoning_content"] == "thinking hard"
    assert out["choices"][0]["finish_reason"] == "stop"
    assert out["usage"]["prompt_tokens_details"]["cached_tokens"] == 4
    st, data = post(port, {"messages": user("long"), "max_tokens": 8})
    assert json.loads(data)["choices"][0]["finish_reason"] == "length"


def test_tool_calls_non_stream_and_stream_agree(server):
    _, port = server
    st, data = post(port, {"messages": user("tool"), "tools": TOOLS})
    choice = json.loads(data)["choices"][0]
    assert choice["finish_reason"] == "tool_calls"
    call = choice["message"]["tool_calls"][0]
    assert call["function"]["name"] == "get_weather"
    assert json.loads(call["function"]["arguments"]) == {"city": "Beijing", "days": 3}
    assert "<tool_call>" not in (choice["message"]["content"] or "")
    st, data = post(port, {"messages": user("tool"), "tools": TOOLS, "stream": True,
                           "stream_options": {"include_usage": True}})
    chunks = sse(data)
    assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
    content = "".join(c["choices"][0]["delta"].get("content") or "" for c in chunks if c["choices"])
    reasoning = "".join(c["choices"][0]["delta"].get("reasoning_content") or "" for c in chunks if c["choices"])
    frags = [d for c in chunks if c["choices"] for d in c["choices"][0]["delta"].get("tool_calls", [])]
    assert content.strip() == "Let me check." and reasoning == "plan it"
    assert "<tool" not in content and "<think" not in content
    assert frags[0]["function"]["name"] == "get_weather" and frags[0]["id"].startswith("call_")
    args = "".join(f["function"].get("arguments", "") for f in frags)
    assert args == call["function"]["arguments"]
    finishes = [c["choices"][0]["finish_reason"] for c in chunks if c["choices"]]
    assert finishes[-1] == "tool_calls"
    assert chunks[-1]["choices"] == [] and chunks[-1]["usage"]["completion_tokens"] > 0


def test_parallel_tool_calls_and_tool_choice(server):
    eng, port = server
    out = json.loads(post(port, {"messages": user("two"), "tools": TOOLS})[1])
    assert [c["function"]["name"] for c in out["choices"][0]["message"]["tool_calls"]] == ["get_weather", "multiply"]
    out = json.loads(post(port, {"messages": user("two"), "tools": TOOLS, "parallel_tool_calls": False})[1])
    assert len(out["choices"][0]["message"]["tool_calls"]) == 1
    chunks = sse(post(port, {"messages": user("two"), "tools": TOOLS, "stream": True})[1])
    idx = {d["index"] for c in chunks if c["choices"] for d in c["choices"][0]["delta"].get("tool_calls", [])}
    assert idx == {0, 1}
    post(port, {"messages": user("hi"), "tools": TOOLS, "tool_choice": "none"})
    assert eng.requests[-1]["tools"] is None
    post(port, {"messages": user("hi"), "tools": TOOLS, "tool_choice": "required"})
    assert eng.requests[-1]["tool_prefix"] == "<tool_call>\n"
    out = json.loads(post(port, {"messages": user("hi"), "tools": TOOLS,
                                 "tool_choice": {"type": "function", "function": {"name": "get_weather"}}})[1])
    assert eng.requests[-1]["tool_prefix"] == "<tool_call>\n<function=get_weather>\n"
    assert out["choices"][0]["message"]["tool_calls"][0]["function"]["name"] == "get_weather"
    post(port, {"messages": user("hi"), "functions": [{"name": "multiply"}], "function_call": {"name": "multiply"}})
    assert eng.requests[-1]["tool_prefix"] == "<tool_call>\n<function=multiply>\n"
    assert post(port, {"messages": user("hi"), "tool_choice": "required"})[0] == 400
    assert post(port, {"messages": user("hi"), "tools": TOOLS, "tool_choice": {"function": {"name": "zzz"}}})[0] == 400


def test_request_normalisation(server):
    eng, port = server
    post(port, {"messages": [{"role": "developer", "content": "be brief"}, {"role": "user", "content": "hi"},
                             {"role": "assistant", "content": None,
                              "tool_calls": [{"id": "c1", "type": "function",
                                              "function": {"name": "multiply", "arguments": "{\"a\": 2}"}}]},
                             {"role": "function", "name": "multiply", "content": "4"}],
                "max_completion_tokens": 7, "enable_thinking": False, "temperature": 0.5})
    r = eng.requests[-1]
    assert r["messages"][0] == {"role": "system", "content": "be brief"}
    assert r["messages"][2]["tool_calls"][0]["function"]["arguments"] == {"a": 2}
    assert r["messages"][3]["role"] == "tool"
    assert r["max_new"] == 7 and r["enable_thinking"] is False and r["temperature"] == 0.5
    assert post(port, {"messages": []})[0] == 400
    assert post(port, {"messages": user("hi"), "max_tokens": 0})[0] == 400
    st, data = post(port, {"messages": "just text"})
    assert st == 200


def test_images(server):
    eng, port = server
    png = base64.b64encode(b"\x89PNG" + b"0" * 100).decode()
    img = {"type": "image_url", "image_url": {"url": f"data:image/png;base64,{png}"}}
    st, _ = post(port, {"messages": [{"role": "user", "content": [{"type": "text", "text": "hi"}, img]}]})
    assert st == 200 and eng.requests[-1]["images"][0]["mime"] == "image/png"
    assert eng.requests[-1]["messages"][0]["content"][1] == {"type": "image"}
    bad = {"type": "image_url", "image_url": {"url": "http://example.com/a.png"}}
    assert post(port, {"messages": [{"role": "user", "content": [bad]}]})[0] == 400
    assert post(port, {"messages": [{"role": "user", "content": [{"type": "video_url", "video_url": {}}]}]})[0] == 400
    assert post(port, {"messages": [{"role": "assistant", "content": [img]}, {"role": "user", "content": "x"}]})[0] == 400
    assert post(port, {"messages": [{"role": "user", "content": [img, img, img]}]})[0] == 400
    big = base64.b64encode(b"1" * 2500).decode()
    bigimg = {"type": "image_url", "image_url": {"url": f"data:image/png;base64,{big}"}}
    assert post(port, {"messages": [{"role": "user", "content": [bigimg]}]})[0] == 413
    mid = base64.b64encode(b"1" * 1800).decode()
    midimg = {"type": "image_url", "image_url": {"url": f"data:image/png;base64,{mid}"}}
    assert post(port, {"messages": [{"role": "user", "content": [midimg, midimg]}]})[0] == 413
    # engine-side refusals keep their status on both paths
    assert post(port, {"messages": user("err")})[0] == 413
    assert post(port, {"messages": user("err"), "stream": True})[0] == 413


def test_cut_off_reasoning_is_not_passed_off_as_the_answer(server):
    """A reply that ends inside the thinking block (token limit) has reasoning but no answer: the text must not
    move into ``content``, and the finish reason says the budget ran out."""
    eng, port = server
    eng_script = eng._script
    eng._script = lambda req: ("", "still thinking about it and never closing", True)
    try:
        st, data = post(port, {"messages": user("hi"), "max_tokens": 7})
        out = json.loads(data)
        msg = out["choices"][0]["message"]
        assert st == 200 and not (msg.get("content") or "").strip()
        assert "still thinking" in (msg.get("reasoning_content") or "")
        assert out["choices"][0]["finish_reason"] == "length"
        chunks = sse(post(port, {"messages": user("hi"), "max_tokens": 7, "stream": True})[1])
        content = "".join(c["choices"][0]["delta"].get("content") or "" for c in chunks if c["choices"])
        reasoning = "".join(c["choices"][0]["delta"].get("reasoning_content") or "" for c in chunks if c["choices"])
        assert not content.strip() and "still thinking" in reasoning
    finally:
        eng._script = eng_script


def test_split_tool_marker_is_held_back_in_the_stream(server):
    """Five-character engine tokens cut ``<tool_call>`` in two: no content delta may carry a piece of the marker
    or of the call body, and the accumulated argument fragments parse to the non-stream arguments."""
    eng, port = server
    chunks = sse(post(port, {"messages": user("tool"), "tools": TOOLS, "stream": True})[1])
    content = "".join(c["choices"][0]["delta"].get("content") or "" for c in chunks if c["choices"])
    assert "<tool" not in content and "function=" not in content and "parameter" not in content
    frags, name = "", None
    for c in chunks:
        for ch in c["choices"]:
            for tc in ch["delta"].get("tool_calls") or []:
                name = tc["function"].get("name") or name
                frags += tc["function"].get("arguments") or ""
    assert name == "get_weather"
    whole = json.loads(post(port, {"messages": user("tool"), "tools": TOOLS})[1])["choices"][0]["message"]["tool_calls"][0]
    assert json.loads(frags) == json.loads(whole["function"]["arguments"]) == {"city": "Beijing", "days": 3}


def test_image_roles_order_and_plain_parts(server):
    eng, port = server

    def img(tag: bytes):
        return {"type": "image_url", "image_url": {"url": "data:image/png;base64," + base64.b64encode(b"\x89PNG" + tag * 20).decode()}}

    a, b = img(b"a"), img(b"b")
    # a parts array of text only flattens to a string, as without vision
    st, _ = post(port, {"messages": [{"role": "user", "content": [{"type": "text", "text": "hel"}, {"type": "text", "text": "lo"}]}]})
    assert st == 200 and eng.requests[-1]["messages"][0]["content"] == "hello" and not eng.requests[-1].get("images")
    # two images keep their order, the template sees one marker per image at its place
    st, _ = post(port, {"messages": [{"role": "user", "content": [a, {"type": "text", "text": "vs"}, b]}]})
    r = eng.requests[-1]
    assert st == 200 and [p["type"] for p in r["messages"][0]["content"]] == ["image", "text", "image"]
    assert [base64.b64decode(i["b64"])[4:5] for i in r["images"]] == [b"a", b"b"]
    # roles: a tool result may carry an image, a system or assistant message may not
    st, _ = post(port, {"messages": [{"role": "user", "content": "look"},
                                     {"role": "assistant", "content": None, "tool_calls": [{"id": "c", "type": "function", "function": {"name": "multiply", "arguments": "{}"}}]},
                                     {"role": "tool", "tool_call_id": "c", "content": [a]}]})
    assert st == 200 and len(eng.requests[-1]["images"]) == 1
    st, data = post(port, {"messages": [{"role": "system", "content": [a]}, {"role": "user", "content": "x"}]})
    assert st == 400 and "user" in json.loads(data)["error"]["message"]
    # malformed payloads are 400 with a readable message
    bad64 = {"type": "image_url", "image_url": {"url": "data:image/png;base64,@@@not-base64@@@"}}
    st, data = post(port, {"messages": [{"role": "user", "content": [bad64]}]})
    assert st == 400 and json.loads(data)["error"]["message"]
    tiff = {"type": "image_url", "image_url": {"url": "data:image/tiff;base64," + base64.b64encode(b"II*\x00").decode()}}
    assert post(port, {"messages": [{"role": "user", "content": [tiff]}]})[0] == 400


def test_malformed_image_urls_are_400_and_a_front_without_vision_answers_503(server):
    eng, port = server
    png = base64.b64encode(b"\x89PNG" + b"0" * 100).decode()
    cases = {"bad base64": "data:image/png;base64,!!!notbase64!!!", "no payload": "data:image/png;base64,",
             "not a url": "not-a-url", "svg": "data:image/svg+xml;base64," + png}
    n = len(eng.requests)
    for label, url in cases.items():
        st, body = post(port, {"messages": [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": url}}]}]})
        assert st == 400 and json.loads(body)["error"]["message"], label
    assert len(eng.requests) == n                                  # nothing malformed reached the engine
    img = {"type": "image_url", "image_url": {"url": f"data:image/png;base64,{png}"}}
    oa.STATE["vision"] = False
    try:
        st, body = post(port, {"messages": [{"role": "user", "content": [img]}]})
        assert st == 503 and "--no-vision" in json.loads(body)["error"]["message"] and len(eng.requests) == n
        st, body = post(port, {"messages": user("hi"), "max_tokens": 3})    # the text path is untouched
        assert st == 200
    finally:
        oa.STATE["vision"] = True
    assert post(port, {"messages": [{"role": "user", "content": [img]}]})[0] == 200


def test_request_field_spellings():
    """Every accepted spelling of the token limit, the thinking switch and the legacy function fields
    (reference ``entrypoints/openai/request.py:369-508``)."""
    from coffin_b200.entrypoints.openai.request import RequestError, include_usage, max_tokens, thinking_flag, tool_plan
    assert max_tokens({"max_completion_tokens": 5, "max_tokens": 9}, 64) == 5
    assert max_tokens({"max_tokens": 9, "max_new_tokens": 3}, 64) == 9
    assert max_tokens({"max_new_tokens": "3"}, 64) == 3 and max_tokens({}, 64) == 64
    for bad in ({"max_tokens": "x"}, {"max_tokens": 0}, {"max_new_tokens": -1}):
        with pytest.raises(RequestError):
            max_tokens(bad, 64)
    assert thinking_flag({}, True) is True and thinking_flag({}, False) is False
    assert thinking_flag({"enable_thinking": False}, True) is False
    assert thinking_flag({"thinking": {"type": "disabled"}}, True) is False
    assert thinking_flag({"thinking": {"type": "enabled"}}, False) is True
    assert thinking_flag({"reasoning_effort": "none"}, True) is False and thinking_flag({"reasoning_effort": "high"}, False) is True
    # the template argument wins over the top-level switch
    assert thinking_flag({"chat_template_kwargs": {"enable_thinking": False}, "enable_thinking": True}, True) is False
    fn = {"name": "get_weather", "parameters": {}}
    tools, forced, single = tool_plan({"functions": [fn], "function_call": {"name": "get_weather"}})
    assert tools == [{"type": "function", "function": fn}] and forced == "<tool_call>\n<function=get_weather>\n" and not single
    assert tool_plan({"functions": [fn], "function_call": "none"})[0] is None
    assert tool_plan({"tools": TOOLS, "tool_choice": "required", "parallel_tool_calls": False})[1:] == ("<tool_call>\n", True)
    for bad in ({"tool_choice": "required"}, {"tools": TOOLS, "tool_choice": {"type": "function", "function": {"name": "nope"}}},
                {"tools": [{"type": "function", "function": {}}]}, {"tools": TOOLS, "tool_choice": "sometimes"}):
        with pytest.raises(RequestError):
            tool_plan(bad)
    assert include_usage({"stream_options": {"include_usage": True}}) and not include_usage({"stream_options": None})
