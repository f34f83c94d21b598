"""The resident engine process on a real unix socket, with the CPU twin as model: protocol ops,
concurrent streams, failure recovery, diagnostic ops, PD hand-off, and the HTTP adapter on top."""
import http.client
import json
import os
import tempfile
import threading
import time

import pytest
import torch

from coffin_b200.config import preset
from coffin_b200.engine.config import EngineConfig
from coffin_b200.oracle.engine_model import OracleEngineModel
from coffin_b200.oracle.model import OracleModel
from coffin_b200.serving.runtime import Server
from coffin_b200.serving.transport import call, serve, stream
from coffin_b200.weights.init import random_state_dict

CFG = preset("tiny")
SD = random_state_dict(CFG, 0)


@pytest.fixture(scope="module")
def engine():
    builder = lambda: OracleEngineModel(CFG, SD, max_seq=512, num_slots=4)
    srv = Server(builder(), EngineConfig(max_seq=512, max_num_seqs=4, graph=False), model_name="tiny", builder=builder)
    sock = os.path.join(tempfile.mkdtemp(), "engine.sock")
    ready = threading.Event()
    t = threading.Thread(target=serve, args=(srv, sock), kwargs={"ready": ready}, daemon=True)
    t.start()
    assert ready.wait(10)
    yield srv, sock
    call(sock, {"op": "stop"})
    t.join(timeout=10)


def test_ping_tokenize_generate(engine):
    srv, sock = engine
    p = call(sock, {"op": "ping"})
    assert p["ok"] and p["model"] == "tiny" and p["decode_capacity"] == 4 and "prefix" in p and "wall_ms" in p
    toks = call(sock, {"op": "tokenize", "prompt": "héllo<|im_end|>"})["tokens"]
    assert toks[-1] == srv.tok.special["<|im_end|>"] and len(toks) == 7
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, 256, (30,), generator=g).tolist()
    rep = call(sock, {"op": "generate", "tokens": prompt, "max_new": 5, "ignore_eos": True})
    with torch.no_grad():
        ref = OracleModel(CFG, SD).generate(prompt, 5)[0]
    assert rep["ok"] and rep["tokens"] == ref and rep["n_prompt"] == 30 and rep["n_new"] == 5
    assert rep["stopped"] == "length" and rep["prefill_ms"] > 0
    assert call(sock, {"op": "nope"})["ok"] is False


def test_concurrent_chat_streams(engine):
    srv, sock = engine
    results = {}

    def run(i):
        evs = list(stream(sock, {"op": "chat_stream", "messages": [{"role": "user", "content": f"question {i}"}],
                                 "max_new": 6, "ignore_eos": True}))
        results[i] = evs

    ts = [threading.Thread(target=run, args=(i,)) for i in range(5)]
    [t.start() for t in ts]
    [t.join(timeout=120) for t in ts]
    for i in range(5):
        evs = results[i]
        assert evs[0]["type"] == "start" and evs[0]["prompt_opens_think"] is True
        assert evs[-1]["type"] == "done" and evs[-1]["n_new"] == 6 and evs[-1]["ok"]
    assert call(sock, {"op": "ping"})["queue"] == {"waiting": 0, "running": 0}


def test_failure_recovery_keeps_service_up(engine):
    srv, sock = engine
    real = srv.model.decode
    state = {"n": 0}

    def flaky(M, graph=True):
        state["n"] += 1
        if state["n"] == 2:
            raise RuntimeError("injected step failure")
        return real(M, graph)

    srv.model.decode = flaky
    try:
        rep = call(sock, {"op": "generate", "prompt": "abc", "max_new": 8, "ignore_eos": True})
        assert rep["ok"] is False and "injected" in rep["error"]
    finally:
        srv.model.decode = real
    rep = call(sock, {"op": "generate", "prompt": "abc", "max_new": 3, "ignore_eos": True})
    assert rep["ok"] and rep["n_new"] == 3
    assert "injected" in call(sock, {"op": "ping"})["last_error"]


def test_diagnostic_ops_and_pd_handoff(engine):
    srv, sock = engine
    b = call(sock, {"op": "bench", "n": 4, "prompt": "hello world"})
    assert b["ok"] and b["n"] == 4 and b["decode_tok_s"] > 0
    s = call(sock, {"op": "spec", "n": 10, "prompt": "abcabcabcabcabcabc", "spec_k": 3})
    assert s["ok"] and s["exact"] is True and "accept_rate" in s["accept"]
    v = call(sock, {"op": "verify", "c": 2, "n": 2, "prompt": "hello"})
    assert v["ok"] and v["verify_ms"] > 0
    d = tempfile.mkdtemp()
    pf = call(sock, {"op": "pd_prefill", "prompt": "the quick brown fox", "out_dir": d})
    assert pf["ok"] and pf["bytes"] > 0
    plain = call(sock, {"op": "generate", "prompt": "the quick brown fox", "max_new": 5, "ignore_eos": True})
    dec = call(sock, {"op": "pd_decode", "out_dir": d, "max_new": 5})
    assert dec["ok"] and dec["tokens"] == plain["tokens"]
    batch = call(sock, {"op": "pd_decode_batch", "items": [{"dir": d}, {"dir": d}], "max_new": 4})
    assert batch["ok"] and all(it["tokens"] == plain["tokens"][:4] for it in batch["items"])
    # the device transport (one device buffer + CUDA IPC handle) is refused cleanly on the CPU twin
    bad = call(sock, {"op": "pd_prefill", "prompt": "x", "out_dir": d, "transport": "device"})
    assert not bad["ok"] and bad.get("status") == 400 and "CUDA" in bad["error"]
    assert call(sock, {"op": "pd_release"}) == {"ok": True, "released": False} or call(sock, {"op": "pd_release"})["ok"]
    r = call(sock, {"op": "reload"})
    assert r["ok"] and r["n_reload"] == 1
    assert call(sock, {"op": "reset"})["ok"]
    assert call(sock, {"op": "generate", "prompt": "x", "max_new": 2, "ignore_eos": True})["ok"]


def test_diagnostic_ops_refuse_counts_beyond_the_block_table(engine):
    """``n`` / ``c*n`` come from the client and become positions that kernels index tables with: a
    count that does not fit the solo block table or the window is answered with status 400, and the
    model's own guard refuses a position outside a row's block table."""
    srv, sock = engine
    for req in ({"op": "spec", "n": 100000, "prompt": "abc"}, {"op": "verify", "c": 8, "n": 100000, "prompt": "abc"},
                {"op": "bench", "n": 10 ** 7, "prompt": "abc"}, {"op": "verify", "c": 3, "n": 1, "prompt": "abc"}):
        rep = call(sock, req)
        assert rep["ok"] is False and rep.get("status") == 400, rep
    assert call(sock, {"op": "bench", "n": 2, "prompt": "abc"})["ok"]


def test_http_adapter_end_to_end(engine):
    from coffin_b200.entrypoints.openai import app as oa
    from coffin_b200.entrypoints.openai.client import EngineClient
    srv, sock = engine
    oa.configure(oa.ReplicaRouter([EngineClient(sock, 60), EngineClient(sock, 60)]), served_model_name="tiny",
                 default_max_tokens=6)
    http_srv = oa.make_server("127.0.0.1", 0)
    threading.Thread(target=http_srv.serve_forever, daemon=True).start()
    port = http_srv.server_address[1]
    try:
        c = http.client.HTTPConnection("127.0.0.1", port, timeout=60)
        c.request("POST", "/v1/chat/completions", json.dumps({"messages": [{"role": "user", "content": "hi"}],
                                                              "max_tokens": 5, "stream": True}))
        data = c.getresponse().read().decode()
        events = [l[6:] for l in data.split("\n") if l.startswith("data: ")]
        assert events[-1] == "[DONE]"
        last = json.loads(events[-2])
        assert last["choices"][0]["finish_reason"] in ("length", "stop")
        c.request("POST", "/v1/chat/completions", json.dumps({"messages": [{"role": "user", "content": "hi"}],
                                                              "max_tokens": 5}))
        out = json.loads(c.getresponse().read().decode())
        assert out["object"] == "chat.completion" and out["usage"]["completion_tokens"] <= 5
        c.close()
    finally:
        http_srv.shutdown()


def test_serving_load_generator_end_to_end(capsys):
    """The open-loop load generator starts an engine process (tiny model, CPU oracle twin) and the
    HTTP front, drives Poisson arrivals with a shared prefix over SSE and reports percentiles; the
    shared prefix must show up as cached prompt tokens."""
    import json
    from coffin_b200.tools import bench_serving
    rc = bench_serving.main(["--spawn", "--preset", "tiny", "--device", "cpu", "--requests", "6", "--rate", "30",
                             "--prefix-tokens", "64", "--suffix-tokens", "8", "--max-tokens", "6", "--max-seq", "512",
                             "--max-num-seqs", "4", "--startup-timeout", "120"])
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rc == 0 and rep["completed"] == 6 and rep["failed"] == 0
    assert rep["output_tokens_total"] == 36
    assert rep["ttft_ms"]["p50"] is not None and rep["tpot_ms"]["p50"] is not None
    assert rep["cached_prompt_tokens_p50"] >= 32


def test_batched_speculation_is_switched_off_when_memory_is_short(capsys):
    from coffin_b200.engine.config import EngineConfig
    from coffin_b200.serving.runtime import SPEC_BATCH_MIN_FREE, free_bytes, guard_spec_batch
    on = EngineConfig(spec_k=4, spec_batch=True)
    assert guard_spec_batch(on, SPEC_BATCH_MIN_FREE).spec_batch
    assert guard_spec_batch(on, -1).spec_batch                      # no memory figure (CPU twin): left alone
    off = guard_spec_batch(on, SPEC_BATCH_MIN_FREE - 1)
    assert not off.spec_batch and off.spec_k == 4
    assert "spec_batch disabled" in capsys.readouterr().out
    assert free_bytes("cpu") == -1


def test_replies_carry_every_key_of_the_wire_contract(engine):
    """The reply keys of the reference's socket protocol (``serving/runtime_parts.py:925-1133``): clients and the
    HTTP front read them by name."""
    srv, sock = engine
    want = {
        "ping": "ok model model_path arch graph max_seq load_s build_s n_req n_reload backend device native_ops total_ops "
                "int8 vram_gib batch decode_capacity vision vision_int8 image_max_pixels image_min_pixels max_images "
                "n_image_req processor queue prefix wall_ms",
        "generate": "tokens text n_prompt n_new max_new window_full cached_tokens prefill_ms decode_ms decode_tok_s stopped "
                    "spec_k spec wall_ms",
        "chat": "text thinking raw tool_calls forced_tool n_prompt n_new max_new window_full cached_tokens prefill_ms "
                "decode_tok_s stopped spec_k spec n_images image_tokens wall_ms",
    }
    replies = {"ping": call(sock, {"op": "ping"}),
               "generate": call(sock, {"op": "generate", "prompt": "hi", "max_new": 3}),
               "chat": call(sock, {"op": "chat", "messages": [{"role": "user", "content": "hi"}], "max_new": 3})}
    for op, keys in want.items():
        assert replies[op].get("ok", True), replies[op]
        assert [k for k in keys.split() if k not in replies[op]] == [], op
    assert set(replies["ping"]["queue"]) >= {"waiting", "running"}
    lines = list(stream(sock, {"op": "chat_stream", "messages": [{"role": "user", "content": "hi"}], "max_new": 3}))
    assert lines[0]["type"] == "start" and {"n_prompt", "prompt_opens_think", "forced_tool"} <= set(lines[0])
    assert lines[-1]["type"] == "done" and {"text", "n_new", "cached_tokens", "prefill_ms"} <= set(lines[-1])
    assert all(ln["type"] == "token" and "text" in ln for ln in lines[1:-1])


def test_client_that_disconnects_mid_stream_frees_its_sequence(engine):
    """A stream client reads the first lines and closes the socket: the engine aborts the sequence (slot and
    blocks come back) and keeps serving."""
    import socket
    srv, sock = engine
    c = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    c.connect(sock)
    c.sendall((json.dumps({"op": "chat_stream", "messages": [{"role": "user", "content": "count slowly"}],
                           "max_new": 400}) + "\n").encode())
    f = c.makefile("r")
    assert json.loads(f.readline())["type"] == "start"
    before = srv.engine.runner.n_decode_steps
    f.close()
    c.close()
    deadline = time.time() + 20
    while time.time() < deadline:
        q = call(sock, {"op": "ping"})["queue"]
        if q["running"] == 0 and q["waiting"] == 0:
            break
        time.sleep(0.05)
    assert q["running"] == 0 and q["waiting"] == 0
    assert len(srv.engine.scheduler.free_slots) == 4
    assert srv.engine.runner.n_decode_steps - before < 300          # cut short, not decoded to the limit
    rep = call(sock, {"op": "generate", "prompt": "still there?", "max_new": 3})
    assert rep["ok"] and rep["n_new"] == 3


def test_peer_closed_probe_tells_silence_from_a_closed_connection():
    import socket
    from coffin_b200.serving.transport import _peer_closed
    a, b = socket.socketpair(socket.AF_UNIX, socket.SOCK_STREAM)
    try:
        assert _peer_closed(a) is False                 # open and silent
        b.sendall(b"x")
        assert _peer_closed(a) is False                 # data waiting is not a close (and is not consumed)
        assert a.recv(1) == b"x"
        b.close()
        assert _peer_closed(a) is True
    finally:
        a.close()
    assert _peer_closed(a) is True                      # a dead descriptor reads as gone, not as an exception
