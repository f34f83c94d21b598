"""Control plane on CPU ranks (gloo, world 2): sampled-token agreement, request fan-out to a
worker, and failure detection when a rank stops beating (made on the host: the rank simply exits)."""
import os
import socket
import time

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _agree(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    from coffin_b200.parallel.control import agree_tokens, init_control_plane, make_fanout
    g = init_control_plane("gloo", timeout_s=30)
    mine = [10 + rank, 20 + rank]           # ranks disagree (as after a numerical divergence)
    q.put((rank, agree_tokens(mine, g)))
    box = [None]
    if rank == 0:
        make_fanout(g)({"op": "ping", "n": 7})
    else:
        dist.broadcast_object_list(box, src=0, group=g)
        q.put(("fanout", box[0]))
    dist.barrier()
    dist.destroy_process_group()


def test_token_agreement_and_fanout():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_agree, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in ps]
    got = [q.get(timeout=60) for _ in range(3)]
    [p.join(timeout=60) for p in ps]
    toks = {k: v for k, v in got if k != "fanout"}
    assert toks[0] == [10, 20] and toks[1] == [10, 20]
    assert dict(got)["fanout"] == {"op": "ping", "n": 7}


def _beat(rank, world, port, q):
    from coffin_b200.parallel.control import Heartbeat
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=__import__("datetime").timedelta(seconds=30))
    hb = Heartbeat(store, rank, world, interval_s=0.05, timeout_s=0.6)
    hb.start()
    if rank == 1:
        time.sleep(0.5)                      # alive for a while, then the rank leaves between steps
        hb.stop()
        q.put(("left", 1))
        time.sleep(3.0)
        return
    time.sleep(0.3)
    q.put(("early", hb.check()))
    deadline = time.monotonic() + 5
    dead = []
    while time.monotonic() < deadline and not dead:
        time.sleep(0.1)
        dead = hb.check()
    q.put(("late", dead))
    hb.stop()


def test_heartbeat_detects_a_rank_that_left():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_beat, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in ps]
    got = dict(q.get(timeout=60) for _ in range(3))
    [p.join(timeout=60) for p in ps]
    assert got["early"] == [] and got["late"] == [1]


def test_server_fails_requests_in_flight_when_a_peer_heartbeat_stops():
    """The failure is made on the host: a fake heartbeat reports rank 1 dead after a few checks; the
    serving loop must fail the running request, launch nothing more and mark itself stopping."""
    import queue

    import torch

    from coffin_b200.config import preset
    from coffin_b200.engine.config import EngineConfig
    from coffin_b200.engine.sequence import SamplingParams
    from coffin_b200.oracle.engine_model import OracleEngineModel
    from coffin_b200.serving.runtime import Server
    from coffin_b200.weights.init import random_state_dict

    class FakeHeartbeat:
        def __init__(self):
            self.n = 0

        def check(self):
            self.n += 1
            return [1] if self.n > 3 else []

    cfg = preset("tiny")
    srv = Server(OracleEngineModel(cfg, random_state_dict(cfg, 0), max_seq=256, num_slots=2),
                 EngineConfig(max_seq=256, max_num_seqs=2, graph=False), model_name="tiny")
    srv.attach_heartbeat(FakeHeartbeat())
    srv.start()
    seq, outq = srv._submit(list(range(5, 25)), SamplingParams(max_tokens=64, ignore_eos=True))
    kinds = []
    while True:
        try:
            kind, val = outq.get(timeout=20)
        except queue.Empty:
            break
        kinds.append(kind)
        if kind in ("error", "done"):
            break
    assert kinds[-1] == "error" and "heartbeat" in val
    assert srv.dead_ranks == [1] and srv.stopping
    steps = srv.model.n_decode_calls
    import time
    time.sleep(0.3)
    assert srv.model.n_decode_calls == steps          # nothing launched after the peer was declared dead
    srv.stop()
