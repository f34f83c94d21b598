"""The engine (scheduler + block manager + radix cache + runner) driven end to end on the CPU
twin of the device model (tiny hybrid config, real logits): batched continuous decoding equals
solo greedy decoding, chunked prefill equals one-shot, prefix hits reuse blocks and snapshots,
preemption recomputes to the same tokens, nothing leaks."""
import pytest
import torch

from coffin_b200.config import preset
from coffin_b200.engine.config import EngineConfig
from coffin_b200.engine.llm_engine import LLMEngine, NO_PROGRESS_LIMIT
from coffin_b200.engine.sequence import SamplingParams
from coffin_b200.oracle.engine_model import OracleEngineModel
from coffin_b200.oracle.model import OracleModel
from coffin_b200.weights.init import random_state_dict

CFG = preset("tiny")
SD = random_state_dict(CFG, 0)


def prompt(n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, CFG.vocab_size, (n,), generator=g).tolist()


def solo(p, n):
    m = OracleModel(CFG, SD)
    with torch.no_grad():
        return m.generate(p, n)[0]


def engine(**kw):
    model_kw = {k: kw.pop(k) for k in ("num_slots", "num_blocks", "max_seq") if k in kw}
    model = OracleEngineModel(CFG, SD, **{"max_seq": 512, "num_slots": 4, **model_kw})
    cfg = EngineConfig(max_seq=512, max_num_seqs=model.num_slots, graph=False, **kw)
    return LLMEngine(model, cfg)


def test_batched_decode_equals_solo_and_no_leak():
    eng = engine(chunk=48, prefill_quantum=48, max_num_batched_tokens=96)
    prompts = [prompt(n, 100 + n) for n in (70, 33, 130)]
    seqs = eng.generate(prompts, SamplingParams(max_tokens=6))
    for p, s in zip(prompts, seqs):
        assert s.output == solo(p, 6)
        assert s.finish_reason == "length"
    eng.bm.radix.clear()
    eng.bm.pool.check()
    assert eng.bm.pool.used_blocks == 0
    assert len(eng.scheduler.free_slots) == 4


def test_prefix_hit_reuses_blocks_and_state():
    eng = engine(snapshot_interval=64)
    shared = prompt(128, 7)
    a = shared + prompt(20, 8)
    b = shared + prompt(31, 9)
    sa = eng.generate([a], SamplingParams(max_tokens=4))[0]
    before = eng.model.n_prefill_calls
    sb = eng.generate([b], SamplingParams(max_tokens=4))[0]
    assert sa.cached_tokens == 0 and sb.cached_tokens == 128
    assert sa.output == solo(a, 4) and sb.output == solo(b, 4)
    assert eng.bm.radix.stats()["tokens_hit"] == 128
    # the same prompt again hits its own tail boundary
    sc = eng.generate([a], SamplingParams(max_tokens=4))[0]
    assert sc.cached_tokens == 128 and sc.output == sa.output
    assert eng.model.n_prefill_calls > before


def test_preemption_recomputes_to_same_tokens():
    # 8 allocatable blocks: three 126-token prompts hold 2 blocks each and each grows into a 3rd
    eng = engine(num_blocks=9, prefix_cache=False, num_slots=3)
    prompts = [prompt(126, 40 + i) for i in range(3)]
    seqs = eng.generate(prompts, SamplingParams(max_tokens=8))
    assert eng.n_preempt >= 1
    for p, s in zip(prompts, seqs):
        assert s.output == solo(p, 8)
    eng.bm.pool.check()
    assert eng.bm.pool.used_blocks == 0


def test_unsatisfiable_pool_raises_instead_of_spinning():
    eng = engine(num_blocks=3, prefix_cache=False, num_slots=2)
    eng.add_request(prompt(200, 1), SamplingParams(max_tokens=2))
    with pytest.raises(RuntimeError, match="no progress"):
        for _ in range(NO_PROGRESS_LIMIT + 5):
            eng.step()


def test_eos_deadline_and_streaming():
    eng = engine()
    p = prompt(40, 3)
    ref = solo(p, 12)
    cut = next((i for i in range(1, 12) if ref[i] not in ref[:i]), None)   # first token not seen before
    if cut is not None:
        s = eng.add_request(p, SamplingParams(max_tokens=12, eos=(ref[cut],)))
        assert list(eng.stream(s)) == ref[:cut] and s.finish_reason == "stop"
    t = eng.add_request(p, SamplingParams(max_tokens=50, deadline=0.0))
    while not t.finished:
        eng.step()
    assert t.finish_reason == "timeout"
    u = eng.add_request(p, SamplingParams(max_tokens=3, temperature=0.8, seed=5))
    v = eng.add_request(p, SamplingParams(max_tokens=3, temperature=0.8, seed=5))
    while not (u.finished and v.finished):
        eng.step()
    assert u.output == v.output


def test_no_head_of_line_blocking_and_reset():
    eng = engine(chunk=32, prefill_quantum=32, max_num_batched_tokens=32)
    long = eng.add_request(prompt(300, 11), SamplingParams(max_tokens=2))
    short = eng.add_request(prompt(20, 12), SamplingParams(max_tokens=2))
    first_done = None
    for _ in range(400):
        eng.step()
        if first_done is None and (long.finished or short.finished):
            first_done = "short" if short.finished else "long"
        if long.finished and short.finished:
            break
    assert long.finished and short.finished
    w = eng.add_request(prompt(50, 13), SamplingParams(max_tokens=100))
    eng.step()
    eng.reset()
    assert w.finished and w.finish_reason == "reset" and not eng.has_work()
    eng.bm.pool.check()
    assert eng.bm.pool.used_blocks == 0


def test_grouped_prefill_shares_forwards_and_matches_solo():
    """A burst of short prompts: their chunks run as groups (one forward for several sequences), cut at
    snapshot boundaries, and every sequence still produces its solo tokens; with grouping off the
    same tokens come out of per-sequence forwards."""
    prompts = [prompt(30 + 17 * i, 60 + i) for i in range(4)]
    ref = [solo(p, 5) for p in prompts]
    eng = engine(chunk=128, prefill_quantum=128, max_num_batched_tokens=256, snapshot_interval=64)
    seqs = eng.generate(prompts, SamplingParams(max_tokens=5))
    assert [s.output for s in seqs] == ref
    assert eng.runner.stats()["prefill_groups"] > 0 and eng.model.n_group_calls > 0
    eng.bm.pool.check()
    off = engine(chunk=128, prefill_quantum=128, max_num_batched_tokens=256, snapshot_interval=64, group_prefill=False)
    assert [s.output for s in off.generate(prompts, SamplingParams(max_tokens=5))] == ref
    assert off.runner.stats()["prefill_groups"] == 0
    # the prefix cache still serves a repeated prompt after a grouped prefill
    again = eng.generate([prompts[3]], SamplingParams(max_tokens=5))[0]
    assert again.output == ref[3] and again.cached_tokens > 0


def test_block_alias_check_catches_a_shared_write_block():
    """The debug check behind ``COFFIN_KV_TRACE``: shared prefix blocks are legal, a block that one
    sequence is about to write and another sequence also references is not."""
    from coffin_b200.engine import debug
    eng = engine(chunk=64, prefill_quantum=64, max_num_batched_tokens=128)
    a = eng.add_request(prompt(100, 21), SamplingParams(max_tokens=4))
    b = eng.add_request(prompt(100, 22), SamplingParams(max_tokens=4))
    for _ in range(3):
        eng.step()
    live = eng.runner.live()
    assert len(live) == 2
    debug.check_block_alias(live, 64, "test")                       # healthy tables
    tb = b.blocks.table
    saved = tb[b.num_computed // 64]
    tb[b.num_computed // 64] = a.blocks.table[a.num_computed // 64]
    with pytest.raises(debug.BlockAliasError):
        debug.check_block_alias(live, 64, "test")
    tb[b.num_computed // 64] = saved
    while not (a.finished and b.finished):
        eng.step()


def test_sparse_verify_option_is_refused_like_in_the_reference():
    import pytest
    from coffin_b200.engine.config import EngineConfig
    from coffin_b200.engine.llm_engine import LLMEngine
    assert EngineConfig().spec_sparse_k == 0
    with pytest.raises(NotImplementedError, match="spec_sparse_k"):
        LLMEngine(object(), EngineConfig(spec_sparse_k=4))


def test_token_budget_bounds_a_step_and_a_sequence_walks_through_its_states():
    from coffin_b200.engine.sequence import SequenceStatus
    eng = engine(chunk=32, prefill_quantum=32, max_num_batched_tokens=64, prefix_cache=False)
    prompts = [prompt(100, 60 + i) for i in range(3)]
    seqs = [eng.add_request(p, SamplingParams(max_tokens=3)) for p in prompts]
    assert all(s.status == SequenceStatus.WAITING for s in seqs)
    seen = {id(s): [s.status] for s in seqs}
    for _ in range(200):
        before = eng.runner.n_prefill_tokens
        eng.step()
        assert eng.runner.n_prefill_tokens - before <= 64           # one step never prefills more than the budget
        for s in seqs:
            if seen[id(s)][-1] != s.status:
                seen[id(s)].append(s.status)
        if all(s.finished for s in seqs):
            break
    for p, s in zip(prompts, seqs):
        assert s.output == solo(p, 3)
        order = [st for st in seen[id(s)] if st != SequenceStatus.PREEMPTED]
        assert order[0] == SequenceStatus.WAITING and order[-1] == SequenceStatus.FINISHED
        assert SequenceStatus.PREFILLING in order and order.index(SequenceStatus.PREFILLING) < len(order) - 1
        if SequenceStatus.RUNNING in order:
            assert order.index(SequenceStatus.PREFILLING) < order.index(SequenceStatus.RUNNING)


def test_one_shot_engine_without_chunking_serves_a_request():
    p = prompt(300, 77)
    for cache, calls in ((False, 1), (True, 2)):      # with the prefix cache the prompt is cut at its last block boundary (a reusable node)
        eng = engine(chunk=512, prefill_quantum=512, max_num_batched_tokens=512, prefix_cache=cache)
        before = eng.model.n_prefill_calls
        s = eng.generate([p], SamplingParams(max_tokens=4))[0]
        assert s.output == solo(p, 4) and eng.model.n_prefill_calls - before == calls


def test_debug_line_reports_the_queues():
    eng = engine(chunk=32, prefill_quantum=32, max_num_batched_tokens=32)
    eng.add_request(prompt(100, 5), SamplingParams(max_tokens=2))
    eng.add_request(prompt(40, 6), SamplingParams(max_tokens=2))
    assert "waiting=2" in eng.debug_line()
    eng.step()
    line = eng.debug_line("prefill")
    assert line.startswith("[step] n=1 kind=prefill") and "free_blocks=" in line and "waiting=2" not in line


def test_shape_and_expansion_traces_print_once_per_shape(capsys):
    from coffin_b200.engine import debug
    debug._shapes_seen.clear()
    assert debug.moe_shape("gate_up", 4096, 128, 1536, 2048, "int4")
    assert not debug.moe_shape("gate_up", 4096, 128, 1536, 2048, "int4")          # seen
    assert debug.moe_shape("down", 4096, 128, 2048, 768, "int4")
    debug.wq_expand((128, 1536, 2048), kept=False)
    said = capsys.readouterr().out
    assert said.count("[moe-shape]") == 2 and "rows=4096 experts=128 n=1536 k=2048 weights=int4" in said
    assert "[wq-expand] (128, 1536, 2048) kept=False" in said and "test_engine_cpu.py" in said


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_arrivals_on_a_tight_pool_match_solo_and_leak_nothing(seed):
    """Requests with random lengths, shared prefixes and token limits arrive at random steps on a pool that forces
    evictions and preemptions; every sequence still produces its solo tokens and every block comes back."""
    import random
    rng = random.Random(seed)
    eng = engine(num_blocks=14, num_slots=3, chunk=64, prefill_quantum=64, max_num_batched_tokens=128, snapshot_interval=64)
    shared = prompt(64 * rng.randint(1, 2), 900 + seed)
    plan = []
    for i in range(7):
        own = prompt(rng.randint(5, 150), 1000 * seed + i)
        p = (shared + own) if rng.random() < 0.5 else own
        plan.append((rng.randint(0, 25), p, rng.randint(1, 6)))
    plan.sort(key=lambda t: t[0])
    live, step = [], 0
    while plan or any(not s.finished for _, s, _ in live):
        while plan and plan[0][0] <= step:
            _, p, n = plan.pop(0)
            live.append((p, eng.add_request(p, SamplingParams(max_tokens=n)), n))
        eng.step()
        eng.bm.pool.check()
        step += 1
        assert step < 3000
    for p, s, n in live:
        assert s.output == solo(p, n), (len(p), n)
    eng.bm.radix.clear()
    eng.bm.pool.check()
    assert eng.bm.pool.used_blocks == 0 and len(eng.scheduler.free_slots) == 3
