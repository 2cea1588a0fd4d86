"""Scheduler over the device mock: ids must equal the scheduler-free reference whatever the batching,
speculation, chunking or prefix reuse does (the reference's "batched ids == solo ids" idiom)."""
import random

import pytest

from saber_engine_b200.sched.alloc import GdnStateAllocator, OutOfBlocks, PagedKvAllocator
from saber_engine_b200.sched.buckets import cut_prompt, select_batch, select_rung
from saber_engine_b200.sched.mock import NullExecutor, reference_generation
from saber_engine_b200.sched.prefix_cache import PrefixCache, chain_hashes
from saber_engine_b200.sched.scheduler import Scheduler, SchedulerConfig
from saber_engine_b200.sched.width import WidthByBatch
from saber_engine_b200.serve.engine_api import EngineRefused, EngineRequest, SamplingParams


def _collect(sub, timeout=5.0):
    toks, last = [], None
    while True:
        ev = sub.events.get(timeout=timeout)
        toks += ev.new_token_ids
        last = ev
        if ev.finished:
            return toks, last


def _run(prompts, max_tokens=24, **kw):
    ex = NullExecutor(seed=3, **kw.pop("ex", {}))
    sched = Scheduler(ex, SchedulerConfig(max_seqs=ex.max_seqs, max_ctx=8192, **kw))
    subs = [sched.submit(EngineRequest(p, SamplingParams(max_tokens=max_tokens))) for p in prompts]
    sched.run_until_idle()
    return ex, sched, [_collect(s) for s in subs]


def test_allocators_lowest_index_and_refcounts():
    kv = PagedKvAllocator(8)
    a = kv.allocate(3)
    assert a == [1, 2, 3]                       # block 0 is the null block
    kv.share(a[:2])
    kv.release(a)
    assert kv.free_blocks == 5 and kv.refcount(1) == 1
    assert kv.allocate(1) == [3]
    with pytest.raises(OutOfBlocks):
        kv.allocate(10)
    g = GdnStateAllocator(3)
    assert [g.allocate(), g.allocate()] == [1, 2]
    g.release(1)
    assert g.allocate() == 1


def test_bucket_laws():
    assert select_batch(3) == 3 and select_batch(5) == 8
    assert select_rung(97) == 128 and select_rung(5000) == 2048
    assert cut_prompt(5000, 0) == [(0, 2048), (2048, 2048), (4096, 904)]
    assert cut_prompt(3000, 1024, cuts=[2048, 2992]) == [(1024, 1024), (2048, 944), (2992, 8)]
    ref = WidthByBatch.reference()
    assert ref.width_for(1) == 8 and ref.width_for(3) == 8 and ref.width_for(4) == 5
    assert WidthByBatch.parse("1:3", captured=(1, 5, 9)).width_for(2) == 5      # rounded UP


def test_ids_equal_reference_solo_batched_and_speculative():
    rnd = random.Random(0)
    prompts = [[rnd.randrange(1024) for _ in range(n)] for n in (5, 40, 300, 17, 1000)]
    _, sched, outs = _run(prompts)
    for p, (toks, last) in zip(prompts, outs):
        assert toks == reference_generation(p, 24, 1024)
        assert last.finish_reason == "length"
    st = sched.stats()
    assert st["accepted_tokens"] > 0 and st["kv_free_blocks"] + len(sched.prefix) * 0 <= st["kv_total_blocks"]
    # width 1 (no speculation) gives the same ids
    _, _, outs1 = _run(prompts, width_table=WidthByBatch({1: 1}, (1, 5, 9)))
    assert [o[0] for o in outs1] == [o[0] for o in outs]


def test_leaky_executor_is_caught():
    """Negative control: an executor that commits a rejected draft must change the ids."""
    rnd = random.Random(1)
    prompts = [[rnd.randrange(1024) for _ in range(30)]]
    _, _, outs = _run(prompts, ex=dict(leaky=True, draft_hit_rate=0.5))
    assert outs[0][0] != reference_generation(prompts[0], 24, 1024)


def test_prefix_cache_hit_skips_prefill_and_keeps_ids():
    rnd = random.Random(2)
    shared = [rnd.randrange(1024) for _ in range(2048)]
    p1 = shared + [rnd.randrange(1024) for _ in range(500)]
    p2 = shared + [rnd.randrange(1024) for _ in range(700)]
    ex = NullExecutor(seed=5)
    sched = Scheduler(ex, SchedulerConfig(max_seqs=8, max_ctx=8192))
    s1 = sched.submit(EngineRequest(p1, SamplingParams(max_tokens=8)))
    sched.run_until_idle()
    before = sched.stats()["prompt_tokens"]
    s2 = sched.submit(EngineRequest(p2, SamplingParams(max_tokens=8)))
    sched.run_until_idle()
    t1, _ = _collect(s1)
    t2, last2 = _collect(s2)
    assert t1 == reference_generation(p1, 8, 1024) and t2 == reference_generation(p2, 8, 1024)
    assert last2.cached_tokens == 2048
    assert sched.stats()["prompt_tokens"] - before == len(p2) - 2048
    assert sched.stats()["prefix_hits"] == 1
    # cached pages are shared in place: the second sequence never wrote into them
    assert sched.arenas.kv.free_blocks < sched.arenas.kv.n_blocks - 1
    sched.prefix.clear()
    assert sched.arenas.kv.free_blocks == sched.arenas.kv.n_blocks - 1


def test_prefix_cache_refuses_hash_collision_without_id_equality():
    kv = PagedKvAllocator(64)
    pc = PrefixCache(kv, min_tokens=16, interval=16)
    toks = list(range(64))
    blocks = kv.allocate(4)
    assert pc.insert(toks, 48, blocks, "snap", 10)
    e = pc.lookup(toks)
    assert e is not None and e.n_tokens == 48
    key = chain_hashes(toks[:48], 16)[-1]
    pc._entries[key].tokens = tuple([999] * 48)          # same key, different ids
    assert pc.lookup(toks) is None and pc.stats.refused_hash_collisions == 1


def test_refusals_abort_and_fatal():
    ex = NullExecutor()
    sched = Scheduler(ex, SchedulerConfig(max_seqs=2, max_ctx=128, max_waiting=1))
    with pytest.raises(EngineRefused):
        sched.submit(EngineRequest(list(range(100)), SamplingParams(max_tokens=100)))   # exceeds ctx
    with pytest.raises(EngineRefused):
        sched.submit(EngineRequest([], SamplingParams()))
    a = sched.submit(EngineRequest([1, 2, 3], SamplingParams(max_tokens=50)))
    sched.step()
    sched.abort(a.seq_id)
    sched.run_until_idle()
    _, last = _collect(a)
    assert last.finish_reason == "abort"
    assert sched.arenas.gdn.free_slots == 2
    b = sched.submit(EngineRequest([1, 2, 3], SamplingParams(max_tokens=50)))
    sched.set_fatal("rank 1 died")
    _, lastb = _collect(b)
    assert lastb.finish_reason == "error" and "rank 1" in lastb.error
    with pytest.raises(EngineRefused):
        sched.submit(EngineRequest([1], SamplingParams()))


def test_stop_token_and_eos():
    p = list(range(20))
    ref = reference_generation(p, 30, 1024)
    ex = NullExecutor(seed=9)
    sched = Scheduler(ex, SchedulerConfig(max_seqs=4, max_ctx=4096))
    s = sched.submit(EngineRequest(p, SamplingParams(max_tokens=30, stop_token_ids=(ref[7],))))
    e = sched.submit(EngineRequest(p, SamplingParams(max_tokens=30), eos_token_id=ref[3]))
    sched.run_until_idle()
    ts, ls = _collect(s)
    te, le = _collect(e)
    assert ts == ref[:8] and ls.finish_reason == "stop"
    assert te == ref[:4] and le.finish_reason == "stop"


def test_step_loop_thread_serves_requests():
    ex = NullExecutor(seed=1)
    sched = Scheduler(ex, SchedulerConfig(max_seqs=8, max_ctx=4096))
    sched.spawn_step_loop()
    try:
        subs = [sched.submit(EngineRequest([i, i + 1, i + 2], SamplingParams(max_tokens=12))) for i in range(12)]
        for i, sub in enumerate(subs):
            toks, _ = _collect(sub, timeout=10)
            assert toks == reference_generation([i, i + 1, i + 2], 12, 1024)
    finally:
        sched.shutdown()


def test_prompt_logprobs_refused_at_submit_when_the_engine_cannot_produce_them():
    from saber_engine_b200.sched.mock import NullExecutor
    from saber_engine_b200.sched.scheduler import Scheduler, SchedulerConfig
    from saber_engine_b200.serve.engine_api import EngineRefused, EngineRequest, SamplingParams
    ex = NullExecutor(vocab=300)
    ex.supports_prompt_logprobs = False
    s = Scheduler(ex, SchedulerConfig(max_seqs=2, max_ctx=512))
    import pytest
    with pytest.raises(EngineRefused) as e:
        s.submit(EngineRequest([1, 2, 3], SamplingParams(max_tokens=2, prompt_logprobs=1)))
    assert e.value.status == 400 and s.fatal is None
    s.submit(EngineRequest([1, 2, 3], SamplingParams(max_tokens=2)))
    s.run_until_idle()
