"""Scheduler laws over the device mock: mixed prefill + decode steps, the park / step race, the
fatal law for every phase, token-id validation, acceptance-EMA widths, prompt-lookup drafts,
victim parking and the memory valve."""
import threading
import time

import pytest

from saber_engine_b200.sched.mem_valve import MemValve
from saber_engine_b200.sched.mock import NullExecutor, reference_generation
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


def _prompt(n, seed):
    import random
    r = random.Random(seed)
    return [r.randrange(1024) for _ in range(n)]


def test_mixed_steps_keep_decode_moving_while_a_prompt_prefills():
    ex = NullExecutor(seed=1)
    sched = Scheduler(ex, SchedulerConfig(max_seqs=4, max_ctx=16384, mixed_steps=True, mixed_chunk_rows=256,
                                          prefix_cache=False))
    a = sched.submit(EngineRequest(_prompt(40, 1), SamplingParams(max_tokens=64)))
    for _ in range(3):
        sched.step()                      # a is decoding now
    b = sched.submit(EngineRequest(_prompt(3000, 2), SamplingParams(max_tokens=8)))
    before = len(ex.launch_log)
    sched.step()
    kinds = [k for k, _, _ in ex.launch_log[before:]]
    assert kinds == ["prefill", "decode"]            # one step, both phases
    assert ex.launch_log[before][2] <= 256           # the chunk is capped while a stream decodes
    sched.run_until_idle()
    ta, _ = _collect(a)
    tb, _ = _collect(b)
    assert ta == reference_generation(_prompt(40, 1), 64, 1024)
    assert tb == reference_generation(_prompt(3000, 2), 8, 1024)
    assert sched.counters["mixed_steps"] >= 3000 // 256
    # negative control: without mixed steps the same arrival stalls the decoding stream
    ex2 = NullExecutor(seed=1)
    s2 = Scheduler(ex2, SchedulerConfig(max_seqs=4, max_ctx=16384, mixed_steps=False, prefix_cache=False))
    s2.submit(EngineRequest(_prompt(40, 1), SamplingParams(max_tokens=64)))
    for _ in range(3):
        s2.step()
    s2.submit(EngineRequest(_prompt(3000, 2), SamplingParams(max_tokens=8)))
    n0 = len(ex2.launch_log)
    s2.step()
    assert [k for k, _, _ in ex2.launch_log[n0:]] == ["prefill"]


class _SlowDecode(NullExecutor):
    """decode() blocks until released: a step in flight while another thread parks."""
    def __init__(self, **kw):
        super().__init__(**kw)
        self.entered, self.release = threading.Event(), threading.Event()

    def decode(self, runs, width):
        self.entered.set()
        self.release.wait(timeout=5)
        return super().decode(runs, width)


def test_park_from_another_thread_cannot_slip_between_plan_and_launch():
    ex = _SlowDecode(seed=2)
    ex.release.set()
    sched = Scheduler(ex, SchedulerConfig(max_seqs=2, max_ctx=4096, prefix_cache=False))
    sub = sched.submit(EngineRequest(_prompt(30, 3), SamplingParams(max_tokens=40)))
    sched.step()
    sched.step()
    ex.release.clear()
    ex.entered.clear()
    t = threading.Thread(target=sched.step)
    t.start()
    assert ex.entered.wait(timeout=5)               # the step is inside the executor with its plan made
    res = {}
    def park():
        try:
            res["key"] = sched.park(sub.seq_id)
        except Exception as exc:                     # pragma: no cover
            res["exc"] = exc
    pt = threading.Thread(target=park)
    pt.start()
    time.sleep(0.1)
    assert "key" not in res                          # parking waits for the step in flight
    ex.release.set()
    t.join(timeout=5)
    pt.join(timeout=5)
    assert "key" in res and sched.fatal is None
    sched.restore(res["key"])
    sched.run_until_idle()
    toks, last = _collect(sub)
    assert toks == reference_generation(_prompt(30, 3), 40, 1024)


def test_token_ids_outside_the_vocabulary_are_refused():
    ex = NullExecutor(seed=0)
    sched = Scheduler(ex, SchedulerConfig(max_seqs=2, max_ctx=4096))
    for bad in ([1] * 600 + [2 ** 40], [5, -1, 7], [3, 1024], [1, 2.5], [True, 2]):
        with pytest.raises(EngineRefused) as ei:
            sched.submit(EngineRequest(bad, SamplingParams(max_tokens=4)))
        assert ei.value.status == 400
    assert sched.fatal is None
    sub = sched.submit(EngineRequest([1, 2, 3], SamplingParams(max_tokens=4)))
    sched.run_until_idle()
    assert len(_collect(sub)[0]) == 4


class _BadSnapshot(NullExecutor):
    def snapshot_state(self, slot):
        raise RuntimeError("snapshot failed")


def test_an_exception_in_any_phase_ends_in_the_fatal_law():
    ex = _BadSnapshot(seed=0)
    sched = Scheduler(ex, SchedulerConfig(max_seqs=2, max_ctx=8192, prefix_cache=True, prefix_cache_min_tokens=64,
                                          prefix_cache_interval=64))
    sub = sched.submit(EngineRequest(_prompt(600, 4), SamplingParams(max_tokens=4)))
    sched.spawn_step_loop()
    toks, last = _collect(sub)
    assert last.finish_reason == "error" and "snapshot failed" in last.error
    assert sched.fatal and "snapshot failed" in sched.fatal
    with pytest.raises(EngineRefused) as ei:
        sched.submit(EngineRequest([1, 2], SamplingParams(max_tokens=2)))
    assert ei.value.status == 503
    sched.shutdown()


def test_ema_width_policy_narrows_after_rejections_and_ids_stay_right():
    ex = NullExecutor(seed=5, draft_hit_rate=0.0)           # every draft is wrong
    sched = Scheduler(ex, SchedulerConfig(max_seqs=2, max_ctx=4096, width_policy="ema", prefix_cache=False,
                                          width_table=WidthByBatch({1: 8}, captured=(1, 5, 8))))
    sub = sched.submit(EngineRequest(_prompt(20, 6), SamplingParams(max_tokens=40)))
    sched.run_until_idle()
    toks, _ = _collect(sub)
    assert toks == reference_generation(_prompt(20, 6), 40, 1024)
    widths = [rows // n for k, n, rows in ex.launch_log if k == "decode"]
    assert widths[0] == 8 and widths[-1] < 8                # the EMA of accepted drafts fell: narrower steps


def test_lookup_drafts_feed_sequences_without_model_drafts():
    class NoDrafts(NullExecutor):
        def _propose(self, digest, first, k):
            return []
    ex = NoDrafts(seed=7)
    sched = Scheduler(ex, SchedulerConfig(max_seqs=2, max_ctx=4096, lookup_drafts=True, prefix_cache=False))
    sub = sched.submit(EngineRequest(_prompt(24, 8), SamplingParams(max_tokens=20)))
    sched.run_until_idle()
    toks, _ = _collect(sub)
    assert toks == reference_generation(_prompt(24, 8), 20, 1024)      # wrong proposals only cost width
    assert sched.counters["lookup_drafts"] > 0


def test_victim_parking_admits_a_waiting_request_and_restores_the_victim():
    ex = NullExecutor(seed=9, n_kv_blocks=40)                # 39 usable pages of 16 tokens
    sched = Scheduler(ex, SchedulerConfig(max_seqs=4, max_ctx=4096, park_victims=True, prefix_cache=False))
    a = sched.submit(EngineRequest(_prompt(100, 10), SamplingParams(max_tokens=300)))    # ~26 pages
    for _ in range(4):
        sched.step()
    b = sched.submit(EngineRequest(_prompt(100, 11), SamplingParams(max_tokens=200)))    # does not fit beside a
    sched.run_until_idle()
    tb, _ = _collect(b)
    ta, _ = _collect(a)
    assert sched.counters["victims_parked"] == 1 and sched.counters["victims_restored"] == 1
    assert ta == reference_generation(_prompt(100, 10), 300, 1024)
    assert tb == reference_generation(_prompt(100, 11), 200, 1024)


def test_the_step_loop_brings_a_parked_victim_back_when_everything_else_is_done():
    """Served mode: once the request that displaced the victim has finished nothing runs and nothing waits,
    but the parked victim is still work -- the loop must not go to sleep on it."""
    class Slow(NullExecutor):
        def decode(self, runs, width):
            time.sleep(0.002)                              # the second request arrives while the first still decodes
            return super().decode(runs, width)

    ex = Slow(seed=9, n_kv_blocks=40)
    sched = Scheduler(ex, SchedulerConfig(max_seqs=4, max_ctx=4096, park_victims=True, prefix_cache=False))
    sched.spawn_step_loop()
    a = sched.submit(EngineRequest(_prompt(100, 10), SamplingParams(max_tokens=300)))
    while not sched.counters["decode_steps"]:
        time.sleep(0.001)
    b = sched.submit(EngineRequest(_prompt(100, 11), SamplingParams(max_tokens=200)))
    tb, _ = _collect(b)
    ta, _ = _collect(a)                                     # would time out with the victim left in the park tier
    assert ta == reference_generation(_prompt(100, 10), 300, 1024)
    assert tb == reference_generation(_prompt(100, 11), 200, 1024)
    assert sched.counters["victims_restored"] == sched.counters["victims_parked"] >= 1
    sched.shutdown()


def test_memory_valve_demotes_parks_and_refuses():
    avail = {"v": 64 << 30}
    valve = MemValve(reader=lambda: avail["v"])
    ex = NullExecutor(seed=12)
    sched = Scheduler(ex, SchedulerConfig(max_seqs=4, max_ctx=4096, mem_valve=valve, mem_valve_every=1))
    a = sched.submit(EngineRequest(_prompt(30, 13), SamplingParams(max_tokens=400)))
    b = sched.submit(EngineRequest(_prompt(30, 14), SamplingParams(max_tokens=400)))
    for _ in range(4):
        sched.step()
    assert len(sched.running) == 2
    avail["v"] = 6 << 30                                     # below the park threshold
    sched.step()
    sched.step()
    assert sched.valve_level == "park" and sched.counters["victims_parked"] >= 1
    avail["v"] = 1 << 30                                     # below the refuse threshold
    sched.step()
    with pytest.raises(EngineRefused) as ei:
        sched.submit(EngineRequest([1, 2, 3], SamplingParams(max_tokens=2)))
    assert ei.value.status == 503
    avail["v"] = 64 << 30                                    # pressure gone: everything finishes, ids intact
    sched.run_until_idle()
    assert _collect(a)[0] == reference_generation(_prompt(30, 13), 400, 1024)
    assert _collect(b)[0] == reference_generation(_prompt(30, 14), 400, 1024)


def test_requests_sharing_a_prefix_wait_for_the_prompt_that_is_caching_it():
    """Eight prompts with a common 2048-token prefix arrive together: the first prefills, the others
    are admitted once its cut point is in the cache, and each of them hits it."""
    shared = _prompt(2048, 20)
    prompts = [shared + _prompt(1000, 30 + j) for j in range(4)]
    ex = NullExecutor(seed=4)
    sched = Scheduler(ex, SchedulerConfig(max_seqs=4, max_ctx=8192, prefix_cache=True))
    subs = [sched.submit(EngineRequest(p, SamplingParams(max_tokens=6))) for p in prompts]
    sched.run_until_idle()
    for p, sub in zip(prompts, subs):
        toks, last = _collect(sub)
        assert toks == reference_generation(p, 6, 1024)
    st = sched.prefix.stats
    assert st.hits == 3 and st.hit_tokens == 3 * 2048
    assert sched.counters["deferred_for_prefix"] > 0
    # negative control: the same arrival without the law computes the prefix four times
    ex2 = NullExecutor(seed=4)
    s2 = Scheduler(ex2, SchedulerConfig(max_seqs=4, max_ctx=8192, prefix_cache=True, prefix_aware_admission=False))
    subs2 = [s2.submit(EngineRequest(p, SamplingParams(max_tokens=6))) for p in prompts]
    s2.run_until_idle()
    assert s2.prefix.stats.hits == 0
    assert sum(r for k, _, r in ex2.launch_log if k == "prefill") > sum(r for k, _, r in ex.launch_log if k == "prefill")
