"""Scheduler + HybridExecutor on the GPU: requests through the public Engine API."""
import pytest
import torch

from saber_engine_b200.models import config as C
from saber_engine_b200.models.hybrid import HybridModel
from saber_engine_b200.runtime.hybrid_executor import HybridExecutor
from saber_engine_b200.sched.scheduler import Scheduler, SchedulerConfig
from saber_engine_b200.sched.width import WidthByBatch
from saber_engine_b200.serve.engine_api import EngineRequest, SamplingParams

pytestmark = pytest.mark.gpu


def _collect(sub):
    toks, last = [], None
    while True:
        ev = sub.events.get(timeout=60)
        toks += ev.new_token_ids
        last = ev
        if ev.finished:
            return toks, last


@pytest.fixture(scope="module")
def executor():
    cfg = C.scaled_hybrid()
    model = HybridModel(cfg, device="cuda", max_seqs=4, max_ctx=2048, max_width=5, seed=1)
    return HybridExecutor(model, decode_batches=(1, 2, 4), decode_widths=(1, 5), prefill_rungs=(64, 256))


def _sched(executor, **kw):
    return Scheduler(executor, SchedulerConfig(max_seqs=4, max_ctx=2048, prefix_cache_min_tokens=64,
                                               prefix_cache_interval=128, **kw))


def test_concurrent_requests_equal_solo_and_spec_equals_plain(executor):
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, executor.vocab, (n,), generator=g).tolist() for n in (20, 70, 300)]
    solo = []
    for p in prompts:
        s = _sched(executor, prefix_cache=False, width_table=WidthByBatch({1: 1}, (1, 5)))
        sub = s.submit(EngineRequest(p, SamplingParams(max_tokens=16)))
        s.run_until_idle()
        solo.append(_collect(sub)[0])
    s = _sched(executor, prefix_cache=False)
    subs = [s.submit(EngineRequest(p, SamplingParams(max_tokens=16))) for p in prompts]
    s.run_until_idle()
    got = [_collect(x)[0] for x in subs]
    assert got == solo
    assert s.stats()["decode_steps"] > 0 and executor.census["graph_replays"] > 0


def test_prefix_cache_reuse_keeps_ids(executor):
    g = torch.Generator().manual_seed(1)
    shared = torch.randint(0, executor.vocab, (256,), generator=g).tolist()
    p1 = shared + torch.randint(0, executor.vocab, (40,), generator=g).tolist()
    p2 = shared + torch.randint(0, executor.vocab, (55,), generator=g).tolist()
    cold = []
    for p in (p1, p2):
        s = _sched(executor, prefix_cache=False)
        sub = s.submit(EngineRequest(p, SamplingParams(max_tokens=12)))
        s.run_until_idle()
        cold.append(_collect(sub)[0])
    s = _sched(executor)
    a = s.submit(EngineRequest(p1, SamplingParams(max_tokens=12)))
    s.run_until_idle()
    b = s.submit(EngineRequest(p2, SamplingParams(max_tokens=12)))
    s.run_until_idle()
    ta, _ = _collect(a)
    tb, lb = _collect(b)
    assert [ta, tb] == cold
    assert lb.cached_tokens == 256


def test_park_and_restore_on_the_device_resumes_with_the_same_ids(executor, tmp_path):
    from saber_engine_b200.sched.park import ParkTier
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, executor.vocab, (90,), generator=g).tolist()
    s = _sched(executor, prefix_cache=False)
    sub = s.submit(EngineRequest(prompt, SamplingParams(max_tokens=40, ignore_eos=True)))
    s.run_until_idle()
    want = _collect(sub)[0]
    s = _sched(executor, prefix_cache=False)
    s.park_tier = ParkTier(ram_budget=1, directory=str(tmp_path))
    sub = s.submit(EngineRequest(prompt, SamplingParams(max_tokens=40, ignore_eos=True)))
    for _ in range(5):
        s.step()
    key = s.park(sub.seq_id)
    # another request takes the slot and overwrites pages while the first one is away
    other = s.submit(EngineRequest(prompt[::-1], SamplingParams(max_tokens=12, ignore_eos=True)))
    s.run_until_idle()
    assert _collect(other)[1].finished
    s.restore(key)
    s.run_until_idle()
    assert _collect(sub)[0] == want
