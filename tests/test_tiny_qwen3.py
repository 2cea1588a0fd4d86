"""Configuration 1: the tiny Qwen3 decoder on the CPU through the real scheduler and paged KV."""
import time

import torch

from saber_engine_b200.models.tiny_qwen3 import TinyExecutor, TinyQwen3
from saber_engine_b200.runtime.lookup import lookup_draft
from saber_engine_b200.sched.scheduler import Scheduler, SchedulerConfig
from saber_engine_b200.serve.engine_api import EngineRequest, SamplingParams


def _collect(sub):
    toks = []
    while True:
        ev = sub.events.get(timeout=30)
        toks += ev.new_token_ids
        if ev.finished:
            return toks


def test_paged_greedy_decode_matches_cache_free_oracle():
    model = TinyQwen3(seed=0)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, 1024, (64,), generator=g).tolist()
    t0 = time.perf_counter()
    ref = model.greedy_reference(prompt, 32)
    t_ref = time.perf_counter() - t0
    sched = Scheduler(TinyExecutor(model), SchedulerConfig(max_seqs=8, max_ctx=4096, prefix_cache=False))
    t0 = time.perf_counter()
    sub = sched.submit(EngineRequest(prompt, SamplingParams(max_tokens=32)))
    sched.run_until_idle()
    t_eng = time.perf_counter() - t0
    assert _collect(sub) == ref
    assert t_eng < 10 * t_ref + 5       # the paged path is not pathologically slower than the oracle


def test_batched_equals_solo_and_chunked_prefill():
    model = TinyQwen3(seed=3)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (10, 100, 33)]
    refs = [model.greedy_reference(p, 10) for p in prompts]
    sched = Scheduler(TinyExecutor(model), SchedulerConfig(max_seqs=8, max_ctx=4096, prefix_cache=False))
    subs = [sched.submit(EngineRequest(p, SamplingParams(max_tokens=10))) for p in prompts]
    sched.run_until_idle()
    assert [_collect(s) for s in subs] == refs


def test_prompt_lookup_drafter_speculates_without_changing_ids():
    model = TinyQwen3(seed=4)
    prompt = [5, 6, 7, 8, 9, 10] * 8
    ref = model.greedy_reference(prompt, 16)
    ex = TinyExecutor(model, draft_fn=lookup_draft, widths=(1, 5))
    sched = Scheduler(ex, SchedulerConfig(max_seqs=4, max_ctx=4096, prefix_cache=False))
    sub = sched.submit(EngineRequest(prompt, SamplingParams(max_tokens=16)))
    sched.run_until_idle()
    assert _collect(sub) == ref
    assert lookup_draft([1, 2, 3, 4, 1, 2], 3) == [3, 4, 1]
    assert lookup_draft([1, 2, 3], 2) == [0, 0]
