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
    # gdn_prefill="rows": the laws below compare token ids of the same prompt prefilled in different pieces
    # (cold, resumed from a cached prefix, restored from a park).  The row-by-row recurrence is the same fp32
    # arithmetic however the rows are cut; the tensor-core chunked default rounds the state copy that feeds a
    # chunk's products to bf16, so a cut inside a 64-row chunk moves the last bits (cuts at chunk boundaries do
    # not: tests/test_kernels_gpu.py), and a random-init model turns last bits into other tokens.
    model = HybridModel(cfg, device="cuda", max_seqs=4, max_ctx=2048, max_width=5, seed=1, gdn_prefill="rows")
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


def test_sampled_requests_draw_from_the_device_seam(executor):
    """Sampled requests on the real engine: the head leaves the 64 best logits per row, the host
    sampler draws from them; top_k = 1 equals greedy, a seed fixes the ids, another seed moves them."""
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, executor.vocab, (90,), generator=g).tolist()
    from saber_engine_b200.serve.sampler import HostSampler

    def run(**kw):
        s = Scheduler(executor, SchedulerConfig(max_seqs=4, max_ctx=2048, prefix_cache=False), sampler=HostSampler())
        sub = s.submit(EngineRequest(prompt, SamplingParams(max_tokens=12, ignore_eos=True, **kw)))
        s.run_until_idle()
        return _collect(sub)[0]
    greedy = run()
    assert run(temperature=1.0, top_k=1, seed=3) == greedy
    a, b, c = run(temperature=1.5, seed=11), run(temperature=1.5, seed=11), run(temperature=1.5, seed=12)
    assert a == b and len(a) == 12
    assert a != greedy or c != greedy          # flat random-init logits: a hot draw leaves the greedy path
    # the seam itself against the logits the program left behind
    bkt = executor._bucket("decode", 1, 5, seam=True)
    import numpy as np
    K, Mh = 64, bkt.Mh
    arr = bkt.seam_host.numpy()
    ids = torch.from_numpy(arr[:Mh * K].reshape(Mh, K).astype(np.int64))
    vals = torch.from_numpy(arr[Mh * K:2 * Mh * K].view(np.float32).reshape(Mh, K).copy())
    lse = torch.from_numpy(arr[2 * Mh * K:].view(np.float32).reshape(Mh, 2)[:, 0].copy())
    logits = bkt.logits[:, :executor.vocab].float().cpu()
    tv, _ = torch.topk(logits, K, dim=-1)
    assert torch.equal(vals, tv) and torch.equal(logits.gather(1, ids), vals)
    assert torch.allclose(lse, torch.logsumexp(logits, -1), atol=1e-3)


def test_greedy_request_with_logprobs_reads_the_seam(executor):
    g = torch.Generator().manual_seed(6)
    prompt = torch.randint(0, executor.vocab, (40,), generator=g).tolist()
    s = _sched(executor, prefix_cache=False)
    sub = s.submit(EngineRequest(prompt, SamplingParams(max_tokens=10, ignore_eos=True, logprobs=2)))
    plain = s.submit(EngineRequest(prompt, SamplingParams(max_tokens=10, ignore_eos=True)))
    s.run_until_idle()
    toks, lps = [], []
    while True:
        ev = sub.events.get(timeout=60)
        toks += ev.new_token_ids
        lps += ev.logprobs or []
        if ev.finished:
            break
    assert toks == _collect(plain)[0]                       # asking for log-probabilities does not move the ids
    assert len(lps) == 10 and [x["token_id"] for x in lps] == toks
    for x in lps:
        assert x["logprob"] <= 0.0 and len(x["top"]) == 2
        assert x["top"][0][0] == x["token_id"] and abs(x["top"][0][1] - x["logprob"]) < 1e-6   # greedy = best candidate
        assert x["top"][1][1] <= x["top"][0][1]


def test_prompt_logprobs_match_a_full_logits_pass(executor):
    """Prompt log-probabilities from the prefill bucket variant (head over every row) against
    log-softmax of the logits that variant leaves behind."""
    g = torch.Generator().manual_seed(8)
    prompt = torch.randint(0, executor.vocab, (64,), generator=g).tolist()
    s = _sched(executor, prefix_cache=False)
    sub = s.submit(EngineRequest(prompt, SamplingParams(max_tokens=3, ignore_eos=True, prompt_logprobs=1)))
    s.run_until_idle()
    ev = sub.events.get(timeout=60)
    plp = ev.prompt_logprobs
    assert ev.first_token and len(plp) == 63 and [x["token_id"] for x in plp] == prompt[1:]
    toks = list(ev.new_token_ids)
    while not ev.finished:
        ev = sub.events.get(timeout=60)
        toks += ev.new_token_ids
    for x in plp:
        assert x["logprob"] <= 1e-3 and x["top"][0][1] >= x["logprob"] - 1e-3 and x["top"][0][1] <= 1e-3
    b = [v for k, v in executor.model.buckets.items() if k[-1] == "plp" and k[2] == 64][0]
    logits_all = b.plp_logits
    ref = torch.log_softmax(logits_all[:63, :executor.vocab].float(), -1).cpu()
    got = torch.tensor([x["logprob"] for x in plp])
    want = ref[torch.arange(63), torch.tensor(prompt[1:])]
    assert torch.allclose(got, want, atol=2e-3), (got - want).abs().max()
    # the same prompt without the field gives the same ids (a separate run: the state slot is reused)
    s2 = _sched(executor, prefix_cache=False)
    plain = s2.submit(EngineRequest(prompt, SamplingParams(max_tokens=3, ignore_eos=True)))
    s2.run_until_idle()
    assert toks == _collect(plain)[0]


def test_device_draws_agree_with_the_host_sampler_during_sampled_decoding(executor):
    from saber_engine_b200.serve.sampler import HostSampler
    g = torch.Generator().manual_seed(9)
    prompt = torch.randint(0, executor.vocab, (50,), generator=g).tolist()
    s = Scheduler(executor, SchedulerConfig(max_seqs=4, max_ctx=2048, prefix_cache=False), sampler=HostSampler())
    sub = s.submit(EngineRequest(prompt, SamplingParams(max_tokens=24, ignore_eos=True, temperature=1.0, top_k=40, seed=7)))
    s.run_until_idle()
    toks = _collect(sub)[0]
    assert len(toks) == 24
    c = s.counters
    assert c["sampled_steps"] > 0 and c["sampled_steps_device_agrees"] >= c["sampled_steps"] - 1
