import math

import torch

from saber_engine_b200.serve.engine_api import SamplingParams
from saber_engine_b200.serve.sampler import HostSampler, apply_penalties, sample_candidates, uniform01


def test_greedy_ties_go_to_the_lower_id():
    tok, _ = sample_candidates([7, 3, 9], [1.0, 2.0, 2.0], SamplingParams(), [], [], 0.3)
    assert tok == 3


def test_top_k_top_p_min_p_restrict_support():
    ids, vals = list(range(10)), [float(10 - i) for i in range(10)]
    seen = {sample_candidates(ids, vals, SamplingParams(temperature=1.0, top_k=2), [], [], u / 50)[0] for u in range(50)}
    assert seen == {0, 1}
    seen = {sample_candidates(ids, vals, SamplingParams(temperature=1.0, top_p=0.5), [], [], u / 50)[0] for u in range(50)}
    assert seen == {0}
    seen = {sample_candidates(ids, vals, SamplingParams(temperature=1.0, min_p=0.3), [], [], u / 50)[0] for u in range(50)}
    assert seen == {0, 1}        # p1/p0 = e^-1 = 0.37 >= 0.3, p2/p0 = 0.135 < 0.3


def test_distribution_matches_softmax():
    ids, vals = [0, 1, 2], [0.0, math.log(2.0), math.log(5.0)]
    n = 4000
    counts = [0, 0, 0]
    for i in range(n):
        counts[sample_candidates(ids, vals, SamplingParams(temperature=1.0), [], [], (i + 0.5) / n)[0]] += 1
    assert abs(counts[0] / n - 1 / 8) < 0.01 and abs(counts[2] / n - 5 / 8) < 0.01


def test_penalties_follow_vllm_order():
    p = SamplingParams(temperature=1.0, repetition_penalty=2.0, frequency_penalty=0.5, presence_penalty=0.25)
    out = apply_penalties([1, 2, 3], [4.0, -4.0, 1.0], p, prompt=[1], output=[2, 2])
    assert out[0] == 2.0                               # positive logit divided (seen in the prompt)
    assert out[1] == -8.0 - 0.5 * 2 - 0.25             # negative multiplied, then frequency and presence
    assert out[2] == 1.0


def test_seeded_draw_depends_only_on_seed_and_position():
    s = HostSampler()
    logits = torch.randn(3, 500)
    seam = s.seam_from_logits(logits)
    p = SamplingParams(temperature=0.9, seed=1234)
    a = [s.sample_row(seam, 1, p, [], [], pos, seq_uid=5) for pos in range(20)]
    b = [s.sample_row(seam, 1, p, [], [], pos, seq_uid=99) for pos in range(20)]   # another engine id
    assert a == b and len(set(a)) > 1
    assert uniform01(1, 2, 3) == uniform01(1, 2, 3) != uniform01(1, 2, 4)
    lp = s.top_logprobs(seam, 0, 5)
    assert len(lp) == 5 and all(v <= 0 for _, v in lp)
