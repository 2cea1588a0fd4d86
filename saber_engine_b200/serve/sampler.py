"""Host sampler over a seam row (top-k candidates + log-sum-exp) or a full logits row.

Order of operations follows vLLM V1 (the parity target of `crates/saber-serve/src/sampler.rs:8-30`):
penalties (repetition, then frequency and presence) -> temperature -> min_p -> top_k -> top_p ->
draw.  The draw is a function of (seed, sequence id, absolute output position) only, never of the
batch or the step it happened to run in, so seeded sampling is invariant to scheduling
(`crates/saber-engine/tests/seeded_invariance.rs:1-20`).

A seam row carries the 64 largest logits (value desc, id asc), the ids, and lse at T = 1: the
sampler renormalises inside the candidate set after filtering, which equals sampling the full
distribution whenever top_k <= 64 or the nucleus fits inside the candidates (otherwise the tail
mass beyond 64 candidates is dropped, as in the reference).
"""
from __future__ import annotations

import hashlib
import math
import struct
from collections import Counter
from typing import Optional

from .engine_api import SamplingParams


def uniform01(seed: int, seq_uid: int, position: int) -> float:
    h = hashlib.blake2b(struct.pack("<qqq", seed, seq_uid, position), digest_size=8).digest()
    return (struct.unpack("<Q", h)[0] >> 11) * (1.0 / (1 << 53))


def apply_penalties(ids, vals, params: SamplingParams, prompt, output):
    if params.repetition_penalty == 1.0 and params.frequency_penalty == 0.0 and params.presence_penalty == 0.0:
        return list(vals)
    out_counts = Counter(output)
    seen = set(prompt) | set(output)
    res = []
    for i, v in zip(ids, vals):
        if params.repetition_penalty != 1.0 and i in seen:
            v = v / params.repetition_penalty if v > 0 else v * params.repetition_penalty
        c = out_counts.get(i, 0)
        if c:
            v -= params.frequency_penalty * c + params.presence_penalty
        res.append(v)
    return res


def sample_candidates(ids, vals, params: SamplingParams, prompt, output, u: float):
    """ids/vals: candidate token ids and raw logits (any order). Returns (token, logprob at T)."""
    vals = apply_penalties(ids, vals, params, prompt, output)
    if params.greedy:
        best = max(range(len(ids)), key=lambda j: (vals[j], -ids[j]))
        return ids[best], 0.0
    t = max(params.temperature, 1e-6)
    order = sorted(range(len(ids)), key=lambda j: (-vals[j], ids[j]))
    lg = [vals[j] / t for j in order]
    tok = [ids[j] for j in order]
    m = lg[0]
    probs = [math.exp(x - m) for x in lg]
    z = sum(probs)
    probs = [p / z for p in probs]
    keep = len(probs)
    if params.min_p > 0:
        thr = params.min_p * probs[0]
        keep = min(keep, sum(1 for p in probs if p >= thr))
    if params.top_k > 0:
        keep = min(keep, params.top_k)
    if params.top_p < 1.0:
        acc, k = 0.0, 0
        for p in probs[:keep]:
            acc += p
            k += 1
            if acc >= params.top_p:
                break
        keep = min(keep, k)
    keep = max(1, keep)
    z = sum(probs[:keep])
    x, acc = u * z, 0.0
    for j in range(keep):
        acc += probs[j]
        if x < acc:
            return tok[j], math.log(probs[j] / z)
    return tok[keep - 1], math.log(probs[keep - 1] / z)


class HostSampler:
    """Sampler object the scheduler calls for sampled sequences."""

    def __init__(self, default_seed: int = 0):
        self.default_seed = default_seed

    def sample_row(self, seam: dict, row: int, params: SamplingParams, prompt, output, position: int,
                   seq_uid: int) -> int:
        ids, vals = seam["ids"][row], seam["vals"][row]
        seed = params.seed if params.seed is not None else self.default_seed ^ (seq_uid * 0x9E3779B1)
        # with an explicit seed the draw must not depend on which engine-assigned id the request got
        uid = 0 if params.seed is not None else seq_uid
        tok, _ = sample_candidates(list(ids), list(vals), params, prompt, output, uniform01(seed, uid, position))
        return int(tok)

    def uniforms(self, params: SamplingParams, seq_uid: int, position0: int, n: int) -> list:
        """The uniform numbers `sample_row` will use at positions position0 .. position0 + n - 1 (the
        device draws with the same numbers)."""
        seed = params.seed if params.seed is not None else self.default_seed ^ (seq_uid * 0x9E3779B1)
        uid = 0 if params.seed is not None else seq_uid
        return [uniform01(seed, uid, position0 + r) for r in range(n)]

    @staticmethod
    def device_params(params: SamplingParams):
        """(temperature, top_k, top_p, min_p) when the device can repeat the host's draw: no penalties."""
        if params.greedy or params.repetition_penalty != 1.0 or params.frequency_penalty != 0.0 or params.presence_penalty != 0.0:
            return None
        return (float(params.temperature), float(params.top_k), float(params.top_p), float(params.min_p))

    @staticmethod
    def seam_from_logits(logits_rows, k: int = 64) -> dict:
        """Build a seam from full logits rows (CPU executors): top-k by (value desc, id asc)."""
        import torch
        k = min(k, logits_rows.shape[-1])
        vals, ids = torch.topk(logits_rows.float(), k, dim=-1)
        lse = torch.logsumexp(logits_rows.float(), -1)
        return {"ids": ids.tolist(), "vals": vals.tolist(), "lse": lse.tolist()}

    @staticmethod
    def top_logprobs(seam: dict, row: int, n: int) -> list:
        lse = seam["lse"][row] if not isinstance(seam["lse"][row], (list, tuple)) else seam["lse"][row][0]
        return [(int(i), float(v - lse)) for i, v in list(zip(seam["ids"][row], seam["vals"][row]))[:n]]
