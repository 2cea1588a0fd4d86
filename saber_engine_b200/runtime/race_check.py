"""Hand-built race checks (there is no sanitizer on the serving path).

* **Shadow digests** (`HybridModel(race_check="shadow")`): an order-free XOR-splitmix digest of the
  residual stream is enqueued after every layer inside the step program and read back with the
  step's result.  `shadow_compare` runs the same step as a serialised eager walk and as a graph
  replay and compares the digests stage by stage: the first differing stage names the layer whose
  launch read something that was not there yet.
* **Poison arm** (`poison_arenas`): fills every pure activation buffer of a bucket with a byte
  pattern (0xFF = NaN in bf16 / fp32) before a step.  A kernel that reads a buffer before the step
  has written it turns the logits into NaN instead of silently reusing last step's bytes.
* **Digest oracle** (`digest_reference`): the same function on the host, to test the kernel.

Parity: `crates/saber-kernels/hip/race_digest.hip:1-26`, `crates/saber-engine/src/device/shadow.rs:1-15`
(shadow digest), `crates/saber-engine/tests/poison_boot.rs:1-3` (`--poison-boot SET:BYTE`),
`crates/saber-engine/src/race.rs:1-25` (counted, not retried).
"""
from __future__ import annotations

import numpy as np
import torch

MASK = (1 << 64) - 1


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = (x + np.uint64(0x9E3779B97F4A7C15))
        x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return x ^ (x >> np.uint64(31))


def digest_reference(raw: bytes) -> int:
    words = np.frombuffer(raw, dtype=np.uint64)
    idx = np.arange(words.size, dtype=np.uint64)
    h = _splitmix64(words ^ _splitmix64(idx))
    return int(np.bitwise_xor.reduce(h)) if words.size else 0


def read_digests(bucket) -> list:
    return [int(v) & MASK for v in bucket.digests.cpu().tolist()]


def poison_arenas(bucket, byte: int = 0xFF) -> int:
    """Returns the number of bytes poisoned."""
    n = 0
    for t in bucket.arenas:
        t.view(torch.uint8).fill_(byte)
        n += t.numel() * t.element_size()
    return n


def shadow_compare(model, bucket, seqs: list) -> dict:
    """Eager (one launch at a time, stream-serialised) against the captured graph, same inputs.
    The step must not commit state (decode rows with shift 0), so both runs start from the same bytes."""
    from ..models.hybrid import run_bucket
    assert bucket.digests is not None, "build the model with race_check='shadow'"
    run_bucket(model, bucket, seqs, eager=True)
    torch.cuda.synchronize()
    a = read_digests(bucket)
    run_bucket(model, bucket, seqs, eager=False)
    torch.cuda.synchronize()
    b = read_digests(bucket)
    diff = [i for i, (x, y) in enumerate(zip(a, b)) if x != y]
    return {"stages": len(a), "mismatches": diff, "first_bad_layer": diff[0] if diff else None}
