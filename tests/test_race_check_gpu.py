"""Race checks on the GPU: digest kernel against its host oracle, eager == graph stage digests,
and the poison arm (activation arenas filled with NaN bytes before a step change nothing)."""
import ctypes as C

import pytest
import torch

from saber_engine_b200.models import config as MC
from saber_engine_b200.models.hybrid import HybridModel, SeqStep, run_bucket
from saber_engine_b200.ops import native as N
from saber_engine_b200.runtime import race_check as RC

pytestmark = pytest.mark.gpu


def test_digest_kernel_matches_host_oracle_and_sees_position():
    x = torch.randint(0, 2 ** 31, (40001 * 2,), dtype=torch.int32, device="cuda")
    out = torch.zeros(2, dtype=torch.int64, device="cuda")
    lib = N.lib()
    N.check(lib.saber_digest_launch(x.data_ptr(), x.numel() * 4, out.data_ptr(), N.stream_handle()), "digest")
    y = x.clone()
    y[[0, 2]] = y[[2, 0]]                      # same multiset of words, two of them swapped
    y[[1, 3]] = y[[3, 1]]
    N.check(lib.saber_digest_launch(y.data_ptr(), y.numel() * 4, out.data_ptr() + 8, N.stream_handle()), "digest")
    torch.cuda.synchronize()
    got = [int(v) & RC.MASK for v in out.cpu().tolist()]
    assert got[0] == RC.digest_reference(x.cpu().numpy().tobytes())
    assert got[1] == RC.digest_reference(y.cpu().numpy().tobytes())
    assert got[0] != got[1]


def test_shadow_digests_eager_equals_graph_and_poison_changes_nothing():
    cfg = MC.scaled_hybrid()
    model = HybridModel(cfg, device="cuda", max_seqs=2, max_ctx=512, max_width=5, seed=3, race_check="shadow")
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (50,), generator=g).tolist()
    blocks = list(range(1, 33))
    model.reset_slot(1)
    pb = model.build_bucket("prefill", 1, 64)
    r = run_bucket(model, pb, [SeqStep(prompt, 0, 1, 0, blocks)])
    db = model.build_bucket("decode", 1, 5)
    rows = [r.tokens[0][0]] + (r.drafts[0] + [0] * 5)[:4]
    seqs = [SeqStep(rows, len(prompt), 1, 0, blocks, uid=1, step_no=0)]
    rep = RC.shadow_compare(model, db, seqs)
    assert rep["stages"] == cfg.n_layers + 1 and rep["mismatches"] == []
    # poison arm: NaN bytes in every activation arena before the step leave result and digests unchanged
    base = run_bucket(model, db, seqs)
    want = RC.read_digests(db)
    logits = db.logits.clone()
    assert RC.poison_arenas(db, 0xFF) > 0
    again = run_bucket(model, db, seqs)
    assert again.tokens == base.tokens and again.drafts == base.drafts
    assert RC.read_digests(db) == want
    assert torch.equal(db.logits, logits) and not torch.isnan(db.logits.float()).any()
    model.scratch.check()
