"""Fused tensor-parallel path on ONE GPU: the ranks are emulated in one process with one heap each
(ordinary device pointers stand in for peer mappings).  All pushing GEMMs are launched before any
consumer, so no kernel ever waits for a launch that has not happened yet."""
import ctypes as C

import pytest
import torch

from saber_engine_b200.ops import functional as F
from saber_engine_b200.ops import layouts as L
from saber_engine_b200.ops import native as N
from saber_engine_b200.ops import reference as R
from saber_engine_b200.parallel.symm import SymmetricComm

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("nranks,M,splits", [(2, 9, 1), (4, 40, 2), (8, 72, 1), (2, 256, 1)])   # the last: two token tiles per CTA
def test_gemm_push_then_reduce_norm_quant(nranks, M, splits):
    torch.manual_seed(nranks)
    H, K = 512, 256 * nranks                      # hidden (GEMM N) and the full reduction dim
    Kr = K // nranks
    group = SymmetricComm.local_group(nranks, DEV, max_elems=max(128, M) * H, rows_max=max(128, M), hidden=H)
    for g in group:
        g._local = True
    w = torch.randn(H, K) * 0.02
    x = torch.randn(M, K)
    res = torch.randn(M, H).to(torch.bfloat16)
    nw = torch.randn(H) * 0.1
    sc = F.scratch(DEV)
    partial_ref = []
    for site in (0, 1, 2):                        # three calls: both parities and a slot reuse
        outs = []
        for r, g in enumerate(group):             # phase 1: every rank's GEMM pushes
            g.seq_base.fill_(site * 0)            # the base only advances at program ends
            wq, ws = L.quantize_weight_rows(w[:, r * Kr:(r + 1) * Kr], 4)
            aq, asc = L.quantize_act_rows(x[:, r * Kr:(r + 1) * Kr])
            if site == 0:
                partial_ref.append(R.gemm_i8(wq, ws, aq, asc).float())
            qw = F.QuantWeight.from_int(wq, ws, 4, DEV)
            m_pad = L.padded_rows(M)
            qa = F.QuantAct(L.tile_act_int8(aq, m_pad).to(DEV), torch.cat([asc, torch.zeros(m_pad - M)]).to(DEV), M, Kr)
            dummy = torch.zeros(M, H, dtype=torch.bfloat16, device=DEV)
            p = F.gemm_params(qw, qa, dummy, sc, splits=splits, mtiles=2 if M > 128 else 0)
            g.gemm_tp(p, site)
            parts = N.lib().saber_gemm_i8_parts(C.byref(p))
            N.check(N.lib().saber_gemm_i8_launch(C.byref(p), 0, N.stream_handle()), "gemm")
            outs.append((qw, qa, dummy))
        torch.cuda.synchronize()
        sc.check()
        ref_sum = R.bf16_round(sum(partial_ref))
        res_ref, n_ref = R.add_rms(ref_sum, res, nw)
        for r, g in enumerate(group):             # phase 2: every rank consumes
            res_d = res.to(DEV).clone()
            qa_out = F.QuantAct.alloc(M, H, DEV)
            normed = torch.zeros(M, H, dtype=torch.bfloat16, device=DEV)
            p = F.row_params(M, H, a=None, res=res_d, w=nw.to(DEV), w_offset=1.0, qa=qa_out, out=normed)
            g.row_tp(p, site, L.token_tile(M), H // 256 * parts)
            N.check(N.lib().saber_row_producer_launch(N.ROW_ADD_RMS, C.byref(p), N.stream_handle()), "consumer")
            torch.cuda.synchronize()
            g.check()
            assert torch.allclose(res_d.float().cpu(), res_ref.float(), atol=3e-2, rtol=2e-2), (site, r)
            assert torch.allclose(normed.float().cpu(), n_ref, atol=4e-2, rtol=3e-2), (site, r)
            if r > 0:
                assert torch.equal(normed, first_normed)     # rank order is fixed: bit-identical on every rank
            else:
                first_normed = normed.clone()
    group[0].close()


def test_consumer_wait_runs_out_cleanly_when_a_rank_never_pushes():
    """Failure detection without a fault: a flag that nothing sets makes the bounded wait run out,
    the kernel records it and returns, and the context stays usable."""
    group = SymmetricComm.local_group(2, DEV, max_elems=16 * 256, rows_max=16, hidden=256)
    for g in group:
        g._local = True
    g = group[0]
    M, H = 4, 256
    res = torch.zeros(M, H, dtype=torch.bfloat16, device=DEV)
    qa = F.QuantAct.alloc(M, H, DEV)
    p = F.row_params(M, H, a=None, res=res, w=torch.zeros(H, device=DEV), w_offset=1.0, qa=qa)
    g.row_tp(p, 0, 16, 1)
    N.check(N.lib().saber_row_producer_launch(N.ROW_ADD_RMS, C.byref(p), N.stream_handle()), "consumer")
    torch.cuda.synchronize()
    with pytest.raises(N.NativeError, match="wait_peer"):
        g.check()
    assert float((torch.ones(4, device=DEV) * 2).sum()) == 8.0      # the context still answers
    group[0].close()


@pytest.mark.parametrize("nranks,M", [(2, 256), (4, 512)])
def test_sequence_parallel_reduce_scatter_norm_allgather_gemm(nranks, M):
    """The sequence-parallel chain on ONE GPU with emulated ranks, phase by phase:
    (1) every rank's row-parallel GEMM pushes each row's partial to the row's OWNER only,
    (2) every rank's add-norm-quant handles the rows it owns and stores the quantised rows into EVERY
        rank's buffer, raising one arrival flag per 128-row tile,
    (3) every rank's next GEMM waits for those flags before it loads its token tiles.
    Every producer runs before its consumers, so no launch waits for a later one."""
    torch.manual_seed(20 + nranks)
    H, K = 512, 256 * nranks
    Kr, rpr = K // nranks, M // nranks
    group = SymmetricComm.local_group(nranks, DEV, max_elems=M * H, rows_max=M, hidden=H)
    for g in group:
        g._local = True
    w = torch.randn(H, K) * 0.02
    w2 = torch.randn(384, H) * 0.02
    x = torch.randn(M, K)
    res = torch.randn(M, H).to(torch.bfloat16)
    nw = torch.randn(H) * 0.1
    sc = F.scratch(DEV)
    wq_full, ws_full = L.quantize_weight_rows(w, 4)
    partial_ref, keep = [], []
    for r, g in enumerate(group):                          # phase 1: reduce-scatter epilogues
        aq, asc = L.quantize_act_rows(x[:, r * Kr:(r + 1) * Kr])
        partial_ref.append(R.gemm_i8(wq_full[:, r * Kr:(r + 1) * Kr], ws_full, aq, asc).float())
        qw = F.QuantWeight.from_int(wq_full[:, r * Kr:(r + 1) * Kr].contiguous(), ws_full, 4, DEV)
        m_pad = L.padded_rows(M)
        qa = F.QuantAct(L.tile_act_int8(aq, m_pad).to(DEV), torch.cat([asc, torch.zeros(m_pad - M)]).to(DEV), M, Kr)
        dummy = torch.zeros(M, H, dtype=torch.bfloat16, device=DEV)
        p = F.gemm_params(qw, qa, dummy, sc, splits=1, mtiles=2)     # owner-only push from paired token tiles
        g.gemm_rs(p, 0, rpr)
        N.check(N.lib().saber_gemm_i8_launch(C.byref(p), 0, N.stream_handle()), "gemm rs")
        keep.append((qw, qa, dummy))
    torch.cuda.synchronize()
    sc.check()
    ref_sum = R.bf16_round(sum(partial_ref))
    res_ref, n_ref = R.add_rms(ref_sum, res, nw)
    res_shards = []
    for r, g in enumerate(group):                          # phase 2: owners norm + quantise + all-gather
        res_d = res.to(DEV).clone()
        qa_heap = g.heap_qact(M, H)
        p = F.row_params(M, H, a=None, res=res_d, w=nw.to(DEV), w_offset=1.0, qa=qa_heap)
        g.row_sp(p, 0, L.token_tile(M), H // 256, rpr)
        N.check(N.lib().saber_row_producer_launch(N.ROW_ADD_RMS, C.byref(p), N.stream_handle()), "sp consumer")
        res_shards.append(res_d)
    torch.cuda.synchronize()
    for r, g in enumerate(group):
        g.check()
        own = slice(r * rpr, (r + 1) * rpr)
        assert torch.allclose(res_shards[r][own].float().cpu(), res_ref[own].float(), atol=3e-2, rtol=2e-2)
        if r + 1 < nranks:                                  # rows of other ranks are not touched here
            other = slice((r + 1) * rpr, (r + 2) * rpr)
            assert torch.equal(res_shards[r][other].cpu(), res[other])
    aq2, asc2 = L.quantize_act_rows(n_ref)
    qw2 = F.QuantWeight.from_float(w2, 4, DEV)
    want = R.gemm_i8(*L.quantize_weight_rows(w2, 4), aq2, asc2).float()
    outs = []
    for r, g in enumerate(group):                          # phase 3: the next GEMM waits on the arrival flags
        qa_heap = g.heap_qact(M, H)
        assert torch.allclose(qa_heap.scale[:M].cpu(), asc2, rtol=2e-2, atol=1e-6)
        out = torch.zeros(M, 384, dtype=torch.bfloat16, device=DEV)
        p = F.gemm_params(qw2, qa_heap, out, sc, splits=1)
        g.gemm_ag(p, 0)
        N.check(N.lib().saber_gemm_i8_launch(C.byref(p), 0, N.stream_handle()), "gemm ag")
        outs.append(out)
    torch.cuda.synchronize()
    sc.check()
    for r, g in enumerate(group):
        g.check()
        err = (outs[r].float().cpu() - want).abs().max().item()
        assert err <= 0.05 * want.abs().max().item() + 1e-3, (r, err)
        assert torch.equal(outs[r], outs[0])                # every rank holds the same gathered rows
    group[0].close()


def test_allgather_wait_runs_out_cleanly_when_no_owner_pushes():
    """The fused all-gather wait is bounded: a flag nothing sets ends in a status word, not a hang."""
    group = SymmetricComm.local_group(2, DEV, max_elems=128 * 256, rows_max=128, hidden=256)
    g = group[0]
    g._local = True
    qw = F.QuantWeight.from_float(torch.randn(256, 256) * 0.02, 4, DEV)
    qa = g.heap_qact(16, 256)
    out = torch.zeros(16, 256, dtype=torch.bfloat16, device=DEV)
    p = F.gemm_params(qw, qa, out, F.scratch(DEV), splits=1)
    g.gemm_ag(p, 5)
    N.check(N.lib().saber_gemm_i8_launch(C.byref(p), 0, N.stream_handle()), "gemm ag")
    torch.cuda.synchronize()
    with pytest.raises(N.NativeError, match="wait_peer"):
        g.check()
    assert float((torch.ones(4, device=DEV) * 2).sum()) == 8.0
    group[0].close()


def _ar_emul(group, xs, checked, fault_rank=None, advance=True):
    """All emulated ranks of a one-device group through ONE cooperative launch."""
    n = len(group)
    outs = [torch.empty_like(x) for x in xs]
    diags = [torch.zeros(16, dtype=torch.int32, device=DEV) for _ in range(n)]
    e = N.ArEmulParams()
    e.nranks, e.checked = n, int(checked)
    for r, g in enumerate(group):
        p = g.allreduce_params(xs[r], outs[r], xs[r].numel(), site=0)
        p.diag, p.chk_fault = diags[r].data_ptr(), int(fault_rank == r)
        e.r[r] = p
    N.check(N.lib().saber_allreduce_emul_launch(C.byref(e), N.stream_handle()), "allreduce (emulated ranks)")
    if advance:
        for g in group:
            g.seq_base += 1              # one call site per "program run"
    torch.cuda.synchronize()
    return outs, [{k: int(d[i]) for k, i in N.AR_DIAG.items()} for d in diags]


@pytest.mark.parametrize("nranks", [2, 4, 8])
def test_allreduce_checked_twin_computes_the_served_bytes_and_counts_a_missing_check_word(nranks):
    """The one-shot all-reduce with every rank in one cooperative launch: the checked twin gives the
    served bytes and clean counters; a rank that pushes its payload but no check word (the control)
    is found by every other rank -- first source recorded, the re-read never converges within its
    bound -- and the reduced bytes are still the served ones."""
    n_elems = 32 * 512 * 8 - 64           # a checked message leaves the slot's last 32 words free
    group = SymmetricComm.local_group(nranks, DEV, max_elems=32 * 512 * 8, rows_max=128, hidden=256)
    torch.manual_seed(nranks)
    xs = [(torch.randn(n_elems, device=DEV) * 0.5).to(torch.bfloat16) for _ in range(nranks)]
    want = torch.zeros(n_elems, device=DEV)
    for x in xs:
        want += x.float()
    want = want.to(torch.bfloat16)
    served, _ = _ar_emul(group, xs, checked=False)
    for o in served:
        assert torch.equal(o, want)                       # fp32 sum in rank order, the same on every rank
    for call in range(3):                                 # both parities of the slots
        outs, diag = _ar_emul(group, xs, checked=True)
        for r in range(nranks):
            assert torch.equal(outs[r], want)
            d = diag[r]
            assert d["blocks"] == 32 and d["mismatch"] == d["never"] == d["drift"] == d["timeout"] == 0, d
    bad = 1
    outs, diag = _ar_emul(group, xs, checked=True, fault_rank=bad)
    for r in range(nranks):
        assert torch.equal(outs[r], want)
        d = diag[r]
        if r == bad:
            assert d["mismatch"] == 0
        else:
            assert d["mismatch"] == 32 and d["never"] == 32 and d["converged"] == 0 and d["first_src"] == bad and d["polls"] == 256, d
    for g in group:
        g.check()
    group[0].close()


@pytest.mark.parametrize("nranks", [2, 4, 8])
def test_sampling_candidates_merge_on_the_device_across_vocabulary_shards(nranks):
    """Every rank takes the 64 best logits of its vocabulary shard; the ranks swap them through the
    heap and merge on the device (all ranks in one cooperative launch here).  Each rank must end with
    the global best 64 (value desc, id asc) and the whole row's log-sum-exps, identical everywhere, so
    the device draw picks the same token on every rank."""
    rows, V = 9, 8192
    group = SymmetricComm.local_group(nranks, DEV, max_elems=128 * 256, rows_max=128, hidden=256)
    torch.manual_seed(nranks)
    logits = (torch.randn(rows, V, device=DEV) * 3).to(torch.bfloat16)
    logits[:, 100] = logits[:, 7000]                     # ties across shards: the lower id wins
    temps = torch.full((rows,), 0.7, device=DEV)
    vs = V // nranks
    shards = [F.topk_seam(logits[:, r * vs:(r + 1) * vs].contiguous(), temps, id_offset=r * vs) for r in range(nranks)]
    want_ids, want_vals, want_lse = F.topk_seam(logits, temps)
    e = N.SeamEmulParams()
    e.nranks = nranks
    for r, g in enumerate(group):
        e.r[r] = g.seam_merge_params(shards[r][0], shards[r][1], shards[r][2], rows, site=0)
    N.check(N.lib().saber_seam_merge_emul_launch(C.byref(e), N.stream_handle()), "seam merge (emulated ranks)")
    torch.cuda.synchronize()
    for r in range(nranks):
        ids, vals, lse = shards[r]
        assert torch.equal(ids, want_ids) and torch.equal(vals, want_vals), r
        assert torch.allclose(lse, want_lse, atol=2e-3, rtol=1e-4)
    # the device draw on two different ranks' merged rows: same candidates, same uniforms, same tokens
    samp = torch.tensor([[0.7, 40, 0.9, 0.0]] * rows, device=DEV)
    u = torch.rand(rows, device=DEV)
    picks = []
    for r in (0, nranks - 1):
        pk = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
        N.check(N.lib().saber_sample_seam_launch(shards[r][0].data_ptr(), shards[r][1].data_ptr(), samp.data_ptr(), u.data_ptr(),
                                                 pk.data_ptr(), rows, N.stream_handle()), "sample_seam")
        picks.append(pk)
    torch.cuda.synchronize()
    assert torch.equal(picks[0], picks[1]) and int(picks[0].min()) >= 0
    for g in group:
        g.check()
    group[0].close()
