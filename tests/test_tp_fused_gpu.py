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


@pytest.mark.parametrize("nranks,M,splits", [(2, 9, 1), (4, 40, 2), (8, 72, 1)])
def test_gemm_push_then_reduce_norm_quant(nranks, M, splits):
    torch.manual_seed(nranks)
    H, K = 512, 256 * nranks                      # hidden (GEMM N) and the full reduction dim
    Kr = K // nranks
    group = SymmetricComm.local_group(nranks, DEV, max_elems=128 * H, rows_max=128, hidden=H)
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
            p = F.gemm_params(qw, qa, dummy, sc, splits=splits)
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
