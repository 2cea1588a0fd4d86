"""Fused tails of the tcgen05 GEMM against the separate launches they replace (same bytes), and the
separate launches against the fp32 restatement."""
import ctypes as C

import pytest
import torch

from saber_engine_b200.ops import functional as F
from saber_engine_b200.ops import layouts as L
from saber_engine_b200.ops import native as N
from saber_engine_b200.ops import reference as R

pytestmark = pytest.mark.gpu


def _launch(p, stages=0):
    N.check(N.lib().saber_gemm_i8_launch(C.byref(p), stages, N.stream_handle()), "gemm_i8")


@pytest.mark.parametrize("M,inter,K", [(8, 256, 512), (64, 1024, 1024), (72, 640, 2048), (5, 128, 256)])
def test_gate_up_silu_quant_in_the_epilogue_equals_gemm_then_row_kernel(M, inter, K):
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(M + inter)
    w = torch.randn(2 * inter, K, generator=g) * 0.05
    x = torch.randn(M, K, generator=g)
    qw = F.QuantWeight.from_float(w, 4, dev)
    qa = F.plain_quant(x.to(torch.bfloat16).to(dev))
    # separate launches on the canonical weight
    gu = F.gemm_i8(qw, qa, splits=1)
    want, act = F.silu_mul_quant(gu, want_out=True)
    # fp32 restatement of the separate launches
    gu_ref = gu.float()
    ref = R.bf16_round(torch.nn.functional.silu(gu_ref[:, :inter]) * gu_ref[:, inter:])
    assert (act.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-6
    # paired weight: GEMM + paired row kernel, then the fused launch
    qp = F.pair_gate_up(qw)
    assert qp.paired
    gu_p = F.gemm_i8(qp, qa, splits=1)
    want_p, _ = F.silu_mul_quant(gu_p, paired=True)
    assert torch.equal(want_p.q[:, :M], want.q[:, :M]) and torch.equal(want_p.scale[:M], want.scale[:M])
    for call in range(2):      # twice: the second launch meets the words the first one left
        got = F.QuantAct.alloc(M, inter, dev)
        got.q.fill_(77)
        got.scale.fill_(-1.0)
        sc = F.scratch(dev)
        p = F.gemm_params(qp, qa, gu_p, sc, splits=1)
        assert F.gemm_tail_ok(p)
        F.gemm_tail_silu_quant(p, got, sc)
        _launch(p)
        torch.cuda.synchronize()
        sc.check()
        assert torch.equal(got.scale[:M], want.scale[:M])
        assert torch.equal(got.q[:, :M], want.q[:, :M])
        assert int(got.q[:, M:].abs().max().item()) == 0 if got.M_pad > M else True
        assert int(sc.tail_sync[0].item()) == 0 and int(sc.tail_sync[64 + 256 * 32:].abs().max().item()) == 0   # barrier word and flags re-armed


@pytest.mark.parametrize("M,H,K,splits,bits", [(8, 512, 1024, 1, 4), (64, 5120, 1024, 4, 4), (72, 1024, 2048, 2, 8),
                                               (9, 6144, 512, 1, 4)])
def test_row_tail_equals_gemm_then_add_rms_kernel(M, H, K, splits, bits):
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(M + H)
    w = torch.randn(H, K, generator=g) * 0.05
    x = torch.randn(M, K, generator=g)
    res0 = (torch.randn(M, H, generator=g)).to(torch.bfloat16).to(dev)
    nw = (torch.randn(H, generator=g) * 0.1).to(dev)
    qw = F.QuantWeight.from_float(w, bits, dev)
    qa = F.plain_quant(x.to(torch.bfloat16).to(dev))
    # separate launches
    delta = F.gemm_i8(qw, qa, splits=splits)
    res_a = res0.clone()
    want, normed_a = F.add_rms_quant(delta, res_a, nw, want_out=True)
    # fp32 restatement
    s = R.bf16_round(delta.float().cpu() + res0.float().cpu())
    ref = R.bf16_round(s * torch.rsqrt((s * s).mean(dim=1, keepdim=True) + 1e-6) * (1.0 + nw.cpu()))
    assert (normed_a.float().cpu() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-6
    for call in range(2):
        res_b = res0.clone()
        tap = torch.zeros_like(res0)
        delta_b = torch.zeros_like(delta)
        got = F.QuantAct.alloc(M, H, dev)
        got.q.fill_(55)
        normed_b = torch.zeros(M, H, dtype=torch.bfloat16, device=dev)
        sc = F.scratch(dev)
        p = F.gemm_params(qw, qa, delta_b, sc, splits=splits)
        assert F.gemm_tail_ok(p)
        rp = F.row_params(M, H, a=delta_b, res=res_b, w=nw, w_offset=1.0, eps=1e-6, out=normed_b, qa=got)
        rp.res_copy = tap.data_ptr()
        F.gemm_tail_row(p, rp, sc)
        _launch(p)
        torch.cuda.synchronize()
        sc.check()
        if splits == 1:                 # (with split-K on one GPU the row tail reads the int32 accumulators: no bf16 tile)
            assert torch.equal(delta_b, delta)
        assert torch.equal(res_b, res_a) and torch.equal(tap, res_a)
        assert torch.equal(normed_b, normed_a)
        assert torch.equal(got.scale[:M], want.scale[:M]) and torch.equal(got.q[:, :M], want.q[:, :M])
        if got.M_pad > M:
            assert int(got.q[:, M:].abs().max().item()) == 0
        assert int(sc.tail_sync[0].item()) == 0 and int(sc.tail_sync[64 + 256 * 32:].abs().max().item()) == 0
        assert int(sc.counters.abs().max().item()) == 0
        assert int(sc.acc.abs().max().item()) == 0        # the shared accumulator blocks stay zero


def test_tails_are_refused_when_the_grid_is_not_resident():
    dev = torch.device("cuda")
    qw = F.QuantWeight.from_float(torch.randn(256 * 200, 256) * 0.05, 4, dev)      # 200 feature tiles > SM count
    qa = F.plain_quant(torch.randn(8, 256).to(torch.bfloat16).to(dev))
    out = torch.zeros(8, 256 * 200, dtype=torch.bfloat16, device=dev)
    sc = F.scratch(dev)
    p = F.gemm_params(qw, qa, out, sc, splits=1)
    assert not F.gemm_tail_ok(p)
    rp = F.row_params(8, 256 * 200, a=out, w=torch.zeros(256 * 200, device=dev), qa=None)
    F.gemm_tail_row(p, rp, sc)
    assert N.lib().saber_gemm_i8_launch(C.byref(p), 0, N.stream_handle()) != 0
    torch.cuda.synchronize()


@pytest.mark.parametrize("M,Nn,K", [(8, 512, 512), (64, 16640, 1024), (72, 1000, 2048)])
def test_half_tile_ctas_equal_whole_tiles(M, Nn, K):
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(Nn)
    qw = F.QuantWeight.from_float(torch.randn(Nn, K, generator=g) * 0.05, 4, dev)
    qa = F.plain_quant(torch.randn(M, K, generator=g).to(torch.bfloat16).to(dev))
    want = F.gemm_i8(qw, qa, splits=1)
    got = F.gemm_i8(qw, qa, splits=1, halves=2)
    torch.cuda.synchronize()
    F.scratch(dev).check()
    assert torch.equal(got, want)


def test_split_k_accumulator_blocks_return_to_zero():
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(3)
    qw = F.QuantWeight.from_float(torch.randn(768, 4096, generator=g) * 0.05, 4, dev)
    qa = F.plain_quant(torch.randn(40, 4096, generator=g).to(torch.bfloat16).to(dev))
    one = F.gemm_i8(qw, qa, splits=1)
    for _ in range(2):
        many = F.gemm_i8(qw, qa, splits=4)
        torch.cuda.synchronize()
        assert torch.equal(one, many)          # integer partial sums: any order, the same bytes
        assert int(F.scratch(dev).acc.abs().max().item()) == 0
