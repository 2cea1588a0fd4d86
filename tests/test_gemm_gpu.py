"""tcgen05 integer GEMM against the exact integer reference (fp64 accumulate of the true ints)."""
import pytest
import torch

from saber_engine_b200.ops import functional as F
from saber_engine_b200.ops import layouts as L
from saber_engine_b200.ops import reference as R

pytestmark = pytest.mark.gpu


def _case(M, N, K, bits, splits=None, seed=0, coop=0, mtiles=0):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=g) * 0.02
    x = torch.randn(M, K, generator=g)
    wq, ws = L.quantize_weight_rows(w, bits)
    aq, asc = L.quantize_act_rows(x)
    ref = R.gemm_i8(wq, ws, aq, asc).float()
    dev = torch.device("cuda")
    qw = F.QuantWeight.from_int(wq, ws, bits, dev)
    m_pad = L.padded_rows(M)
    qa = F.QuantAct(L.tile_act_int8(aq, m_pad).to(dev), torch.cat([asc, torch.zeros(m_pad - M)]).to(dev), M, K)
    out = F.gemm_i8(qw, qa, splits=splits, coop=coop, mtiles=mtiles)
    torch.cuda.synchronize()
    F.scratch(dev).check()
    got = out.float().cpu()
    err = (got - ref).abs().max().item()
    tol = 1e-2 * ref.abs().max().item() + 1e-6   # bf16 rounding of the same exact value
    assert err <= tol, f"M={M} N={N} K={K} bits={bits} splits={splits}: max err {err} tol {tol}"
    return out


@pytest.mark.parametrize("bits", [8, 4])
def test_gemm_small_direct(bits):
    _case(5, 256, 512, bits, splits=1)


@pytest.mark.parametrize("bits", [8, 4])
def test_gemm_ragged_n_and_k_loop(bits):
    _case(9, 200, 2048, bits, splits=1)   # N not a tile multiple; 16 k-blocks > ring depth


def test_gemm_split_k_exact_and_counters_rezeroed():
    a = _case(40, 384, 4096, 4, splits=4, seed=1)
    b = _case(40, 384, 4096, 4, splits=4, seed=1)   # second launch reuses the scratch
    assert torch.equal(a, b)
    sc = F.scratch(torch.device("cuda"))
    assert int(sc.counters.abs().max().item()) == 0
    # the last-arriver form (what a grid larger than the SM count falls back to) gives the same bytes
    c = _case(40, 384, 4096, 4, splits=4, seed=1, coop=-1)
    assert torch.equal(a, c)
    assert int(sc.counters.abs().max().item()) == 0
    d = _case(72, 304, 2048, 4, splits=8, seed=2)       # ragged N, more splits than row residues of some tiles
    e = _case(72, 304, 2048, 4, splits=8, seed=2, coop=-1)
    assert torch.equal(d, e)


def test_gemm_auto_splits_decode_shape():
    _case(9, 5120, 6144, 4)


def test_gemm_prefill_tiles():
    _case(300, 512, 1024, 4, splits=1)    # nt = 128, three token tiles, last one ragged
    _case(72, 256, 1024, 8, splits=2)     # nt = 80


def test_gemm_two_token_tiles_per_cta():
    """Long row runs of 4-bit weights: one widened weight block feeds two 128-row MMAs."""
    # (the launcher pairs tiles by itself only when one tile per CTA needs more than a wave: forced here)
    _case(512, 512, 1024, 4, splits=1, seed=11, mtiles=2)        # two pairs, whole
    _case(400, 300 + 4, 2048, 4, splits=1, seed=12, mtiles=2)    # last pair: second tile ragged (16 live rows), ragged N
    _case(700, 256, 512, 4, splits=1, seed=13, mtiles=2)         # M_pad = 768: three pairs, the last one half empty
    _case(512, 512, 1024, 8, splits=1, seed=14, mtiles=2)        # int8 weights keep one tile per CTA
    _case(2048, 40960, 256, 4, splits=1, seed=15)                # 160 x 16 single-tile CTAs: the launcher pairs by itself


def test_gemm_back_to_back_launches_keep_their_pipeline_phases():
    """Deep K loops in every ring configuration (odd and even stage counts, two and three operand
    buffers), launched back to back: the two transform groups take the k-blocks in turn and must
    never read a stage before its copy has landed."""
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(21)
    for (M, Nn, K, mt) in [(512, 512, 17408, 2), (128, 768, 8192, 0), (64, 512, 17408, 0), (80, 256, 5120, 0)]:
        w = torch.randn(Nn, K, generator=g) * 0.02
        x = torch.randn(M, K, generator=g)
        wq, ws = L.quantize_weight_rows(w, 4)
        aq, asc = L.quantize_act_rows(x)
        ref = R.gemm_i8(wq, ws, aq, asc).float()
        qw = F.QuantWeight.from_int(wq, ws, 4, dev)
        m_pad = L.padded_rows(M)
        qa = F.QuantAct(L.tile_act_int8(aq, m_pad).to(dev), torch.cat([asc, torch.zeros(m_pad - M)]).to(dev), M, K)
        outs = [F.gemm_i8(qw, qa, splits=1, mtiles=mt) for _ in range(20)]
        torch.cuda.synchronize()
        F.scratch(dev).check()
        tol = 1e-2 * ref.abs().max().item() + 1e-6
        for o in outs:
            assert (o.float().cpu() - ref).abs().max().item() <= tol


def test_gemm_int8_weights_on_cta_pairs_gives_the_bytes_of_the_one_cta_kernel():
    """`tcgen05.mma.cta_group::2`: a cluster of two CTAs per 512 x 256 output tile, each loading its token
    rows and its half of the weight tile.  Same integers, same scales, same rounding as the one-CTA kernel."""
    import ctypes as C
    from saber_engine_b200.ops import native as N
    dev = torch.device("cuda")
    lib = N.lib()
    for (M, Nn, K, seed) in [(512, 256, 256, 21), (1024, 512, 1024, 22), (700, 304, 2048, 23), (1300, 256, 512, 25), (2048, 1024, 5120, 24), (2048, 20480, 256, 26)]:
        g = torch.Generator().manual_seed(seed)
        w = torch.randn(Nn, K, generator=g) * 0.02
        x = torch.randn(M, K, generator=g)
        wq, ws = L.quantize_weight_rows(w, 8)
        aq, asc = L.quantize_act_rows(x)
        qw = F.QuantWeight.from_int(wq, ws, 8, dev)
        m_pad = L.round_up(M, 512)
        qa = F.QuantAct(L.tile_act_int8(aq, m_pad).to(dev), torch.cat([asc, torch.zeros(m_pad - M)]).to(dev), M, K)
        ldo = L.round_up(Nn, 8)
        one = torch.zeros(M, ldo, dtype=torch.bfloat16, device=dev)
        two = torch.zeros(M, ldo, dtype=torch.bfloat16, device=dev)
        p1 = F.gemm_params(qw, qa, one, F.scratch(dev), splits=1)
        N.check(lib.saber_gemm_i8_launch(C.byref(p1), 0, N.stream_handle()), "one-CTA gemm")
        p2 = F.gemm_params(qw, qa, two, F.scratch(dev), splits=1)
        assert lib.saber_gemm_w8_2sm_ok(C.byref(p2)) == 1
        N.check(lib.saber_gemm_w8_2sm_launch(C.byref(p2), 0, N.stream_handle()), "CTA-pair gemm")       # persistent pairs (default)
        three = torch.zeros(M, ldo, dtype=torch.bfloat16, device=dev)
        p3 = F.gemm_params(qw, qa, three, F.scratch(dev), splits=1)
        lib.saber_set_gemm_2sm_persistent(0)
        N.check(lib.saber_gemm_w8_2sm_launch(C.byref(p3), 0, N.stream_handle()), "CTA-pair gemm, one tile per cluster")
        lib.saber_set_gemm_2sm_persistent(1)
        torch.cuda.synchronize()
        F.scratch(dev).check()
        assert torch.equal(one, three)
        ref = R.gemm_i8(wq, ws, aq, asc).float()
        assert (one[:, :Nn].float().cpu() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-6
        assert torch.equal(one, two), (M, Nn, K, (one.float() - two.float()).abs().max().item())
