"""FP4 pack formats on the CPU: quantisers, exact dequantisers, the MXFP4 -> fp8 fold and its tile
layout, NVFP4 -> MXFP4 requantisation."""
import torch

from saber_engine_b200.ops import layouts as L
from saber_engine_b200.pack import quant_fp4 as Q


def _w(n=300, k=256, seed=0):
    g = torch.Generator().manual_seed(seed)
    spread = torch.exp2(torch.randint(-6, 3, (n, k // 32), generator=g).float()).repeat_interleave(32, 1)
    return torch.randn(n, k, generator=g) * spread * 0.02


def test_e2m1_grid_and_rounding():
    x = torch.tensor([0.0, 0.2, 0.25, 0.3, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.6, -6.5])
    got = Q.e2m1_decode(Q.e2m1_encode(x))
    assert got.tolist() == [0.0, 0.0, 0.0, 0.5, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, -0.5, -6.0]


def test_mxfp4_roundtrip_error_and_scale_law():
    w = _w()
    codes, e = Q.quantize_mxfp4(w)
    assert codes.max() < 16 and e.shape == (300, 8)
    dq = Q.dequant_mxfp4(codes, e)
    assert ((dq - w).pow(2).mean().sqrt() / w.pow(2).mean().sqrt()) < 0.15
    # every block's largest magnitude lands on the top binade of e2m1 (4 or 6)
    top = (codes & 7).reshape(300, 8, 32).amax(-1)
    assert (top >= 6).all()


def test_fold_is_exact_within_ten_binades_and_flushes_below():
    w = _w()
    codes, e = Q.quantize_mxfp4(w)
    shift, rs = Q.fold_mxfp4(codes, e)
    assert int(shift.max()) <= 10
    assert torch.equal(Q.dequant_folded(codes, shift, rs), Q.dequant_mxfp4(codes, e))
    # a block 2^12 below the row's largest: 0.5 (field 11) and 1.0 / 1.5 (field 12) are flushed, 2..6 survive
    codes2 = torch.tensor([[1, 2, 3, 4, 5, 6, 7, 0] * 4 + [7] * 32], dtype=torch.uint8)
    e2 = torch.tensor([[100, 112]], dtype=torch.uint8)
    sh2, rs2 = Q.fold_mxfp4(codes2, e2)
    assert sh2.tolist() == [[12, 0]]
    got = Q.dequant_folded(codes2, sh2, rs2)[0, :8]
    want = Q.dequant_mxfp4(codes2, e2)[0, :8]
    assert got[:3].abs().sum() == 0 and torch.equal(got[3:], want[3:])


def test_mxfp4_tile_layout_positions():
    w = _w(260, 256, seed=1)
    codes, e = Q.quantize_mxfp4(w)
    shift, _ = Q.fold_mxfp4(codes, e)
    t = L.tile_weight_mxfp4(codes, shift)
    assert t.shape == (2, 2, L.MX_TILE_BYTES)
    # row 5 and row 133 of tile 0, k-block 1, logical chunk 3 (K 176..191 of the block = 128 + 48..63)
    r, kb, lc = 5, 1, 3
    pc = lc ^ (r & 7)
    ci = r * 8 + pc
    words = t[0, kb, ci * 16: ci * 16 + 16].view(torch.int32)
    for j in range(4):
        wv = int(words[j]) & 0xFFFFFFFF
        lo = [(wv >> (4 * i)) & 15 for i in range(4)]
        hi = [(wv >> (16 + 4 * i)) & 15 for i in range(4)]
        k0 = kb * 128 + lc * 16 + 4 * j
        assert lo == codes[r, k0:k0 + 4].tolist()
        assert hi == codes[r + 128, k0:k0 + 4].tolist()
    assert int(t[0, kb, 16384 + r * 4 + (lc >> 1)]) == int(shift[r, kb * 4 + (lc >> 1)])
    assert int(t[1, kb, 16384 + 3 * 4 + 2]) == int(shift[256 + 3, kb * 4 + 2])


def test_nvfp4_roundtrip_and_requant_to_mxfp4():
    w = _w(64, 128, seed=2)
    codes, bs, g = Q.quantize_nvfp4(w)
    dq = Q.dequant_nvfp4(codes, bs, g)
    assert ((dq - w).pow(2).mean().sqrt() / w.pow(2).mean().sqrt()) < 0.13
    assert torch.equal(bs, bs.to(torch.float8_e4m3fn).float())          # block scales are e4m3 numbers
    c2, e2 = Q.nvfp4_to_mxfp4(codes, bs, g)
    d2 = Q.dequant_mxfp4(c2, e2)
    assert ((d2 - dq).pow(2).mean().sqrt() / dq.pow(2).mean().sqrt()) < 0.12


def test_fp8_activation_law():
    x = torch.randn(5, 128)
    q, s = Q.quantize_act_rows_e4m3(x)
    assert torch.allclose(s, x.to(torch.bfloat16).float().abs().amax(1) / 448.0)
    assert (q.float().abs().amax(1) == 448.0).all()
