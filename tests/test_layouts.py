"""CPU tests of the operand layouts and quantisation laws."""
import torch

from saber_engine_b200.ops import layouts as L


def test_weight_int8_tile_roundtrip():
    q = torch.randint(-127, 128, (200, 384), dtype=torch.int8)
    t = L.tile_weight_int8(q)
    assert t.shape == (1, 3, 32768)
    assert torch.equal(L.untile_weight_int8(t, 200, 384), q)


def test_weight_int4_pack_roundtrip_and_widen_law():
    q = torch.randint(-8, 8, (300, 256), dtype=torch.int8)
    p = L.tile_weight_int4(q)
    assert p.shape == (2, 2, 16384) and p.dtype == torch.uint8
    assert torch.equal(L.unpack_weight_int4(p, 300, 256), q)
    # the kernel's widening: low half = (byte << 4) & 0xF0, high half = byte & 0xF0, image = 16*w
    img = torch.cat([(p << 4) & 0xF0, p & 0xF0], -1)
    assert torch.equal(L.untile_weight_int8(img, 300, 256).to(torch.int16), q.to(torch.int16) * 16)


def test_swizzle_places_chunk_at_xor_position():
    q = torch.zeros(256, 128, dtype=torch.int8)
    q[5, 16 * 3] = 77            # row 5, logical chunk 3
    t = L.tile_weight_int8(q)[0, 0]
    off = 5 * 128 + ((3 ^ 5) * 16)
    assert t[off].item() == 77 and int((t != 0).sum()) == 1


def test_act_tile_roundtrip_and_quant_law():
    x = torch.randn(9, 256)
    q, s = L.quantize_act_rows(x)
    assert q.abs().max() <= 127
    xb = x.to(torch.bfloat16).float()
    assert torch.allclose(q.float() * s[:, None], xb, atol=float(s.max()) * 0.51)
    t = L.tile_act_int8(q, 16)
    assert t.shape == (2, 16, 128)
    assert torch.equal(L.untile_act_int8(t, 9), q)
    assert L.token_tile(9) == 16 and L.token_tile(72) == 80 and L.token_tile(4096) == 128


def test_negative_control_nibble_swap_is_caught():
    q = torch.randint(-8, 8, (128, 128), dtype=torch.int8)
    p = L.tile_weight_int4(q)
    swapped = ((p << 4) & 0xF0) | ((p >> 4) & 0x0F)   # nibble-swapped pack must not decode
    assert not torch.equal(L.unpack_weight_int4(swapped, 128, 128), q)
