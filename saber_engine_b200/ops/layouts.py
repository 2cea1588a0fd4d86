"""Operand layouts of the tcgen05 integer GEMM and the quantisation laws, in plain torch (CPU or GPU).

Weights
    int8 image of one tile = 256 output rows x 128 bytes of K under the 128-byte swizzle
    (16-byte chunk index XOR (row & 7)); tiles are stored `[n_tile][k_block]`.  A W4 tile is 16 KiB:
    byte j = (image[j] >> 4) | (image[j + 16384] & 0xF0) where the image holds 16*w.
Activations
    `[k_block][M_pad][128]` int8 with the same swizzle keyed on (m & 7), plus one fp32 scale per row.

Quantisation laws (parity: `tools/pack/build_pack.py:22-40` for weights, `macaq_i8.h:1-13` for
activations, adapted): weights are symmetric per output row, int4 in [-8, 7] or int8 in [-127, 127];
activations are per-token dynamic int8, scale = amax / 127, q = clamp(rint(x * (127 / amax))).
"""
from __future__ import annotations

import math

import torch

TILE_N = 256          # output features per weight tile (the N side of one MMA)
TILE_K = 128


def round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def token_tile(M: int) -> int:
    """Token-tile width nt the GEMM uses for M rows: a multiple of 16, at most 128."""
    if M <= 128:
        return max(16, round_up(M, 16))
    return 128


def padded_rows(M: int) -> int:
    return round_up(M, token_tile(M))


# ------------------------------------------------------------------------------- weights
def quantize_weight_rows(w: torch.Tensor, bits: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Symmetric per-output-row quantisation. Returns (int8 values, fp32 row scale)."""
    w = w.float()
    qmax = 7.0 if bits == 4 else 127.0
    amax = w.abs().amax(dim=1).clamp_min(1e-12)
    scale = amax / qmax
    q = torch.round(w / scale[:, None]).clamp_(-qmax - (1 if bits == 4 else 0), qmax)
    return q.to(torch.int8), scale


def _swizzle_tiles(img: torch.Tensor) -> torch.Tensor:
    """img [..., R rows, 128 bytes] -> same shape with 16-byte chunks XOR-swizzled by row & 7."""
    lead = img.shape[:-2]
    R = img.shape[-2]
    x = img.reshape(*lead, R, 8, 16)
    rows = torch.arange(R, device=img.device) & 7
    chunks = torch.arange(8, device=img.device)
    src = (chunks[None, :] ^ rows[:, None])  # physical chunk c' holds logical chunk c' ^ r
    idx = src[..., None].expand(R, 8, 16)
    idx = idx.reshape((1,) * len(lead) + (R, 8, 16)).expand(*lead, R, 8, 16)
    return torch.gather(x, -2, idx).reshape(*lead, R, 128)


def tile_weight_int8(q: torch.Tensor) -> torch.Tensor:
    """int8 [N, K] -> uint8 tiles [N_pad/256, K/128, 32768] (the swizzled image of each tile)."""
    N, K = q.shape
    assert K % TILE_K == 0
    n_pad = round_up(N, TILE_N)
    if n_pad != N:
        q = torch.cat([q, torch.zeros(n_pad - N, K, dtype=q.dtype, device=q.device)], 0)
    t = q.view(torch.uint8).reshape(n_pad // TILE_N, TILE_N, K // 128, 128).permute(0, 2, 1, 3).contiguous()
    return _swizzle_tiles(t).reshape(n_pad // TILE_N, K // 128, TILE_N * 128)


def tile_weight_int4(q: torch.Tensor) -> torch.Tensor:
    """int8 values in [-8, 7], [N, K] -> packed W4 tiles [N_pad/256, K/128, 16384].

    The int8 image of a tile holds 16*w; packed byte j = (image[j] >> 4) | (image[j + 16384] & 0xF0),
    so the kernel widens a stage in place with two mask operations per word: low nibbles rebuild the
    first half of the image, high nibbles the second half.
    """
    img = tile_weight_int8((q.to(torch.int16) * 16).to(torch.int8))
    half = TILE_N * 128 // 2
    lo, hi = img[..., :half], img[..., half:]
    return ((lo >> 4) & 0x0F) | (hi & 0xF0)


def untile_weight_int8(tiles: torch.Tensor, N: int, K: int) -> torch.Tensor:
    """Inverse of tile_weight_int8 (for tests): tiles -> int8 [N, K]."""
    nt, kb, _ = tiles.shape
    t = _swizzle_tiles(tiles.reshape(nt, kb, TILE_N, 128))  # the XOR swizzle is an involution
    return t.permute(0, 2, 1, 3).reshape(nt * TILE_N, kb * 128)[:N, :K].contiguous().view(torch.int8)


def unpack_weight_int4(tiles: torch.Tensor, N: int, K: int) -> torch.Tensor:
    """Packed W4 tiles -> int8 values in [-8, 7], [N, K] (for tests and the CPU oracle)."""
    img = torch.cat([(tiles << 4) & 0xF0, tiles & 0xF0], dim=-1)
    w16 = untile_weight_int8(img, N, K)
    return (w16.to(torch.int16) // 16).to(torch.int8)


# ------------------------------------------------------------------------------- activations
def quantize_act_rows(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-token int8: (q int8 [M, K], scale fp32 [M]). Input is taken at bf16 precision."""
    x = x.to(torch.bfloat16).float()
    amax = x.abs().amax(dim=1)
    inv = torch.where(amax > 0, 127.0 / amax, torch.zeros_like(amax))
    q = torch.round(x * inv[:, None]).clamp_(-127, 127).to(torch.int8)
    return q, amax / 127.0


def tile_act_int8(q: torch.Tensor, m_pad: int) -> torch.Tensor:
    """int8 [M, K] -> tiled [K/128, M_pad, 128] with the (m & 7) chunk swizzle."""
    M, K = q.shape
    assert K % TILE_K == 0 and m_pad >= M
    if m_pad != M:
        q = torch.cat([q, torch.zeros(m_pad - M, K, dtype=q.dtype, device=q.device)], 0)
    x = q.reshape(m_pad, K // 128, 8, 16).permute(1, 0, 2, 3)  # [kb, m, chunk, 16]
    rows = torch.arange(m_pad, device=q.device) & 7
    chunks = torch.arange(8, device=q.device)
    src = chunks[None, :] ^ rows[:, None]
    idx = src[None, :, :, None].expand(K // 128, m_pad, 8, 16)
    return torch.gather(x, 2, idx).reshape(K // 128, m_pad, 128).contiguous()


def untile_act_int8(t: torch.Tensor, M: int) -> torch.Tensor:
    kb, m_pad, _ = t.shape
    x = t.reshape(kb, m_pad, 8, 16)
    rows = torch.arange(m_pad, device=t.device) & 7
    chunks = torch.arange(8, device=t.device)
    src = chunks[None, :] ^ rows[:, None]
    idx = src[None, :, :, None].expand(kb, m_pad, 8, 16)
    return torch.gather(x, 2, idx).permute(1, 0, 2, 3).reshape(m_pad, kb * 128)[:M].contiguous()


# ------------------------------------------------------------------------------- MXFP4 (folded to fp8 in the kernel)
MX_TILE_BYTES = 16384 + 1024


def tile_weight_mxfp4(codes: torch.Tensor, shift: torch.Tensor) -> torch.Tensor:
    """e2m1 codes uint8 [N, K] + per-(row, 32-block) shifts uint8 [N, K/32] -> uint8 tiles
    [N_pad/256, K/128, 17408].

    The first 16 KiB of a tile follow the int8 image's chunk order (row-major 128-byte rows, 16-byte
    chunks XOR-swizzled by row & 7): packed chunk `ci` carries the 16 codes of image chunk `ci`
    (row r < 128) and of image chunk `ci + 1024` (row r + 128) as four 32-bit words, word j = codes
    4j..4j+3 of row r in its low 16 bits (one nibble each) and of row r + 128 in its high 16 bits, so
    a 16-bit half is directly the selector of one byte-permute.  The last 1 KiB holds the shifts,
    [256 rows][4 blocks]."""
    N, K = codes.shape
    img = tile_weight_int8(codes.to(torch.int8)).view(torch.uint8)            # [nt, kb, 32768] one code per byte
    nt, kb, _ = img.shape
    lo = img[..., :16384].reshape(nt, kb, 1024, 4, 4).to(torch.int32)         # chunk, word, code
    hi = img[..., 16384:].reshape(nt, kb, 1024, 4, 4).to(torch.int32)
    b0 = lo[..., 0] | (lo[..., 1] << 4)
    b1 = lo[..., 2] | (lo[..., 3] << 4)
    b2 = hi[..., 0] | (hi[..., 1] << 4)
    b3 = hi[..., 2] | (hi[..., 3] << 4)
    packed = torch.stack([b0, b1, b2, b3], dim=-1).to(torch.uint8).reshape(nt, kb, 16384)
    n_pad = nt * TILE_N
    sh = torch.zeros(n_pad, K // 32, dtype=torch.uint8, device=codes.device)
    sh[:N] = shift
    sh = sh.reshape(nt, TILE_N, kb, 4).permute(0, 2, 1, 3).reshape(nt, kb, 1024)
    return torch.cat([packed, sh], dim=-1).contiguous()


def untile_weight_mxfp4(tiles: torch.Tensor, N: int, K: int):
    """Inverse of tile_weight_mxfp4 (tests, CPU oracle): -> (codes uint8 [N, K], shift uint8 [N, K/32])."""
    nt, kb, _ = tiles.shape
    packed = tiles[..., :16384].reshape(nt, kb, 1024, 4, 4).to(torch.int32)      # chunk, word, byte
    lo = torch.stack([packed[..., 0] & 15, packed[..., 0] >> 4, packed[..., 1] & 15, packed[..., 1] >> 4], dim=-1)
    hi = torch.stack([packed[..., 2] & 15, packed[..., 2] >> 4, packed[..., 3] & 15, packed[..., 3] >> 4], dim=-1)
    img = torch.cat([lo.reshape(nt, kb, 16384), hi.reshape(nt, kb, 16384)], dim=-1).to(torch.uint8)
    codes = untile_weight_int8(img, N, K).view(torch.uint8)
    sh = tiles[..., 16384:].reshape(nt, kb, TILE_N, 4).permute(0, 2, 1, 3).reshape(nt * TILE_N, kb * 4)
    return codes, sh[:N].contiguous()


# ------------------------------------------------------------------------------- Hadamard rotation
def hadamard32_matrix(device=None) -> torch.Tensor:
    """Orthonormal 32 x 32 Hadamard matrix (Sylvester order, entries +-1/sqrt(32))."""
    h = torch.ones(1, 1, device=device)
    for _ in range(5):
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return h / math.sqrt(32.0)


def hadamard32_rows(x: torch.Tensor, sign: torch.Tensor) -> torch.Tensor:
    """x [M, K] -> every 32-block of (x * sign) times the orthonormal Hadamard matrix (the rotation
    the row producers apply before they quantise; H is symmetric, so the same call rotates weights)."""
    M, K = x.shape
    h = hadamard32_matrix(x.device)
    return ((x.float() * sign.float()).reshape(M, K // 32, 32) @ h).reshape(M, K)


# ------------------------------------------------------------------------------- paired gate | up tiles
def pair_gate_up_int4(tiles: torch.Tensor, scale: torch.Tensor, inter: int):
    """Packed W4 tiles of a merged [gate rows; up rows] linear (2 * inter rows, inter a multiple of
    128) -> tiles whose rows 0-127 are gate features [128 t, 128 t + 128) and rows 128-255 the up
    features of the same indices, so that one CTA of the GEMM owns whole (gate, up) pairs.  A packed
    tile keeps rows r and r + 128 in the two nibbles of one byte and the swizzle only looks at
    r & 7, so the regrouping is a nibble shuffle between tiles.  Returns (tiles, scale)."""
    assert inter % 128 == 0 and tiles.shape[0] * TILE_N == 2 * inter, (tiles.shape, inter)
    nb = inter // 128
    blocks = torch.stack([tiles & 0x0F, tiles >> 4], dim=1).reshape(2 * nb, *tiles.shape[1:])   # block b = rows [128 b, 128 b + 128)
    out = blocks[:nb] | (blocks[nb:] << 4)
    sc = torch.cat([scale[:inter].reshape(nb, 128), scale[inter:2 * inter].reshape(nb, 128)], dim=1).reshape(-1)
    return out.contiguous(), sc.contiguous()


def unpair_gate_up_int4(tiles: torch.Tensor, scale: torch.Tensor, inter: int):
    """Inverse of pair_gate_up_int4."""
    nb = inter // 128
    assert tiles.shape[0] == nb
    blocks = torch.cat([tiles & 0x0F, tiles >> 4], dim=0)            # [gate blocks; up blocks] = canonical block order
    pairs = blocks.reshape(nb, 2, *tiles.shape[1:])
    out = pairs[:, 0] | (pairs[:, 1] << 4)
    s2 = scale.reshape(nb, 2, 128)
    sc = torch.cat([s2[:, 0].reshape(-1), s2[:, 1].reshape(-1)])
    return out.contiguous(), sc.contiguous()


# ------------------------------------------------------------------------------- KV pages in core-matrix order
def kv_pages_to_core(cache: torch.Tensor) -> torch.Tensor:
    """Paged KV pool uint8 [blocks, kv heads, 2, 16, 256] in the plain [token][dim] page order -> the
    page order the tcgen05 attention multiplies in place (same shape and bytes per page):
    K [2 key groups][16 dim chunks][8 keys][16 dims], V [32 dim groups][8 dims][16 keys]."""
    nb, nkv = cache.shape[:2]
    k = cache[:, :, 0].reshape(nb, nkv, 2, 8, 16, 16).permute(0, 1, 2, 4, 3, 5).reshape(nb, nkv, 4096)
    v = cache[:, :, 1].reshape(nb, nkv, 16, 32, 8).permute(0, 1, 3, 4, 2).reshape(nb, nkv, 4096)
    return torch.stack([k, v], dim=2).reshape(nb, nkv, 2, 16, 256).contiguous()


def kv_pages_from_core(cache: torch.Tensor) -> torch.Tensor:
    """Inverse of kv_pages_to_core."""
    nb, nkv = cache.shape[:2]
    k = cache[:, :, 0].reshape(nb, nkv, 2, 16, 8, 16).permute(0, 1, 2, 4, 3, 5).reshape(nb, nkv, 16, 256)
    v = cache[:, :, 1].reshape(nb, nkv, 32, 8, 16).permute(0, 1, 4, 2, 3).reshape(nb, nkv, 16, 256)
    return torch.stack([k, v], dim=2).contiguous()


# ------------------------------------------------------------------------------- native FP4 (block-scaled MMA)
FP4_KB = 256          # values per k-block: a 128-byte row of packed e2m1 pairs


def pack_e2m1(codes: torch.Tensor) -> torch.Tensor:
    """uint8 codes [.., K] (one per byte) -> packed bytes [.., K/2]: the even value in the low nibble."""
    return (codes[..., 0::2] & 0x0F) | ((codes[..., 1::2] & 0x0F) << 4)


def unpack_e2m1(packed: torch.Tensor) -> torch.Tensor:
    out = torch.empty(*packed.shape[:-1], packed.shape[-1] * 2, dtype=torch.uint8, device=packed.device)
    out[..., 0::2] = packed & 0x0F
    out[..., 1::2] = packed >> 4
    return out


def scale_atoms(sf: torch.Tensor, per_kb: int) -> torch.Tensor:
    """Block scales as the 512-byte atoms the tensor core's scale copy moves: sf uint8 [R, n_sf] with R
    a multiple of 128 and n_sf a multiple of `per_kb` (scales per row and k-block, itself a multiple of
    4) -> uint8 [n_sf / per_kb, R / 128, per_kb / 4, 512]; inside an atom (128 rows x 4 scales) the byte
    of (row r, scale s) sits at (r % 32) * 16 + (r // 32) * 4 + s."""
    R, n_sf = sf.shape
    assert R % 128 == 0 and n_sf % per_kb == 0 and per_kb % 4 == 0
    x = sf.reshape(R // 128, 4, 32, n_sf // per_kb, per_kb // 4, 4)      # [chunk, r // 32, r % 32, kb, atom, s]
    return x.permute(3, 0, 4, 2, 1, 5).contiguous().reshape(n_sf // per_kb, R // 128, per_kb // 4, 512)


def tile_weight_fp4(codes: torch.Tensor, sf: torch.Tensor, vs: int) -> torch.Tensor:
    """e2m1 codes uint8 [N, K] + block scales uint8 [N, K / vs] (vs = 16: ue4m3, 32: ue8m0) -> tiles uint8
    [N_pad/256, K/256, 32768 + SF]: the swizzled image of the packed 256 x 128-byte tile, then its scale
    atoms in the order the kernel copies them: [atom along K][128-row chunk][512]."""
    N, K = codes.shape
    assert K % FP4_KB == 0
    n_pad = round_up(N, TILE_N)
    if n_pad != N:
        codes = torch.cat([codes, torch.zeros(n_pad - N, K, dtype=codes.dtype, device=codes.device)], 0)
        sf = torch.cat([sf, torch.zeros(n_pad - N, sf.shape[1], dtype=sf.dtype, device=sf.device)], 0)
    img = tile_weight_int8(pack_e2m1(codes).view(torch.int8))                  # [n_tiles, K/256, 32768]
    per_kb = FP4_KB // vs
    at = scale_atoms(sf, per_kb)                                                # [K/256, n_pad/128, per_kb/4, 512]
    at = at.reshape(K // FP4_KB, n_pad // TILE_N, 2, per_kb // 4, 512).permute(1, 0, 3, 2, 4)   # [tile, kb, atom, chunk, 512]
    return torch.cat([img, at.reshape(n_pad // TILE_N, K // FP4_KB, -1)], dim=-1).contiguous()


def tile_act_fp4(codes: torch.Tensor, sf: torch.Tensor, vs: int, m_pad: int):
    """e2m1 codes uint8 [M, K] + block scales uint8 [M, K / vs] -> (packed rows uint8 [K/256, M_pad, 128] in
    the activation swizzle, scale atoms uint8 [K/256, ceil(M_pad/128), (256/vs)/4 * 512]); rows past M are zero."""
    M, K = codes.shape
    q = tile_act_int8(pack_e2m1(codes).view(torch.int8), m_pad).view(torch.uint8)
    r_pad = round_up(m_pad, 128)
    full = torch.zeros(r_pad, sf.shape[1], dtype=torch.uint8, device=sf.device)
    full[:M] = sf
    per_kb = FP4_KB // vs
    at = scale_atoms(full, per_kb)
    return q, at.reshape(K // FP4_KB, r_pad // 128, -1).contiguous()


def untile_scale_atoms(at: torch.Tensor) -> torch.Tensor:
    """Inverse of scale_atoms: uint8 [n_kb, R/128, per_kb/4, 512] -> [R, n_kb * per_kb]."""
    n_kb, chunks, atoms, _ = at.shape
    x = at.reshape(n_kb, chunks, atoms, 32, 4, 4).permute(1, 4, 3, 0, 2, 5)       # [chunk, r // 32, r % 32, kb, atom, s]
    return x.reshape(chunks * 128, n_kb * atoms * 4).contiguous()


def untile_weight_fp4(tiles: torch.Tensor, N: int, K: int, vs: int):
    """Inverse of tile_weight_fp4 (tests, the CPU oracle): -> (codes uint8 [N, K], block scales uint8 [N, K / vs])."""
    n_tiles, n_kb, _ = tiles.shape
    img = tiles[..., :32768].contiguous()
    codes = unpack_e2m1(untile_weight_int8(img, n_tiles * TILE_N, K // 2).view(torch.uint8))[:N]
    per_kb = FP4_KB // vs
    at = tiles[..., 32768:].reshape(n_tiles, n_kb, per_kb // 4, 2, 512).permute(1, 0, 3, 2, 4)    # [kb, tile, chunk, atom, 512]
    sf = untile_scale_atoms(at.reshape(n_kb, n_tiles * 2, per_kb // 4, 512).contiguous())
    return codes.contiguous(), sf[:N].contiguous()


def untile_act_fp4(q: torch.Tensor, sf_atoms: torch.Tensor, M: int, vs: int):
    """Inverse of tile_act_fp4: -> (codes uint8 [M, K], block scales uint8 [M, K / vs])."""
    codes = unpack_e2m1(untile_act_int8(q.view(torch.int8), M).view(torch.uint8))
    n_kb, chunks, _ = sf_atoms.shape
    per_kb = FP4_KB // vs
    sf = untile_scale_atoms(sf_atoms.reshape(n_kb, chunks, per_kb // 4, 512))
    return codes, sf[:M].contiguous()
