"""FP4 weight formats: MXFP4 (e2m1 values, one e8m0 scale per 32) and NVFP4 (e2m1 values, one e4m3
scale per 16, one fp32 scale per tensor); quantisers, exact dequantisers, and the MXFP4 -> fp8 fold
the GEMM kernel runs on.

The fold: inside one output row every 32-block's power-of-two scale is expressed as a right shift
k >= 0 against the row's largest block exponent (`wref`); an e2m1 magnitude times 2^-k is exactly an
e4m3 number as long as its e4m3 exponent field stays >= 1, so the kernel widens a nibble to an fp8
byte with one table lookup per four weights (the table is the e4m3 image of the eight e2m1
magnitudes, shifted by k) and multiplies fp8 x fp8 on the tensor cores; the epilogue applies
2^wref per output feature and the per-token activation scale.  Magnitudes that would need an
e4m3 exponent field of 0 are flushed to zero (they are >= 2^10 below the row's largest block).

Parity: `crates/saber-kernels/hip/mxfp4_common.h:20-45` (e8m0 block scale folded to e4m3 via kMag,
epilogue acc * 2^(wref-127) * As[m]), `tools/pack/build_pack.py:22-40` (NVFP4 -> MXFP4 requant),
`crates/saber-kernels/hip/moe_fn148.hip:3-6` (NVFP4: e2m1 + e4m3/16 + f32 global).
"""
from __future__ import annotations

import torch

E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
# e4m3 bytes of the eight e2m1 magnitudes scaled by 2^5: 0.5 -> exponent field 11 ... 6 -> field 14
FOLD_BASE = (0x00, 0x58, 0x60, 0x64, 0x68, 0x6C, 0x70, 0x74)
FOLD_EXP = (0, 11, 12, 12, 13, 13, 14, 14)
FOLD_GAIN_LOG2 = 5            # the folded byte decodes to magnitude * 2^(5 - k)


def e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest (ties to even code) e2m1 codes (uint8, bit 3 = sign) of values in [-6, 6]."""
    mag = x.abs().clamp(max=6.0)
    grid = E2M1_VALUES.to(x.device)
    d = (mag[..., None] - grid).abs()
    idx = d.argmin(dim=-1)
    # ties: prefer the even code (argmin takes the first = lower; adjust where the upper is even)
    lo = idx.clamp(max=6)
    tie = (d.gather(-1, lo[..., None]).squeeze(-1) == d.gather(-1, (lo + 1)[..., None]).squeeze(-1)) & (idx == lo)
    idx = torch.where(tie & (lo % 2 == 1), lo + 1, idx)
    return (idx.to(torch.uint8) | ((x < 0).to(torch.uint8) << 3))


def e2m1_decode(codes: torch.Tensor) -> torch.Tensor:
    v = E2M1_VALUES.to(codes.device)[(codes & 7).long()]
    return torch.where((codes & 8) != 0, -v, v)


# ----------------------------------------------------------------------------------------- MXFP4
def quantize_mxfp4(w: torch.Tensor):
    """fp32 [N, K] (K % 32 == 0) -> (codes uint8 [N, K], e8m0 uint8 [N, K/32])."""
    N, K = w.shape
    b = w.float().reshape(N, K // 32, 32)
    amax = b.abs().amax(dim=-1)
    e = torch.floor(torch.log2(amax.clamp_min(2.0 ** -126))) - 2          # so that amax / 2^e is in [4, 8)
    e = e.clamp(-127, 127)
    scale = torch.exp2(e)
    codes = e2m1_encode(b / scale[..., None]).reshape(N, K)
    return codes, (e + 127).to(torch.uint8)


def dequant_mxfp4(codes: torch.Tensor, e8m0: torch.Tensor) -> torch.Tensor:
    N, K = codes.shape
    scale = torch.exp2(e8m0.float() - 127.0)
    return (e2m1_decode(codes).reshape(N, K // 32, 32) * scale[..., None]).reshape(N, K)


def fold_mxfp4(codes: torch.Tensor, e8m0: torch.Tensor):
    """-> (shift uint8 [N, K/32], row_scale fp32 [N]): value = fold_byte_value * row_scale, where the
    fold byte of magnitude m at shift k decodes to m * 2^(5 - k) (or 0 when flushed)."""
    wref = e8m0.to(torch.int32).amax(dim=1, keepdim=True)
    shift = (wref - e8m0.to(torch.int32)).clamp(max=15).to(torch.uint8)
    row_scale = torch.exp2(wref.squeeze(1).float() - 127.0 - FOLD_GAIN_LOG2)
    return shift, row_scale


def dequant_folded(codes: torch.Tensor, shift: torch.Tensor, row_scale: torch.Tensor) -> torch.Tensor:
    """What the GEMM kernel multiplies with: the folded fp8 value (flush included) times row_scale."""
    N, K = codes.shape
    mag = (codes & 7).long().reshape(N, K // 32, 32)
    k = shift.long()[..., None]
    exp = torch.tensor(FOLD_EXP, device=codes.device)[mag]
    alive = exp > k
    val = E2M1_VALUES.to(codes.device)[mag] * torch.exp2((FOLD_GAIN_LOG2 - k).float())
    val = torch.where(alive, val, torch.zeros_like(val))
    sign = torch.where((codes & 8).reshape(N, K // 32, 32) != 0, -1.0, 1.0)
    return (val * sign).reshape(N, K) * row_scale[:, None]


# ----------------------------------------------------------------------------------------- NVFP4
def _e4m3_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float8_e4m3fn).float()


def quantize_nvfp4(w: torch.Tensor):
    """fp32 [N, K] (K % 16 == 0) -> (codes uint8 [N, K], block scale e4m3-as-float [N, K/16], global fp32)."""
    N, K = w.shape
    b = w.float().reshape(N, K // 16, 16)
    g = (w.abs().max() / (6.0 * 448.0)).clamp_min(1e-30)
    bs = _e4m3_round((b.abs().amax(dim=-1) / 6.0 / g).clamp(max=448.0))
    denom = (bs * g).clamp_min(1e-30)
    codes = e2m1_encode(b / denom[..., None]).reshape(N, K)
    return codes, bs, g.float()


def dequant_nvfp4(codes: torch.Tensor, block_scale: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    N, K = codes.shape
    return (e2m1_decode(codes).reshape(N, K // 16, 16) * (block_scale * g)[..., None]).reshape(N, K)


def nvfp4_to_mxfp4(codes: torch.Tensor, block_scale: torch.Tensor, g: torch.Tensor):
    """Requantise an NVFP4 tensor to MXFP4 (the pack builder's NVFP4 -> MXFP4 transform)."""
    return quantize_mxfp4(dequant_nvfp4(codes, block_scale, g))


# ------------------------------------------------------------------------- activations (fp8 e4m3)
def quantize_act_rows_e4m3(x: torch.Tensor):
    """Per-token fp8: (q float8 values as fp32 [M, K], scale fp32 [M]); scale = amax / 448."""
    x = x.to(torch.bfloat16).float()
    amax = x.abs().amax(dim=1)
    inv = torch.where(amax > 0, 448.0 / amax, torch.zeros_like(amax))
    q = (x * inv[:, None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q, amax / 448.0
