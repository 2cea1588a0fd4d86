"""Native block-scaled FP4 GEMM (tcgen05.mma kind::mxf4nvf4 / kind::mxf4, scales in tensor memory)
against the exact fp32 dequantisation of both operands."""
import pytest
import torch

from saber_engine_b200.ops import functional as F
from saber_engine_b200.pack import quant_fp4 as Q

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(fmt, M, N, K, splits, seed=0):
    torch.manual_seed(seed)
    w = torch.randn(N, K) * 0.05
    w[:, ::7] *= 4.0                                  # block scales that differ a lot inside a row
    x = torch.randn(M, K)
    x[:, 5::16] *= 3.0
    if fmt == 4:
        codes, bs, g = Q.quantize_nvfp4(w)
        qw = F.QuantWeight.from_nvfp4(codes, bs, g, device=DEV)
        wd = Q.dequant_nvfp4(codes, bs, g)
    else:
        codes, e = Q.quantize_mxfp4(w)
        qw = F.QuantWeight.from_mxfp4_native(codes, e, device=DEV)
        wd = Q.dequant_mxfp4(codes, e)
    qa = F.quant_act_fp4(x, fmt, device=DEV)
    vs = 16 if fmt == 4 else 32
    sf = (qa.sf.cpu(), None)
    # exact dequantisation of the activations from what the quantiser kept
    xc = Q.e2m1_decode(qa._codes)
    if fmt == 4:
        b = x.to(torch.bfloat16).float().reshape(M, K // 16, 16)
        bs_x = Q._e4m3_round((b.abs().amax(dim=-1) / 6.0 / qa._g[:, None]).clamp(max=448.0))
        xd = (xc.reshape(M, K // 16, 16) * (bs_x * qa._g[:, None])[..., None]).reshape(M, K)
    else:
        _, e_x = Q.quantize_mxfp4(x.to(torch.bfloat16).float())
        xd = Q.dequant_mxfp4(qa._codes, e_x)
    want = xd.double() @ wd.double().T
    got = F.gemm_i8(qw, qa, splits=splits).float().cpu()
    F.scratch(DEV).check()
    err = (got.double() - want).abs().max().item()
    ref = want.abs().max().item()
    assert got.shape == (M, N)
    assert err <= 6e-3 * ref, (fmt, M, N, K, splits, err, ref)


@pytest.mark.parametrize("fmt", [4, 5])
@pytest.mark.parametrize("M,N,K,splits", [(8, 512, 1024, 1), (64, 304, 2048, 1), (128, 256, 512, 1), (200, 512, 1024, 1),
                                           (40, 512, 2048, 2), (72, 768, 4096, 4)])
def test_fp4_gemm_matches_the_exact_dequantisation(fmt, M, N, K, splits):
    _case(fmt, M, N, K, splits, seed=M + K)
