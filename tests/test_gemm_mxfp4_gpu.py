"""MXFP4 GEMM on the GPU (e2m1 weights folded to fp8 in the kernel, fp8 e4m3 per-token activations,
fp32 accumulation on the tensor cores) against the fp32 product of the same quantised operands."""
import pytest
import torch

from saber_engine_b200.ops import functional as F
from saber_engine_b200.pack import quant_fp4 as Q

pytestmark = pytest.mark.gpu


def _case(M, N, K, splits, seed=0):
    g = torch.Generator().manual_seed(seed)
    spread = torch.exp2(torch.randint(-5, 2, (N, K // 32), generator=g).float()).repeat_interleave(32, 1)
    w = torch.randn(N, K, generator=g) * spread * 0.02
    x = torch.randn(M, K, generator=g)
    codes, e = Q.quantize_mxfp4(w)
    shift, rs = Q.fold_mxfp4(codes, e)
    wq = Q.dequant_folded(codes, shift, rs)                    # what the kernel multiplies with
    aq, asc = Q.quantize_act_rows_e4m3(x)
    ref = (aq.float().double() @ wq.double().t()).float() * asc[:, None]
    qw = F.QuantWeight.from_mxfp4(codes, e, "cuda")
    qa = F.plain_quant(x.to(torch.bfloat16).cuda(), fp8=True)
    assert torch.allclose(qa.scale[:M].cpu(), asc)
    out = F.gemm_i8(qw, qa, splits=splits)
    torch.cuda.synchronize()
    F.scratch("cuda").check()
    got = out.float().cpu()
    err = (got - ref).abs().max().item()
    tol = 1e-2 * ref.abs().max().item() + 1e-6
    assert err <= tol, f"M={M} N={N} K={K} splits={splits}: max err {err} tol {tol}"
    return out


def test_mxfp4_direct_small_and_ragged():
    _case(5, 256, 512, 1)
    _case(9, 200, 2048, 1, seed=1)


def test_mxfp4_split_k_and_token_tiles():
    a = _case(40, 384, 4096, 4, seed=2)
    b = _case(40, 384, 4096, 4, seed=2)
    assert torch.equal(a, b)                                    # fixed split order: same bits every launch
    _case(300, 512, 1024, 1, seed=3)
    _case(72, 5120, 2048, 2, seed=4)


def test_mxfp4_two_token_tiles_per_cta():
    _case(512, 512, 1024, 1, seed=5)
    _case(900, 256, 2048, 1, seed=6)
