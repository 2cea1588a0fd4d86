"""The device vision tower and the GEMM's bf16 mode against fp32 PyTorch restatements."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bf(x):
    return x.to(torch.bfloat16).float()


@pytest.mark.parametrize("M,N,K,epi", [(40, 1152, 1536, 0), (300, 4304, 1152, 1), (352, 1152, 4304, 3), (96, 520, 4608, 2)])
def test_bf16_gemm_mode_bias_activation_residual(M, N, K, epi):
    from saber_engine_b200.ops import functional as F, layouts as L, native as N_
    from saber_engine_b200.vision.tower_gpu import VisionTowerGPU, _Lin
    from saber_engine_b200.vision.tower import VisionConfig, _gelu_erf, _gelu_tanh
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(M + N)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    b = torch.randn(N, generator=g) * 0.1
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    res = torch.randn(M, N, generator=g).to(torch.bfloat16)
    lin = _Lin(w, b, dev)
    tw = VisionTowerGPU.__new__(VisionTowerGPU)                  # only the launch helpers are used
    tw.cfg, tw.dev, tw.launches = VisionConfig.tiny(), dev, 0
    m_pad = L.padded_rows(M)
    tw.a_buf = torch.zeros(lin.K_pad * 2 * m_pad, dtype=torch.uint8, device=dev)
    tw._rows(x.to(dev), M, K, lin.K_pad, m_pad)
    out = res.to(dev).clone() if epi == 3 else torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    tw._gemm(lin, M, m_pad, out, epi, res=out if epi == 3 else None)
    F.scratch(dev).check()
    y = _bf(x.float() @ w.float().t() + b)
    want = {0: y, 1: _gelu_tanh(y), 2: _gelu_erf(y), 3: _bf(y + res.float())}[epi]
    err = (out.float().cpu() - want).abs().max().item()
    assert err <= 2e-2 * want.abs().max().item() + 1e-3, err


def test_tower_matches_cpu_restatement():
    from saber_engine_b200.vision.tower import VisionConfig, VisionWeights, tower_reference
    from saber_engine_b200.vision.tower_gpu import VisionTowerGPU
    cfg = VisionConfig.tiny(depth=2, out_hidden=256)
    wts = VisionWeights.random(cfg, seed=5)
    grids = [(1, 8, 12), (1, 16, 16)]
    Lr = sum(t * h * w for t, h, w in grids)
    px = torch.randn(Lr, cfg.patch_row, generator=torch.Generator().manual_seed(1))
    tower = VisionTowerGPU(cfg, wts, "cuda")
    hid = tower.forward(px, grids, return_hidden=True).float().cpu()
    want_h = tower_reference(cfg, wts, px, grids, return_hidden=True)
    eh = (hid - want_h).abs().max().item()
    assert eh <= 3e-2 * want_h.abs().max().item(), eh
    got = tower.forward(px, grids).float().cpu()
    want = tower_reference(cfg, wts, px, grids)
    assert got.shape == (Lr // 4, 256)
    err = (got - want).abs().max().item()
    assert err <= 3e-2 * want.abs().max().item() + 1e-3, err
    assert tower.launches == 2 * (3 + 8 * cfg.depth) + 4        # two forwards; the first stops before the merger
