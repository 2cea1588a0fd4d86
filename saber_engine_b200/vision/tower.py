"""The vision tower: configuration, weights, host metadata (position-table gather, 2-D rotary tables)
and the CPU restatement (fp32 arithmetic with bf16 rounding where the device kernels round).

Ops: patch embed (a GEMM of the patch rows against the Conv3d weight viewed [width, 1536]) ->
bilinear gather of the learned 48 x 48 position table added to the rows -> `depth` blocks
`x += proj(attn(rope(qkv(LN1(x)))))`, `x += fc2(gelu_tanh(fc1(LN2(x))))` (LayerNorm with bias,
non-causal attention inside each image, 2-D rotary embedding with neox halves) -> merger
`LN -> view [L/4, 4 * width] -> fc1 -> GELU(erf) -> fc2 -> [L/4, out]`.

Parity: `crates/saber-kernels/hip/vision.hip:1-30` (the op list and its rounding points).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch


@dataclass(frozen=True)
class VisionConfig:
    width: int = 1152
    heads: int = 16
    depth: int = 27
    mlp: int = 4304
    patch_row: int = 1536            # 3 * 2 * 16 * 16
    out_hidden: int = 5120
    pos_grid: int = 48
    merge: int = 2
    eps: float = 1e-6
    rope_theta: float = 10000.0

    @property
    def head_dim(self) -> int:
        return self.width // self.heads

    @staticmethod
    def qwen38(out_hidden: int = 5120) -> "VisionConfig":
        return VisionConfig(out_hidden=out_hidden)

    @staticmethod
    def tiny(depth: int = 2, out_hidden: int = 256) -> "VisionConfig":
        """Same head geometry (16 x 72), fewer blocks: for tests."""
        return VisionConfig(depth=depth, out_hidden=out_hidden)


@dataclass
class VisionWeights:
    """bf16 matrices [out, in], fp32 biases and LayerNorm parameters."""
    patch_w: torch.Tensor
    patch_b: torch.Tensor
    pos_table: torch.Tensor           # bf16 [pos_grid^2, width]
    blocks: list                      # dicts: ln1_w ln1_b qkv_w qkv_b proj_w proj_b ln2_w ln2_b fc1_w fc1_b fc2_w fc2_b
    merger: dict                      # ln_w ln_b fc1_w fc1_b fc2_w fc2_b

    @staticmethod
    def random(cfg: VisionConfig, seed: int = 0, std: float = 0.02) -> "VisionWeights":
        g = torch.Generator().manual_seed(seed)

        def mat(o, i, s=std):
            return (torch.randn(o, i, generator=g) * s).to(torch.bfloat16)

        def vec(n, s=0.02, base=0.0):
            return (torch.randn(n, generator=g) * s + base).float()
        W, Hm = cfg.width, cfg.mlp
        blocks = []
        for _ in range(cfg.depth):
            blocks.append(dict(ln1_w=vec(W, 0.05, 1.0), ln1_b=vec(W), qkv_w=mat(3 * W, W), qkv_b=vec(3 * W),
                               proj_w=mat(W, W), proj_b=vec(W), ln2_w=vec(W, 0.05, 1.0), ln2_b=vec(W),
                               fc1_w=mat(Hm, W), fc1_b=vec(Hm), fc2_w=mat(W, Hm), fc2_b=vec(W)))
        M4 = W * cfg.merge * cfg.merge
        merger = dict(ln_w=vec(W, 0.05, 1.0), ln_b=vec(W), fc1_w=mat(M4, M4), fc1_b=vec(M4),
                      fc2_w=mat(cfg.out_hidden, M4), fc2_b=vec(cfg.out_hidden))
        return VisionWeights(mat(W, cfg.patch_row), vec(W), mat(cfg.pos_grid ** 2, W, 0.1), blocks, merger)


# --------------------------------------------------------------------------------- host metadata
def _merge_order(a: np.ndarray, t: int, h: int, w: int, m: int) -> np.ndarray:
    """[h * w, ...] row-major over the patch grid -> the tower's row order (h/m, w/m, m, m), repeated t times."""
    tail = a.shape[1:]
    x = a.reshape(h // m, m, w // m, m, *tail).transpose(0, 2, 1, 3, *range(4, 4 + len(tail)))
    x = x.reshape(h * w, *tail)
    return np.concatenate([x] * t, axis=0) if t > 1 else x


def pos_gather_table(grids: Sequence[tuple], cfg: VisionConfig):
    """Per patch row: four indices into the position table and four bilinear weights (fp32)."""
    G, idx_all, wt_all = cfg.pos_grid, [], []
    for t, h, w in grids:
        hs = np.linspace(0, G - 1, h, dtype=np.float32)
        ws = np.linspace(0, G - 1, w, dtype=np.float32)
        hf, wf = hs.astype(np.int64), ws.astype(np.int64)
        hc, wc = np.minimum(hf + 1, G - 1), np.minimum(wf + 1, G - 1)
        dh, dw = hs - hf, ws - wf
        idx = np.stack([(hf[:, None] * G + wf[None]), (hf[:, None] * G + wc[None]),
                        (hc[:, None] * G + wf[None]), (hc[:, None] * G + wc[None])], axis=-1).reshape(h * w, 4)
        wt = np.stack([(1 - dh)[:, None] * (1 - dw)[None], (1 - dh)[:, None] * dw[None],
                       dh[:, None] * (1 - dw)[None], dh[:, None] * dw[None]], axis=-1).reshape(h * w, 4)
        idx_all.append(_merge_order(idx.astype(np.int32), t, h, w, cfg.merge))
        wt_all.append(_merge_order(wt.astype(np.float32), t, h, w, cfg.merge))
    return np.concatenate(idx_all, 0), np.concatenate(wt_all, 0)


def rope_tables(grids: Sequence[tuple], cfg: VisionConfig):
    """cos / sin fp32 [L, head_dim / 2]: the first quarter of the head's pairs turns with the patch's
    row index, the second with its column index."""
    quarter = cfg.head_dim // 4
    inv = 1.0 / (cfg.rope_theta ** (np.arange(0, 2 * quarter, 2, dtype=np.float32) / (2 * quarter)))
    ang_all = []
    for t, h, w in grids:
        hi, wi = np.meshgrid(np.arange(h), np.arange(w), indexing="ij")
        hw = np.stack([hi.reshape(-1), wi.reshape(-1)], axis=-1).astype(np.float32)     # [h*w, 2]
        hw = _merge_order(hw, t, h, w, cfg.merge)
        ang_all.append(np.concatenate([hw[:, :1] * inv[None], hw[:, 1:] * inv[None]], axis=1))
    ang = np.concatenate(ang_all, 0).astype(np.float32)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def attn_blocks(grids: Sequence[tuple], rows_per_block: int = 64) -> np.ndarray:
    """int32 [n_blocks, 4]: {first row of the image, rows of the image, first query (relative), 0}."""
    out, row = [], 0
    for t, h, w in grids:
        n = t * h * w
        for q0 in range(0, n, rows_per_block):
            out.append((row, n, q0, 0))
        row += n
    return np.asarray(out, dtype=np.int32).reshape(-1, 4)


# --------------------------------------------------------------------------------- CPU restatement
def _bf(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).float()


def _linear(x, w, b):
    return _bf(x @ w.float().t() + b)


def _ln(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return _bf((x - mu) * torch.rsqrt(var + eps) * w + b)


def _gelu_tanh(x):
    return _bf(0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3))))


def _gelu_erf(x):
    return _bf(0.5 * x * (1.0 + torch.erf(x * 0.7071067811865476)))


def tower_reference(cfg: VisionConfig, wts: VisionWeights, pixel_values: torch.Tensor,
                    grids: Sequence[tuple], return_hidden: bool = False) -> torch.Tensor:
    """fp32 [L, patch_row] -> bf16-valued fp32 [L / merge^2, out_hidden]."""
    idx, wt = pos_gather_table(grids, cfg)
    cos, sin = (torch.from_numpy(a) for a in rope_tables(grids, cfg))
    x = _linear(_bf(pixel_values.float()), wts.patch_w, wts.patch_b)
    tab = wts.pos_table.float()
    wb = _bf(torch.from_numpy(wt))
    pe = _bf(tab[torch.from_numpy(idx[:, 0]).long()] * wb[:, 0:1])
    for i in range(1, 4):
        pe = _bf(pe + _bf(tab[torch.from_numpy(idx[:, i]).long()] * wb[:, i:i + 1]))
    x = _bf(x + pe)
    H, D, half = cfg.heads, cfg.head_dim, cfg.head_dim // 2
    bounds, row = [], 0
    for t, h, w in grids:
        bounds.append((row, row + t * h * w))
        row += t * h * w
    for blk in wts.blocks:
        y = _ln(x, blk["ln1_w"], blk["ln1_b"], cfg.eps)
        qkv = _linear(y, blk["qkv_w"], blk["qkv_b"]).reshape(-1, 3, H, D)
        q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]

        def rot(z):
            z1, z2 = z[..., :half], z[..., half:]
            c, s = cos[:, None, :], sin[:, None, :]
            return torch.cat([_bf(z1 * c - z2 * s), _bf(z2 * c + z1 * s)], dim=-1)
        q, k = rot(q), rot(k)
        att = torch.empty(x.shape[0], H, D)
        for a, b in bounds:
            s = torch.einsum("qhd,khd->hqk", q[a:b], k[a:b]) / math.sqrt(D)
            att[a:b] = torch.einsum("hqk,khd->qhd", torch.softmax(s, dim=-1), v[a:b])
        att = _bf(att.reshape(-1, H * D))
        x = _bf(_linear(att, blk["proj_w"], blk["proj_b"]) + x)
        y = _ln(x, blk["ln2_w"], blk["ln2_b"], cfg.eps)
        y = _gelu_tanh(_linear(y, blk["fc1_w"], blk["fc1_b"]))
        x = _bf(_linear(y, blk["fc2_w"], blk["fc2_b"]) + x)
    if return_hidden:
        return x
    m = wts.merger
    y = _ln(x, m["ln_w"], m["ln_b"], cfg.eps).reshape(-1, cfg.width * cfg.merge * cfg.merge)
    y = _gelu_erf(_linear(y, m["fc1_w"], m["fc1_b"]))
    return _linear(y, m["fc2_w"], m["fc2_b"])
