"""Plain PyTorch fp32 restatements of every native op. These are the oracles the GPU numerics tests
compare against and the compute path of the CPU executor; they are never a silent fallback for a
missing native library on a GPU box."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as Fn

from . import layouts as L


def bf16_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).float()


def gemm_i8(wq: torch.Tensor, w_scale: torch.Tensor, aq: torch.Tensor, a_scale: torch.Tensor) -> torch.Tensor:
    """wq int8 [N, K] (true integer values), aq int8 [M, K]; exact integer accumulate in fp64."""
    acc = aq.double() @ wq.double().t()
    return (acc.float() * (a_scale.float()[:, None] * w_scale.float()[None, :])).to(torch.bfloat16)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, w_offset: float) -> torch.Tensor:
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * (w.float() + w_offset)


def add_rms(x, res, w, eps=1e-6, w_offset=1.0):
    """Returns (new residual bf16, normed bf16-rounded fp32)."""
    s = (x.float() if x is not None else 0) + (res.float() if res is not None else 0)
    return s.to(torch.bfloat16), bf16_round(rms_norm(s, w, eps, w_offset))


def silu_mul(gu: torch.Tensor) -> torch.Tensor:
    K = gu.shape[1] // 2
    g, u = gu[:, :K].float(), gu[:, K:].float()
    return bf16_round(Fn.silu(g) * u)


def gate_sigmoid(a: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    return bf16_round(a.float() * torch.sigmoid(gate.float()))


def gdn_gated_norm(o: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps=1e-6) -> torch.Tensor:
    M, K = o.shape
    oh = o.float().reshape(M, K // 128, 128)
    n = oh * torch.rsqrt(oh.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return bf16_round(n.reshape(M, K) * Fn.silu(z.float()))


def quant_rows(h: torch.Tensor):
    return L.quantize_act_rows(h)


def softplus(x):
    return torch.where(x > 20, x, torch.log1p(torch.exp(x)))


def gdn_conv_step(x_rows: torch.Tensor, window: torch.Tensor, conv_w: torch.Tensor, n_q: int, n_k: int):
    """x_rows fp32 [n, C] (bf16-rounded), window fp32 [3, C]; returns (out [n, C], inputs incl. window)."""
    allx = torch.cat([window, x_rows], 0)
    n = x_rows.shape[0]
    outs = []
    for r in range(n):
        y = (allx[r:r + 4] * conv_w.t()).sum(0)
        outs.append(Fn.silu(y))
    out = torch.stack(outs, 0)
    C = out.shape[1]
    q = out[:, :n_q].reshape(n, -1, 128)
    k = out[:, n_q:n_q + n_k].reshape(n, -1, 128)
    q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) / math.sqrt(128.0)
    k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    out = torch.cat([q.reshape(n, n_q), k.reshape(n, n_k), out[:, n_q + n_k:]], 1)
    return out, allx


def gdn_recurrent_step(S: torch.Tensor, qkv: torch.Tensor, b: torch.Tensor, a: torch.Tensor,
                       A_log: torch.Tensor, dt_bias: torch.Tensor, n_q: int, n_k: int, HV: int, HK: int):
    """S fp32 [HV, 128(v), 128(k)]; qkv fp32 [n, C]; b, a fp32 [n, HV]. Returns (out [n, HV*128], states per row)."""
    n = qkv.shape[0]
    rep = HV // HK
    outs, states = [], []
    S = S.clone()
    for r in range(n):
        q = qkv[r, :n_q].reshape(HK, 128).repeat_interleave(rep, 0)
        k = qkv[r, n_q:n_q + n_k].reshape(HK, 128).repeat_interleave(rep, 0)
        v = qkv[r, n_q + n_k:].reshape(HV, 128)
        g = -torch.exp(A_log.float()) * softplus(a[r].float() + dt_bias.float())
        beta = torch.sigmoid(b[r].float())
        S = S * torch.exp(g)[:, None, None]
        kv = torch.einsum("hvk,hk->hv", S, k)
        u = (v - kv) * beta[:, None]
        S = S + u[:, :, None] * k[:, None, :]
        outs.append(torch.einsum("hvk,hk->hv", S, q).reshape(-1))
        states.append(S.clone())
    return torch.stack(outs, 0), states


def mrope_axis(j: int, sections) -> int:
    if j % 3 == 1 and j < 3 * sections[1]:
        return 1
    if j % 3 == 2 and j < 3 * sections[2]:
        return 2
    return 0


def qk_norm_rope(x: torch.Tensor, w: torch.Tensor, pos3: torch.Tensor, rot_dim=64,
                 sections=(11, 11, 10), theta=1e7, eps=1e-6, w_offset=1.0) -> torch.Tensor:
    """x fp32 [M, heads, 256]; pos3 int [3, M]. Norm (bf16-rounded) then rotate-half M-RoPE."""
    y = bf16_round(rms_norm(x, w, eps, w_offset))
    half = rot_dim // 2
    j = torch.arange(half, dtype=torch.float32)
    inv_freq = torch.exp2(-(2.0 * j / rot_dim) * math.log2(theta))
    axes = torch.tensor([mrope_axis(int(i), sections) for i in range(half)])
    posf = pos3.float()[axes, :].t()                       # [M, half]
    ang = posf * inv_freq[None, :]
    cs, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    lo, hi = y[..., :half], y[..., half:rot_dim]
    out = y.clone()
    out[..., :half] = lo * cs - hi * sn
    out[..., half:rot_dim] = hi * cs + lo * sn
    return out


def fp8_round(x: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    return (x.float() / scale).to(torch.float8_e4m3fn).float() * scale


def attention_rows(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kv_len: int, window: int = 0) -> torch.Tensor:
    """One sequence. q fp32 [n, nq, 256]; k, v fp32 [kv_len, nkv, 256]; right-aligned causal mask
    (window > 0: a row sees its last `window` keys only)."""
    n, nq, _ = q.shape
    nkv = k.shape[1]
    g = nq // nkv
    kk = k.repeat_interleave(g, 1)
    vv = v.repeat_interleave(g, 1)
    s = torch.einsum("nhd,khd->hnk", q, kk) / math.sqrt(256.0)
    rows = torch.arange(n)[:, None]
    keys = torch.arange(kv_len)[None, :]
    mask = keys < (kv_len - (n - 1) + rows)
    if window > 0:
        mask = mask & (keys >= (kv_len - (n - 1) + rows - window))
    s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(s, -1)
    return torch.einsum("hnk,khd->nhd", p, vv)
