"""Mixture-of-experts layer weights: router, routed experts (stacked, expert-major, GEMM-ready
tiles) and the gated shared expert; plus the seeded generator.

Sharding (expert parallel): rank r owns experts [r * E / tp, (r + 1) * E / tp); the router is
replicated, so every rank computes the same routes from the (replicated) hidden state and keeps the
local ones.  The shared expert is split along its intermediate dim over the first
`shared_inter / 128` ranks at most (a rank's slice of the down projection must span whole 128-wide
reduction blocks); its sigmoid gate row is replicated.

Parity: expert ownership and replicated routing follow `crates/saber-kernels/src/moe.rs:19-27` and
`crates/saber-kernels/hip/moe_route.hip:8-24`; the expert pointer table of the reference's grouped
GEMM (`moe_grouped.hip`, `xptr`) becomes one stacked tensor with a constant stride per expert.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..ops import layouts as L
from ..ops.functional import QuantWeight
from .config import HybridConfig


@dataclass
class ExpertStack:
    """E_local experts of one linear in the grouped-GEMM layout."""
    tiles: torch.Tensor      # uint8 [E_local, N_pad/256, K/128, 16384]
    scale: torch.Tensor      # fp32 [E_local, N_pad] (already / 16)
    N: int
    K: int
    mx: bool = False         # MXFP4 experts: tiles uint8 [E_local, N_pad/256, K/128, 17408] (codes + block shifts), scale = row scale of the fold

    @property
    def n_experts(self) -> int:
        return self.tiles.shape[0]

    @property
    def N_pad(self) -> int:
        return self.tiles.shape[1] * L.TILE_N

    @property
    def stride_bytes(self) -> int:
        return self.tiles.stride(0)

    def expert(self, e: int) -> QuantWeight:
        return QuantWeight(self.tiles[e], self.scale[e], self.N, self.K, True, mx=self.mx)

    @staticmethod
    def from_mxfp4(codes: torch.Tensor, e8m0: torch.Tensor, device=None) -> "ExpertStack":
        """e2m1 codes uint8 [E, N, K] + e8m0 block scales uint8 [E, N, K/32]: the fold of every output row
        (block scales as shifts against the row's largest, the row scale in `scale`)."""
        from ..pack import quant_fp4 as Q
        E, Nn, K = codes.shape
        assert Nn % L.TILE_N == 0 and K % 128 == 0, "expert linears must be whole tiles"
        shift, row_scale = Q.fold_mxfp4(codes.reshape(E * Nn, K), e8m0.reshape(E * Nn, K // 32))
        tiles = L.tile_weight_mxfp4(codes.reshape(E * Nn, K), shift).reshape(E, Nn // L.TILE_N, K // 128, -1)
        dev = device if device is not None else codes.device
        return ExpertStack(tiles.to(dev).contiguous(), row_scale.reshape(E, Nn).float().to(dev).contiguous(), Nn, K, mx=True)

    @staticmethod
    def from_int(q: torch.Tensor, s: torch.Tensor, device=None) -> "ExpertStack":
        """q int8 [E, N, K] in [-8, 7], s fp32 [E, N]."""
        E, Nn, K = q.shape
        assert Nn % L.TILE_N == 0 and K % 128 == 0, "expert linears must be whole tiles"
        tiles = L.tile_weight_int4(q.reshape(E * Nn, K)).reshape(E, Nn // L.TILE_N, K // 128, -1)
        dev = device if device is not None else q.device
        return ExpertStack(tiles.to(dev).contiguous(), (s.float() / 16.0).to(dev).contiguous(), Nn, K)


def shared_ranks(cfg: HybridConfig, tp: int) -> int:
    return max(1, min(tp, cfg.moe.shared_inter // 128))


def expert_range(cfg: HybridConfig, tp: int, rank: int) -> tuple:
    per = cfg.moe.n_experts // tp
    return rank * per, per


def quantize_experts(w: torch.Tensor) -> tuple:
    """fp32 [E, N, K] -> (int8 [E, N, K], fp32 [E, N]); symmetric int4 per output row."""
    E, Nn, K = w.shape
    q, s = L.quantize_weight_rows(w.reshape(E * Nn, K), 4)
    return q.reshape(E, Nn, K), s.reshape(E, Nn)


def random_moe_layer(cfg: HybridConfig, tp: int, rank: int, dev, g: torch.Generator, std: float,
                     chunk: int = 32) -> dict:
    """Every rank draws every expert from the same generator state and keeps its own."""
    m = cfg.moe
    H, I, Is = cfg.hidden, m.expert_inter, m.shared_inter
    assert m.n_experts % tp == 0, "experts must divide by the parallel degree"
    e_lo, e_n = expert_range(cfg, tp, rank)

    def rand(*shape):
        return torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * std

    router_w = rand(m.n_experts, H) * 4.0          # wider logits: a sharper, more realistic router
    q, s = L.quantize_weight_rows(router_w, 8)
    router = QuantWeight.from_int(q, s, 8, dev)
    mxe = getattr(m, "expert_format", "iu8") == "mxfp4"

    def quant_e(w):
        if not mxe:
            return quantize_experts(w)
        from ..pack import quant_fp4 as Q
        E_, N_, K_ = w.shape
        codes, e = Q.quantize_mxfp4(w.reshape(E_ * N_, K_))
        return codes.reshape(E_, N_, K_), e.reshape(E_, N_, K_ // 32)
    gu_parts, dn_parts = [], []
    for c0 in range(0, m.n_experts, chunk):
        n = min(chunk, m.n_experts - c0)
        wgu = rand(n, 2 * I, H)                    # gate rows then up rows
        wdn = rand(n, H, I)
        lo, hi = max(c0, e_lo), min(c0 + n, e_lo + e_n)
        if lo < hi:
            gu_parts.append(quant_e(wgu[lo - c0:hi - c0]))
            dn_parts.append(quant_e(wdn[lo - c0:hi - c0]))
        del wgu, wdn
    make = ExpertStack.from_mxfp4 if mxe else ExpertStack.from_int
    gu = make(torch.cat([p[0] for p in gu_parts]), torch.cat([p[1] for p in gu_parts]), dev)
    dn = make(torch.cat([p[0] for p in dn_parts]), torch.cat([p[1] for p in dn_parts]), dev)
    # shared expert: gate | up | one sigmoid-gate row, then down
    wsg, wsu, wgate = rand(Is, H), rand(Is, H), rand(1, H) * 4.0
    wsd = rand(H, Is)
    n_sh = shared_ranks(cfg, tp)
    out = dict(router=router, gate_up=gu, down=dn, e_lo=e_lo, e_n=e_n, shared_gate_up=None,
               shared_down=None, shared_inter=0)
    if rank < n_sh:
        isl = Is // n_sh
        i0 = rank * isl
        qg, sg = L.quantize_weight_rows(torch.cat([wsg[i0:i0 + isl], wsu[i0:i0 + isl], wgate], 0), 4)
        out["shared_gate_up"] = QuantWeight.from_int(qg, sg, 4, dev)
        qd, sd = L.quantize_weight_rows(wsd, 4)      # full-row scales, then the K slice
        out["shared_down"] = QuantWeight.from_int(qd[:, i0:i0 + isl].contiguous(), sd, 4, dev)
        out["shared_inter"] = isl
    return out
