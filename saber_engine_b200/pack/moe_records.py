"""Pack records of a mixture-of-experts layer (router, stacked experts, shared expert) and their
loader.  The stacked expert tensors are one record per linear: shape (E_local, N, K), expert-major,
each expert in the same 256 x 128 tile order as a dense W4 linear.

Parity: the reference stores experts as per-expert records reached through a pointer table
(`crates/saber-kernels/hip/moe_grouped.hip`, `xptr`) and tiers them (`crates/saber-mem/src/expert_tier.rs:1-40`);
with 180 GB of HBM the experts of a rank stay resident, so one contiguous record per linear with a
constant per-expert stride replaces table and tiers.
"""
from __future__ import annotations

import numpy as np
import torch

from ..models.moe_weights import ExpertStack
from . import format as PF

SHARD_EXPERTS = PF.SHARD_DIM0


def _np(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().numpy()


def moe_records(prefix: str, moe: dict):
    from .build import _qw_records
    yield from _qw_records(f"{prefix}.moe.router", moe["router"], PF.SHARD_REPLICATED)
    for key in ("gate_up", "down"):
        st: ExpertStack = moe[key]
        yield (f"{prefix}.moe.experts.{key}.weight_i4", _np(st.tiles), "u8", (st.n_experts, st.N, st.K),
               PF.LAYOUT_W4_TILE256, SHARD_EXPERTS)
        yield (f"{prefix}.moe.experts.{key}.weight_i4_scale", _np(st.scale), "f32", (st.n_experts, st.N),
               PF.LAYOUT_ROW_SCALE_F32, SHARD_EXPERTS)
    yield (f"{prefix}.moe.experts.range", np.array([moe["e_lo"], moe["e_n"], moe["shared_inter"]], dtype=np.int32),
           "i32", (3,), PF.LAYOUT_RAW, SHARD_EXPERTS)
    if moe["shared_gate_up"] is not None:
        yield from _qw_records(f"{prefix}.moe.shared.gate_up_proj", moe["shared_gate_up"], PF.SHARD_DIM0_SEGMENTS)
        yield from _qw_records(f"{prefix}.moe.shared.down_proj", moe["shared_down"], PF.SHARD_DIM1)


def load_moe(reader, prefix: str, device, verify: bool = True):
    from .build import _load_qw, _tensor
    if not reader.has(f"{prefix}.moe.experts.range"):
        return None
    rng = _tensor(reader, f"{prefix}.moe.experts.range", "cpu", torch.int32, None, verify).tolist()
    out = dict(router=_load_qw(reader, f"{prefix}.moe.router", device, verify), e_lo=rng[0], e_n=rng[1],
               shared_inter=rng[2], shared_gate_up=None, shared_down=None)
    for key in ("gate_up", "down"):
        name = f"{prefix}.moe.experts.{key}.weight_i4"
        E, Nn, K = reader.records[name].shape
        tiles = _tensor(reader, name, device, torch.uint8, (E, Nn // 256, K // 128, 16384), verify)
        scale = _tensor(reader, name + "_scale", device, torch.float32, (E, Nn), verify)
        out[key] = ExpertStack(tiles, scale, Nn, K)
    if reader.has(f"{prefix}.moe.shared.gate_up_proj.weight_i4"):
        out["shared_gate_up"] = _load_qw(reader, f"{prefix}.moe.shared.gate_up_proj", device, verify)
        out["shared_down"] = _load_qw(reader, f"{prefix}.moe.shared.down_proj", device, verify)
    return out
