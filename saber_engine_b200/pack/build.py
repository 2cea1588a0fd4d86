"""Pack builder and loader for the hybrid models: ModelWeights <-> SBRPACK1 records.

`write_pack` produces `<out>/tp<N>/{manifest.json, rank*.pack}` from a seeded random-init model
(N(0, 0.02), quantised to the W4A8-iu8 layouts); `load_weights` is the inverse the engine uses at
boot (the pack drives the engine: W4 vs W8 of a linear is decided by which record exists, not by a
flag, as in `README.md:204-209` of the reference).

Parity: `tools/pack/build_pack.py:985-1100` (records, plan / tier descriptors, manifest), the
TP shard policy of `crates/saber-plan/src/model.rs:589-672`, and the self-checks of
`tools/pack/check_manifest.py`.
"""
from __future__ import annotations

import dataclasses
from pathlib import Path
from typing import Optional

import numpy as np
import torch

from ..models import config as MC
from ..models.weights import DrafterWeights, LayerWeights, ModelWeights, random_init
from ..ops.functional import QuantWeight
from . import format as PF

FORMAT_TAG = "w4a8_iu8_b200/1"


def _np(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()
    return t.numpy()


def _qw_records(name: str, w: Optional[QuantWeight], shard: int):
    if w is None:
        return
    if getattr(w, "paired", False):      # records keep the canonical row order (gate rows, then up rows)
        from ..ops.functional import unpair_gate_up
        w = unpair_gate_up(w)
    if getattr(w, "mx", False):
        # MXFP4: e2m1 codes + block shifts in the GEMM's tile order, and the per-row 2^wref scale
        yield (f"{name}.weight_mxfp4", _np(w.tiles), "u8", (w.N, w.K), PF.LAYOUT_MXFP4_TILE, shard)
        yield (f"{name}.weight_mxfp4_scale", _np(w.scale), "f32", (w.N,), PF.LAYOUT_ROW_SCALE_F32, shard)
    elif w.w4:
        yield (f"{name}.weight_i4", _np(w.tiles), "u8", (w.N, w.K), PF.LAYOUT_W4_TILE256, shard)
        yield (f"{name}.weight_i4_scale", _np(w.scale), "f32", (w.N,), PF.LAYOUT_ROW_SCALE_F32, shard)
    else:
        yield (f"{name}.weight_i8", _np(w.tiles), "u8", (w.N, w.K), PF.LAYOUT_W8_TILE256, shard)
        yield (f"{name}.weight_i8_scale", _np(w.scale), "f32", (w.N,), PF.LAYOUT_ROW_SCALE_F32, shard)


def weight_records(mw: ModelWeights):
    R = PF.SHARD_REPLICATED
    yield ("embed_tokens.weight", _np(mw.embed), "bf16", tuple(mw.embed.shape), PF.LAYOUT_RAW, R)
    yield ("norm.weight", _np(mw.final_norm), "f32", tuple(mw.final_norm.shape), PF.LAYOUT_RAW, R)
    yield from _qw_records("lm_head", mw.lm_head, PF.SHARD_DIM0)
    for i, lw in enumerate(mw.layers):
        p = f"layers.{i}"
        yield (f"{p}.input_layernorm.weight", _np(lw.in_norm), "f32", tuple(lw.in_norm.shape), PF.LAYOUT_RAW, R)
        yield (f"{p}.post_attention_layernorm.weight", _np(lw.post_norm), "f32", tuple(lw.post_norm.shape), PF.LAYOUT_RAW, R)
        yield from _qw_records(f"{p}.{lw.kind}.in_proj", lw.mixer_in, PF.SHARD_DIM0_SEGMENTS)
        yield from _qw_records(f"{p}.{lw.kind}.out_proj", lw.mixer_out, PF.SHARD_DIM1)
        yield from _qw_records(f"{p}.mlp.gate_up_proj", lw.gate_up, PF.SHARD_DIM0_SEGMENTS)
        yield from _qw_records(f"{p}.mlp.down_proj", lw.down, PF.SHARD_DIM1)
        for key in ("conv_w", "A_log", "dt_bias", "gdn_norm", "q_norm", "k_norm"):
            t = getattr(lw, key)
            if t is not None:
                shard = PF.SHARD_DIM0 if key in ("conv_w", "A_log", "dt_bias") else R
                yield (f"{p}.{lw.kind}.{key}", _np(t), "f32", tuple(t.shape), PF.LAYOUT_RAW, shard)
        if lw.moe:
            from .moe_records import moe_records
            yield from moe_records(p, lw.moe)
    if mw.drafter is not None:
        d = mw.drafter
        yield from _qw_records("drafter.aux_fc", d.aux_fc, R)
        yield ("drafter.pos_emb", _np(d.pos_emb), "bf16", tuple(d.pos_emb.shape), PF.LAYOUT_RAW, R)
        for j, lw in enumerate(d.layers):
            yield (f"drafter.layers.{j}.norm", _np(lw["norm"]), "f32", tuple(lw["norm"].shape), PF.LAYOUT_RAW, R)
            yield from _qw_records(f"drafter.layers.{j}.gate_up_proj", lw["gate_up"], R)
            yield from _qw_records(f"drafter.layers.{j}.down_proj", lw["down"], R)
        yield ("drafter.final_norm", _np(d.final_norm), "f32", tuple(d.final_norm.shape), PF.LAYOUT_RAW, R)
        yield from _qw_records("drafter.head", d.head, R)


def plan_descriptor(cfg, tp: int) -> dict:
    if getattr(cfg, "weight_format", "iu8") == "mxfp4":
        return {"format": "mxfp4_fold_b200/1", "model": cfg.name, "tp": tp, "config": MC.as_dict(cfg),
                "transforms": ["mxfp4_e2m1_e8m0_per32", "fold_shift_vs_row_max", "rowwise_int8_sym(w8 set, lm_head)",
                               "tile256x128_sw128"]}
    return {"format": FORMAT_TAG, "model": cfg.name, "tp": tp, "config": MC.as_dict(cfg),
            "transforms": ["rowwise_int4_sym", "rowwise_int8_sym(w8 set, lm_head)", "tile256x128_sw128"]}


def tier_descriptor(cfg, seed: int) -> dict:
    return {"source": "random-init N(0, 0.02)", "seed": seed, "model": cfg.name}


def write_pack(cfg, out_dir, tp: int = 1, seed: int = 0, device="cpu") -> Path:
    d = Path(out_dir) / f"tp{tp}"
    d.mkdir(parents=True, exist_ok=True)
    plan, tier = plan_descriptor(cfg, tp), tier_descriptor(cfg, seed)
    ranks = []
    for rank in range(tp):
        mw = random_init(cfg, tp, rank, device, seed)
        w = PF.PackWriter(d / f"rank{rank}.pack", tp, rank, plan, tier, build_unix=0)
        for name, arr, dtype, shape, layout, shard in weight_records(mw):
            w.add(name, arr, dtype, shape, layout, shard)
        ranks.append(w.finish())
        del mw
    PF.write_manifest(d, tp, plan, tier, ranks, shard_policy={"kv_heads": "replicate when tp > n_kv_heads"},
                      model=cfg.name)
    return d


def _tensor(reader: PF.PackReader, name: str, device, dtype: torch.dtype, shape=None, verify=True):
    rec = reader.records[name]
    buf = np.array(reader.payload(name, verify=verify))
    t = torch.from_numpy(buf)
    if dtype == torch.bfloat16:
        t = t.view(torch.int16).view(torch.bfloat16)
    elif dtype != torch.uint8:
        t = t.view(dtype)
    return t.reshape(shape if shape is not None else rec.shape).to(device)


def _load_qw(reader, name: str, device, verify=True) -> Optional[QuantWeight]:
    key = f"{name}.weight_mxfp4"
    if reader.has(key):          # the record that exists decides the kernel, not a flag
        Nn, K = reader.records[key].shape
        n_tiles, kb = (Nn + 255) // 256, K // 128
        tiles = _tensor(reader, key, device, torch.uint8, (n_tiles, kb, 17408), verify)
        scale = _tensor(reader, key + "_scale", device, torch.float32, (n_tiles * 256,), verify)
        return QuantWeight(tiles, scale, Nn, K, True, mx=True)
    for bits, tag in ((4, "i4"), (8, "i8")):
        key = f"{name}.weight_{tag}"
        if reader.has(key):
            rec = reader.records[key]
            Nn, K = rec.shape
            n_tiles, kb = (Nn + 255) // 256, K // 128
            tiles = _tensor(reader, key, device, torch.uint8, (n_tiles, kb, 16384 if bits == 4 else 32768), verify)
            scale = _tensor(reader, key + "_scale", device, torch.float32, (n_tiles * 256,), verify)
            return QuantWeight(tiles, scale, Nn, K, bits == 4)
    return None


def load_weights(pack_dir, cfg, tp: int, rank: int, device, verify: bool = True) -> ModelWeights:
    d = Path(pack_dir)
    if (d / f"tp{tp}").is_dir():
        d = d / f"tp{tp}"
    problems = PF.check_manifest(d) if verify else []
    if problems:
        raise PF.PackError("pack refused: " + "; ".join(problems))
    plan_hash = PF.sha256(PF.canonical_json(plan_descriptor(cfg, tp)))
    r = PF.PackReader(d / f"rank{rank}.pack", plan_hash, tp, rank)
    f32 = lambda n: _tensor(r, n, device, torch.float32, None, verify)      # noqa: E731
    layers = []
    for i in range(cfg.n_layers):
        kind = "attn" if cfg.is_attention_layer(i) else "gdn"
        p = f"layers.{i}"
        lw = LayerWeights(kind, f32(f"{p}.input_layernorm.weight"), f32(f"{p}.post_attention_layernorm.weight"),
                          _load_qw(r, f"{p}.{kind}.in_proj", device, verify), _load_qw(r, f"{p}.{kind}.out_proj", device, verify),
                          _load_qw(r, f"{p}.mlp.gate_up_proj", device, verify), _load_qw(r, f"{p}.mlp.down_proj", device, verify))
        for key in ("conv_w", "A_log", "dt_bias", "gdn_norm", "q_norm", "k_norm"):
            if r.has(f"{p}.{kind}.{key}"):
                setattr(lw, key, f32(f"{p}.{kind}.{key}"))
        if cfg.moe is not None:
            from .moe_records import load_moe
            lw.moe = load_moe(r, p, device, verify)
        layers.append(lw)
    mw = ModelWeights(_tensor(r, "embed_tokens.weight", device, torch.bfloat16, None, verify), layers,
                      f32("norm.weight"), _load_qw(r, "lm_head", device, verify))
    if r.has("drafter.pos_emb") and cfg.drafter is not None:
        dw = DrafterWeights(_load_qw(r, "drafter.aux_fc", device, verify),
                            _tensor(r, "drafter.pos_emb", device, torch.bfloat16, None, verify))
        for j in range(cfg.drafter.n_layers):
            dw.layers.append(dict(norm=f32(f"drafter.layers.{j}.norm"),
                                  gate_up=_load_qw(r, f"drafter.layers.{j}.gate_up_proj", device, verify),
                                  down=_load_qw(r, f"drafter.layers.{j}.down_proj", device, verify)))
        dw.final_norm = f32("drafter.final_norm")
        dw.head = _load_qw(r, "drafter.head", device, verify)
        mw.drafter = dw
    return mw
