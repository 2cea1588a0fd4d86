"""Per-rank weights of the hybrid decoder in GEMM-ready form, and their random-init generator.

Record names follow the pack convention (`layers.<i>.<block>.<linear>`); the same names key the
SBRPACK1 records, so a model is filled either from a pack (`from_records`) or from a seeded
N(0, 0.02) generator that quantises straight into the device layouts (`random_init`).
Sharding follows `models.config.shard`: column-parallel linears split output features (merged
q|gate|k|v and q|k|v|z|b|a by segment), row-parallel linears split the reduction dim.

Parity: linear inventory and shard kinds of `crates/saber-plan/src/model.rs:589-672`; quantisation
laws of `tools/pack/build_pack.py:22-40` restated for the synthetic W4A8-iu8 pack (symmetric per
output row, int4, int8 for the designated set, lm_head int8).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, Optional

import torch

from ..ops import layouts as L
from ..ops.functional import QuantWeight
from .config import HybridConfig, ShardShape, shard


@dataclass
class LayerWeights:
    kind: str                              # "gdn" | "attn"
    in_norm: torch.Tensor                  # fp32 [H]
    post_norm: torch.Tensor                # fp32 [H]
    mixer_in: QuantWeight                  # gdn: q|k|v|z|b|a ; attn: q|gate|k|v
    mixer_out: QuantWeight                 # row-parallel
    gate_up: Optional[QuantWeight] = None  # dense MLP: gate rows then up rows
    down: Optional[QuantWeight] = None
    # GDN
    conv_w: Optional[torch.Tensor] = None  # fp32 [C, 4]
    A_log: Optional[torch.Tensor] = None
    dt_bias: Optional[torch.Tensor] = None
    gdn_norm: Optional[torch.Tensor] = None  # fp32 [128]
    # attention
    q_norm: Optional[torch.Tensor] = None  # fp32 [256]
    k_norm: Optional[torch.Tensor] = None
    # MoE
    moe: Optional[dict] = None


@dataclass
class DrafterWeights:
    aux_fc: QuantWeight
    pos_emb: torch.Tensor                  # bf16 [block, Hd]
    layers: list = field(default_factory=list)   # dicts: norm, gate_up, down
    final_norm: Optional[torch.Tensor] = None
    head: Optional[QuantWeight] = None


@dataclass
class ModelWeights:
    embed: torch.Tensor                    # bf16 [vocab, H] (replicated on every rank)
    layers: list
    final_norm: torch.Tensor
    lm_head: QuantWeight                   # column-parallel over the vocab
    drafter: Optional[DrafterWeights] = None

    def nbytes(self) -> int:
        tot = self.embed.numel() * 2
        def qw(w): return 0 if w is None else w.tiles.numel() + w.scale.numel() * 4
        for lw in self.layers:
            tot += qw(lw.mixer_in) + qw(lw.mixer_out) + qw(lw.gate_up) + qw(lw.down)
            if lw.moe:
                tot += sum(qw(v) for v in lw.moe.values() if hasattr(v, "tiles"))
        tot += qw(self.lm_head)
        if self.drafter:
            tot += qw(self.drafter.aux_fc) + qw(self.drafter.head)
            for d in self.drafter.layers:
                tot += qw(d["gate_up"]) + qw(d["down"])
                if "attn" in d:
                    tot += qw(d["attn"]["kv_ctx"]) + qw(d["attn"]["qkv"]) + qw(d["attn"]["o_proj"])
        return tot


def linear_bits(cfg: HybridConfig, name: str) -> int:
    return 8 if name in cfg.w8_linears else 4


_FORMAT = {"fmt": "iu8", "had": False, "gen": None}     # format of the model being generated (set by random_init)


def _rotate(w: torch.Tensor):
    """(rotated weight, sign vector) when the model rotates activations, else (w, None).  The signs
    are drawn from the model's generator, so every rank draws the same vector for the same linear."""
    if not _FORMAT["had"]:
        return w, None
    K = w.shape[1]
    sign = (torch.randint(0, 2, (K,), generator=_FORMAT["gen"], device=w.device).float() * 2 - 1)
    return L.hadamard32_rows(w, sign), sign


def _quant_on(dev, w: torch.Tensor, bits: int, rotate: bool = False) -> QuantWeight:
    if rotate:
        w, sign = _rotate(w)
        qw = _quant_on(dev, w, bits)
        qw.had_sign = None if sign is None else sign.to(dev)
        return qw
    if bits == 4 and _FORMAT["fmt"] == "mxfp4":
        from ..pack import quant_fp4 as Q
        codes, e = Q.quantize_mxfp4(w)
        return QuantWeight.from_mxfp4(codes, e, dev)
    if bits == 4 and _FORMAT["fmt"] == "nvfp4" and w.shape[1] % 256 == 0:
        from ..pack import quant_fp4 as Q
        codes, bs, g = Q.quantize_nvfp4(w)
        return QuantWeight.from_nvfp4(codes, bs, g, dev)
    q, s = L.quantize_weight_rows(w, bits)
    return QuantWeight.from_int(q, s, bits, dev)


def _quant_cols(dev, w_full: torch.Tensor, bits: int, c0: int, c1: int, rotate: bool = False) -> QuantWeight:
    if rotate:
        w_full, sign = _rotate(w_full)
        qw = _quant_cols(dev, w_full, bits, c0, c1)
        qw.had_sign = None if sign is None else sign[c0:c1].contiguous().to(dev)
        return qw
    return _quant_cols_plain(dev, w_full, bits, c0, c1)


def _quant_cols_plain(dev, w_full: torch.Tensor, bits: int, c0: int, c1: int) -> QuantWeight:
    """Row-parallel shard: quantise the FULL rows (one scale per output feature over the whole
    reduction dim), then keep columns [c0, c1).  Every TP degree therefore holds the same integers
    and the same scales as TP=1, split along K."""
    if bits == 4 and _FORMAT["fmt"] == "mxfp4":
        from ..pack import quant_fp4 as Q
        codes, e = Q.quantize_mxfp4(w_full)
        shift, row_scale = Q.fold_mxfp4(codes, e)          # row reference over the FULL row
        tiles = L.tile_weight_mxfp4(codes[:, c0:c1].contiguous(), shift[:, c0 // 32:c1 // 32].contiguous())
        sc = torch.zeros(tiles.shape[0] * L.TILE_N, dtype=torch.float32, device=w_full.device)
        sc[:w_full.shape[0]] = row_scale
        return QuantWeight(tiles.to(dev).contiguous(), sc.to(dev), w_full.shape[0], c1 - c0, True, mx=True)
    if bits == 4 and _FORMAT["fmt"] == "nvfp4" and (c1 - c0) % 256 == 0 and c0 % 256 == 0:
        from ..pack import quant_fp4 as Q
        codes, bs, g = Q.quantize_nvfp4(w_full)            # block and tensor scales of the FULL matrix
        return QuantWeight.from_nvfp4(codes[:, c0:c1].contiguous(), bs[:, c0 // 16:c1 // 16].contiguous(), g, dev)
    q, s = L.quantize_weight_rows(w_full, bits)
    return QuantWeight.from_int(q[:, c0:c1].contiguous(), s, bits, dev)


def random_init(cfg: HybridConfig, tp: int, rank: int, device, seed: int = 0,
                std: float = 0.02) -> ModelWeights:
    """Seeded N(0, std) weights quantised into the device layouts.

    Every rank draws the FULL tensor of a linear from the same generator state and keeps its own
    shard, so TP=1 and TP=n describe the same model (the pack builder's `tp1 vs tp2` equality).
    """
    sh = shard(cfg, tp, rank)
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    _FORMAT.update(fmt=cfg.weight_format, had=bool(cfg.act_hadamard), gen=g)
    H, d, D = cfg.hidden, cfg.gdn_head_dim, cfg.head_dim

    def rand(n, k):
        return torch.randn(n, k, generator=g, device=dev, dtype=torch.float32) * std

    def vec(n, scale=0.1, base=0.0):
        return (torch.randn(n, generator=g, device=dev) * scale + base).float()

    def rows(w, first, count):
        return w[first:first + count]

    layers = []
    for i in range(cfg.n_layers):
        name = f"layers.{i}"
        if cfg.is_attention_layer(i):
            gate = 2 if cfg.attn_out_gate else 1
            wq = rand(cfg.n_q_heads * D * gate, H)      # [q heads | gate heads]
            wk = rand(cfg.n_kv_heads * D, H)
            wv = rand(cfg.n_kv_heads * D, H)
            nq, nkv = sh.n_q_heads, sh.n_kv_heads
            parts = [rows(wq, sh.q_head_first * D, nq * D)]
            if cfg.attn_out_gate:
                parts.append(rows(wq, cfg.n_q_heads * D + sh.q_head_first * D, nq * D))
            parts += [rows(wk, sh.kv_head_first * D, nkv * D), rows(wv, sh.kv_head_first * D, nkv * D)]
            mixer_in = _quant_on(dev, torch.cat(parts, 0), linear_bits(cfg, name + ".mixer.in"), rotate=True)
            wo = rand(H, cfg.n_q_heads * D)
            mixer_out = _quant_cols(dev, wo, linear_bits(cfg, name + ".mixer.out"),
                                    sh.q_head_first * D, (sh.q_head_first + nq) * D, rotate=True)
            lw = LayerWeights("attn", vec(H), vec(H), mixer_in, mixer_out,
                              q_norm=vec(D), k_norm=vec(D))
            del wq, wk, wv, wo
        else:
            HK, HV = cfg.gdn_k_heads, cfg.gdn_v_heads
            wq, wk = rand(HK * d, H), rand(HK * d, H)
            wv, wz = rand(HV * d, H), rand(HV * d, H)
            wb, wa = rand(HV, H), rand(HV, H)
            hk, hv = sh.gdn_k_heads, sh.gdn_v_heads
            k0, v0 = rank * hk, rank * hv
            parts = [rows(wq, k0 * d, hk * d), rows(wk, k0 * d, hk * d), rows(wv, v0 * d, hv * d),
                     rows(wz, v0 * d, hv * d), rows(wb, v0, hv), rows(wa, v0, hv)]
            mixer_in = _quant_on(dev, torch.cat(parts, 0), linear_bits(cfg, name + ".mixer.in"), rotate=True)
            wo = rand(H, HV * d)
            mixer_out = _quant_cols(dev, wo, linear_bits(cfg, name + ".mixer.out"), v0 * d, (v0 + hv) * d)
            conv_full = torch.randn(2 * HK * d + HV * d, 4, generator=g, device=dev) * 0.5
            conv = torch.cat([conv_full[k0 * d:(k0 + hk) * d],
                              conv_full[HK * d + k0 * d:HK * d + (k0 + hk) * d],
                              conv_full[2 * HK * d + v0 * d:2 * HK * d + (v0 + hv) * d]], 0).contiguous()
            A_full, dt_full = vec(HV, 0.5), vec(HV, 0.5)
            lw = LayerWeights("gdn", vec(H), vec(H), mixer_in, mixer_out, conv_w=conv,
                              A_log=A_full[v0:v0 + hv].contiguous(), dt_bias=dt_full[v0:v0 + hv].contiguous(),
                              gdn_norm=vec(d, 0.1, 1.0))
            del wq, wk, wv, wz, wb, wa, wo
        if cfg.moe is None:
            I = cfg.ffn_inter
            wg, wu = rand(I, H), rand(I, H)
            i0, il = rank * sh.ffn_inter, sh.ffn_inter
            lw.gate_up = _quant_on(dev, torch.cat([wg[i0:i0 + il], wu[i0:i0 + il]], 0),
                                   linear_bits(cfg, name + ".mlp.gate_up"), rotate=True)
            wd = rand(H, I)
            lw.down = _quant_cols(dev, wd, linear_bits(cfg, name + ".mlp.down"), i0, i0 + il, rotate=True)
            del wg, wu, wd
        else:
            from .moe_weights import random_moe_layer
            lw.moe = random_moe_layer(cfg, tp, rank, dev, g, std)
        layers.append(lw)

    embed = (torch.randn(cfg.vocab, H, generator=g, device=dev) * std).to(torch.bfloat16)
    if cfg.tie_embeddings:
        head_w = embed.float()
    else:
        head_w = rand(cfg.vocab, H)
    lm_head = _quant_on(dev, head_w[sh.vocab_first:sh.vocab_first + sh.vocab].contiguous(), cfg.lm_head_bits)
    del head_w
    mw = ModelWeights(embed, layers, vec(H), lm_head)

    if cfg.drafter is not None:
        dc = cfg.drafter
        Hd = dc.hidden
        dw = DrafterWeights(aux_fc=_quant_on(dev, rand(Hd, dc.n_taps * H), 4),
                            pos_emb=(torch.randn(dc.block, Hd, generator=g, device=dev) * std).to(torch.bfloat16))
        for li in range(dc.n_layers):
            lw = dict(norm=vec(Hd),
                      gate_up=_quant_on(dev, rand(2 * dc.inter, Hd), 4),
                      down=_quant_on(dev, rand(Hd, dc.inter), 4))
            if li < getattr(dc, "attn_layers", 0):
                nq, nkv, D = dc.attn_q_heads, dc.attn_kv_heads, cfg.head_dim
                lw["attn"] = dict(norm=vec(Hd), q_norm=vec(D), k_norm=vec(D),
                                  kv_ctx=_quant_on(dev, rand(2 * nkv * D, H), 4),          # context K | V from the target's tap row
                                  qkv=_quant_on(dev, rand((nq + 2 * nkv) * D, Hd), 4),      # the block rows' q | k | v
                                  o_proj=_quant_on(dev, rand(Hd, nq * D), 4))
            dw.layers.append(lw)
        dw.final_norm = vec(Hd)
        dw.head = _quant_on(dev, rand(cfg.vocab, Hd), dc.head_bits)
        mw.drafter = dw
    return mw
