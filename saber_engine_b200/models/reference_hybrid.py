"""Plain PyTorch fp32 forward of the hybrid decoder over a whole sequence (no cache), reading the
SAME quantised weights the native programs use.  It is the oracle of the end-to-end GPU tests and
restates the per-layer math in one place: add-RMS(1+w) -> per-token int8 -> integer GEMM -> ...
"""
from __future__ import annotations

import torch

from ..ops import layouts as L
from ..ops import reference as R
from ..ops.functional import QuantWeight
from .config import HybridConfig, shard
from .weights import ModelWeights


def dequant_linear(w: QuantWeight):
    """(int8 true values [N, K], fp32 row scale [N]) on the CPU, rows in the canonical order."""
    if getattr(w, "paired", False):
        from ..ops.functional import unpair_gate_up
        w = unpair_gate_up(w)
    tiles = w.tiles.cpu()
    if w.w4:
        q = L.unpack_weight_int4(tiles, w.N, w.K)
        s = w.scale.cpu()[: w.N] * 16.0
    else:
        q = L.untile_weight_int8(tiles, w.N, w.K)
        s = w.scale.cpu()[: w.N]
    return q, s


def _mx_dense(w: QuantWeight) -> torch.Tensor:
    """The fp32 matrix an MXFP4 linear multiplies with (fold and flush included)."""
    from ..pack import quant_fp4 as Q
    codes, shift = L.untile_weight_mxfp4(w.tiles.cpu(), w.N, w.K)
    return Q.dequant_folded(codes, shift, w.scale.cpu()[: w.N])


def _mx_linear(x: torch.Tensor, wq: torch.Tensor) -> torch.Tensor:
    from ..pack import quant_fp4 as Q
    aq, asc = Q.quantize_act_rows_e4m3(x)
    return ((aq.float().double() @ wq.double().t()).float() * asc[:, None]).to(torch.bfloat16)


def _fp4_dense(w: QuantWeight) -> torch.Tensor:
    """The fp32 matrix a native FP4 linear multiplies with (exact dequantisation of its tiles)."""
    from ..pack import quant_fp4 as Q
    vs = 16 if w.fp4 == 4 else 32
    codes, sf = L.untile_weight_fp4(w.tiles.cpu(), w.N, w.K, vs)
    if w.fp4 == 4:
        return Q.dequant_nvfp4(codes, sf.view(torch.float8_e4m3fn).float(), w.scale.cpu()[0])
    return Q.dequant_mxfp4(codes, sf)


def _fp4_linear(x: torch.Tensor, w: QuantWeight) -> torch.Tensor:
    """NVFP4 rows (per-token fp32 scale, e4m3 scale per 16, e2m1 codes) times the dequantised weight."""
    from ..pack import quant_fp4 as Q
    x = x.to(torch.bfloat16).float()
    M, K = x.shape
    g = (x.abs().amax(dim=1) / (6.0 * 448.0))
    b = x.reshape(M, K // 16, 16)
    bs = Q._e4m3_round((b.abs().amax(dim=-1) / 6.0 / g[:, None].clamp_min(1e-38)).clamp(max=448.0))
    denom = (bs * g[:, None]).clamp_min(1e-30)
    xd = (Q.e2m1_decode(Q.e2m1_encode(b / denom[..., None])) * denom[..., None]).reshape(M, K)
    return (xd.double() @ _fp4_dense(w).double().t()).float().to(torch.bfloat16)


def qlinear(x_bf16_rounded: torch.Tensor, w: QuantWeight) -> torch.Tensor:
    """Quantise rows per token, exact integer GEMM, scale, round to bf16 (as fp32 values)."""
    if getattr(w, "had_sign", None) is not None:      # the producer rotates before it quantises
        x_bf16_rounded = R.bf16_round(L.hadamard32_rows(x_bf16_rounded, w.had_sign.cpu()))
    if getattr(w, "fp4", 0):
        return _fp4_linear(x_bf16_rounded, w).float()
    if getattr(w, "mx", False):
        return _mx_linear(x_bf16_rounded, _mx_dense(w)).float()
    q, s = dequant_linear(w)
    aq, asc = L.quantize_act_rows(x_bf16_rounded)
    return R.gemm_i8(q, s, aq, asc).float()


def qlinear_row_parallel(x_bf16_rounded: torch.Tensor, w: QuantWeight, tp: int) -> torch.Tensor:
    """What `tp` ranks compute for a row-parallel linear: every rank quantises ITS slice of the
    activations per token, multiplies with its slice of the integers (full-row weight scales),
    rounds its partial to bf16; the partials are added in fp32 in rank order and rounded once."""
    if tp == 1:
        return qlinear(x_bf16_rounded, w)
    if getattr(w, "had_sign", None) is not None:
        x_bf16_rounded = R.bf16_round(L.hadamard32_rows(x_bf16_rounded, w.had_sign.cpu()))
    if getattr(w, "mx", False):
        wq = _mx_dense(w)
        ks = wq.shape[1] // tp
        acc = torch.zeros(x_bf16_rounded.shape[0], wq.shape[0])
        for r in range(tp):
            acc += _mx_linear(x_bf16_rounded[:, r * ks:(r + 1) * ks], wq[:, r * ks:(r + 1) * ks]).float()
        return R.bf16_round(acc)
    q, s = dequant_linear(w)
    K = q.shape[1]
    ks = K // tp
    acc = torch.zeros(x_bf16_rounded.shape[0], q.shape[0])
    for r in range(tp):
        aq, asc = L.quantize_act_rows(x_bf16_rounded[:, r * ks:(r + 1) * ks])
        acc += R.gemm_i8(q[:, r * ks:(r + 1) * ks], s, aq, asc).float()
    return R.bf16_round(acc)


def moe_route_ref(logits: torch.Tensor, top_k: int, norm: bool = True):
    """softmax fp32 -> top-k with the lower id winning ties -> optional renormalisation."""
    p = torch.softmax(logits.float(), dim=-1)
    order = torch.sort(-p, dim=-1, stable=True).indices[:, :top_k]
    w = torch.gather(p, 1, order)
    if norm:
        w = w / w.sum(dim=-1, keepdim=True)
    return order, w


def moe_mlp_ref(cfg: HybridConfig, moe: dict, n: torch.Tensor, tp: int = 1) -> torch.Tensor:
    """The MoE MLP on bf16-rounded normed rows `n` with UNSHARDED weights; tp > 1 restates the
    expert-parallel arithmetic (local sums rounded to bf16 per rank, added in rank order)."""
    from .moe_weights import shared_ranks
    m = cfg.moe
    M, H = n.shape
    I = m.expert_inter
    logits = qlinear(n, moe["router"])
    ids, wts = moe_route_ref(logits, m.top_k, m.norm_topk_prob)
    per = m.n_experts // tp
    # routed experts: each (token, k) route is an independent row
    y = torch.zeros(M, m.top_k, H)
    for e in ids.unique().tolist():
        tok, kk = (ids == e).nonzero(as_tuple=True)
        x = n[tok]
        if getattr(moe["gate_up"], "mx", False):
            # MXFP4 experts: the sorted rows are the layer's int8 rows turned into e4m3 (q * 448 / 127, row scale * 127 / 448)
            aq, asc = L.quantize_act_rows(x)
            f8 = (aq.float() * (448.0 / 127.0)).to(torch.float8_e4m3fn).float()
            gu = ((f8.double() @ _mx_dense(moe["gate_up"].expert(e)).double().t()).float() * (asc * (127.0 / 448.0))[:, None]).to(torch.bfloat16).float()
            y[tok, kk] = qlinear(R.silu_mul(gu), moe["down"].expert(e))
            continue
        gu = qlinear(x, moe["gate_up"].expert(e))
        y[tok, kk] = qlinear(R.silu_mul(gu), moe["down"].expert(e))
    # shared expert
    sgu = qlinear(n, moe["shared_gate_up"])
    Is = m.shared_inter
    gate = torch.sigmoid(sgu[:, 2 * Is])
    n_sh = shared_ranks(cfg, tp)
    isl = Is // n_sh
    q_d, s_d = dequant_linear(moe["shared_down"])
    total = torch.zeros(M, H)
    for r in range(tp):
        acc = torch.zeros(M, H)
        for k in range(m.top_k):
            own = (ids[:, k] // per) == r
            acc += torch.where(own[:, None], wts[:, k, None] * y[:, k], torch.zeros(()))
        if r < n_sh:
            sl = slice(r * isl, (r + 1) * isl)
            act = R.silu_mul(torch.cat([sgu[:, sl], sgu[:, Is + r * isl:Is + (r + 1) * isl]], 1))
            aq, asc = L.quantize_act_rows(act)
            acc += gate[:, None] * R.gemm_i8(q_d[:, sl], s_d, aq, asc).float()
        total += R.bf16_round(acc)
    return R.bf16_round(total)


@torch.no_grad()
def forward_full(cfg: HybridConfig, w: ModelWeights, ids: torch.Tensor, kv_fp8: bool = True, tp: int = 1) -> dict:
    """ids int [T] (one sequence from position 0). Returns logits [T, vocab] and per-layer residuals.
    `w` are the UNSHARDED weights; tp > 1 restates the arithmetic of a tensor-parallel run."""
    sh = shard(cfg, 1, 0)
    T = ids.numel()
    H, D, d = cfg.hidden, cfg.head_dim, cfg.gdn_head_dim
    h = w.embed.cpu()[ids.long()].float()
    delta = None
    pos3 = torch.arange(T, dtype=torch.int32)[None, :].repeat(3, 1)
    taps = []
    for i, lw in enumerate(w.layers):
        hb, n = R.add_rms(delta, h.to(torch.bfloat16), lw.in_norm.cpu(), cfg.eps, cfg.norm_offset)
        h = hb.float()
        taps.append(h.clone())
        y = qlinear(n, lw.mixer_in)
        if lw.kind == "gdn":
            n_q = n_k = sh.gdn_k_heads * d
            C = sh.gdn_conv_c
            hv = sh.gdn_v_heads
            qkv, _ = R.gdn_conv_step(R.bf16_round(y[:, :C]), torch.zeros(3, C), lw.conv_w.cpu(), n_q, n_k)
            z = y[:, C:C + hv * d]
            b, a = y[:, C + hv * d:C + hv * d + hv], y[:, C + hv * d + hv:C + hv * d + 2 * hv]
            o, _ = R.gdn_recurrent_step(torch.zeros(hv, d, d), qkv, b, a, lw.A_log.cpu(), lw.dt_bias.cpu(),
                                        n_q, n_k, hv, sh.gdn_k_heads)
            mix = R.gdn_gated_norm(o, z, lw.gdn_norm.cpu(), cfg.eps)
        else:
            nq, nkv = sh.n_q_heads, sh.n_kv_heads
            gate = 2 if cfg.attn_out_gate else 1
            q = y[:, :nq * D].reshape(T, nq, D)
            k_off = nq * D * gate
            k = y[:, k_off:k_off + nkv * D].reshape(T, nkv, D)
            v = y[:, k_off + nkv * D:k_off + 2 * nkv * D].reshape(T, nkv, D)
            kw = dict(rot_dim=cfg.rot_dim, sections=cfg.mrope_sections, theta=cfg.rope_theta, eps=cfg.eps,
                      w_offset=cfg.norm_offset)
            qr = R.bf16_round(R.qk_norm_rope(q, lw.q_norm.cpu(), pos3, **kw))
            kr = R.qk_norm_rope(k, lw.k_norm.cpu(), pos3, **kw)
            if kv_fp8:
                kr, v = R.fp8_round(kr), R.fp8_round(v)
            ao = R.bf16_round(R.attention_rows(qr, kr, v, T)).reshape(T, nq * D)
            mix = R.gate_sigmoid(ao, y[:, nq * D:2 * nq * D]) if cfg.attn_out_gate else ao
        delta = qlinear_row_parallel(mix, lw.mixer_out, tp).to(torch.bfloat16)
        hb, n = R.add_rms(delta, h.to(torch.bfloat16), lw.post_norm.cpu(), cfg.eps, cfg.norm_offset)
        h = hb.float()
        if cfg.moe is None:
            gu = qlinear(n, lw.gate_up)
            delta = qlinear_row_parallel(R.silu_mul(gu), lw.down, tp).to(torch.bfloat16)
        else:
            delta = moe_mlp_ref(cfg, lw.moe, n, tp).to(torch.bfloat16)
    hb, n = R.add_rms(delta, h.to(torch.bfloat16), w.final_norm.cpu(), cfg.eps, cfg.norm_offset)
    logits = qlinear(n, w.lm_head)
    return {"logits": logits, "taps": taps, "final": n}
