"""Small stand-alone cases of the hot kernels, one per `--case`, for profiler captures and quick
timings: each case builds a few GB of operands at most, launches its kernel a handful of times on
distinct operand copies (so every launch streams from HBM, not from L2) and prints the CUDA-event
time of the last launches.

    python -m saber_engine_b200.runtime.kernel_cases --case gemm_w4_gate_up_m72
    ncu --set full --clock-control none -k regex:gemm_i8_kernel -s 2 -c 1 -o prof \\
        python -m saber_engine_b200.runtime.kernel_cases --case gemm_w4_gate_up_m72

Parity: the role of the reference's per-op timing arms and `chain-bench` instrument
(`crates/saber-exec/src/steploop.rs:1-25`).
"""
from __future__ import annotations

import argparse
import ctypes as C

import torch

from ..ops import functional as F
from ..ops import layouts as L
from ..ops import native as N

DEV = "cuda"


def _time(fns, label: str, nbytes: float = 0.0) -> None:
    """fns: one callable per operand copy; warm-up over all, then time a second pass."""
    for f in fns:
        f()
    torch.cuda.synchronize()
    e = [torch.cuda.Event(enable_timing=True) for _ in range(len(fns) + 1)]
    e[0].record()
    for i, f in enumerate(fns):
        f()
        e[i + 1].record()
    torch.cuda.synchronize()
    us = sorted(e[i].elapsed_time(e[i + 1]) * 1e3 for i in range(len(fns)))
    med = us[len(us) // 2]
    extra = f"  {nbytes / med / 1e6:.2f} TB/s algorithmic" if nbytes else ""
    print(f"{label}: median {med:.1f} us over {len(fns)} launches (host-launched, includes ~5 us of launch){extra}")
    F.scratch(DEV).check()


def _gemm(Nn, K, M, w4, splits, copies=3):
    n_pad = L.round_up(Nn, 256)
    tile = 16384 if w4 else 32768
    ws = [F.QuantWeight(torch.randint(0, 255, (n_pad // 256, K // 128, tile), dtype=torch.uint8, device=DEV),
                        torch.rand(n_pad, device=DEV) * 1e-3, Nn, K, bool(w4)) for _ in range(copies)]
    qa = F.plain_quant(torch.randn(M, K, device=DEV).to(torch.bfloat16))
    out = torch.empty(M, Nn, dtype=torch.bfloat16, device=DEV)
    sc = F.scratch(DEV)
    ps = [F.gemm_params(w, qa, out, sc, splits=splits) for w in ws]
    lib = N.lib()
    fns = [lambda p=p: N.check(lib.saber_gemm_i8_launch(C.byref(p), 0, N.stream_handle()), "gemm") for p in ps]
    _time(fns, f"gemm_i8 N={Nn} K={K} M={M} w4={w4} splits={ps[0].splits}", n_pad * K * (0.5 if w4 else 1.0))
    return ws, qa, out


def _gemm_2sm(Nn, K, M, copies=3):
    """int8 weights over a long row run on CTA pairs (cta_group::2), beside the one-CTA kernel on the same operands."""
    n_pad = L.round_up(Nn, 256)
    ws = [F.QuantWeight(torch.randint(0, 255, (n_pad // 256, K // 128, 32768), dtype=torch.uint8, device=DEV),
                        torch.rand(n_pad, device=DEV) * 1e-3, Nn, K, False) for _ in range(copies)]
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    q0 = F.plain_quant(x)
    m_pad = L.round_up(M, 512)
    qa = F.QuantAct(torch.zeros(K // 128, m_pad, 128, dtype=torch.int8, device=DEV), torch.zeros(m_pad, device=DEV), M, K)
    qa.q[:, : q0.M_pad] = q0.q[:, : min(q0.M_pad, m_pad)]
    qa.scale[: q0.M_pad] = q0.scale[: min(q0.M_pad, m_pad)]
    out = torch.empty(M, Nn, dtype=torch.bfloat16, device=DEV)
    sc = F.scratch(DEV)
    ps = [F.gemm_params(w, qa, out, sc, splits=1) for w in ws]
    lib = N.lib()
    fns = [lambda p=p: N.check(lib.saber_gemm_w8_2sm_launch(C.byref(p), 0, N.stream_handle()), "gemm 2sm") for p in ps]
    lib.saber_set_gemm_2sm_persistent(1)
    _time(fns, f"gemm_w8_2sm persistent N={Nn} K={K} M={M}", n_pad * K * 1.0)
    lib.saber_set_gemm_2sm_persistent(0)
    _time(fns, f"gemm_w8_2sm one tile per cluster N={Nn} K={K} M={M}", n_pad * K * 1.0)
    lib.saber_set_gemm_2sm_persistent(1)
    fns = [lambda p=p: N.check(lib.saber_gemm_i8_launch(C.byref(p), 0, N.stream_handle()), "gemm") for p in ps]
    _time(fns, f"gemm_i8 (one CTA, two token tiles) N={Nn} K={K} M={M} w8", n_pad * K * 1.0)
    return ws, qa, out


def _gemm_fp4(Nn, K, M, fmt, splits, copies=3):
    """Native block-scaled FP4 GEMM (4 = NVFP4, 5 = MXFP4): random packed operands and scales."""
    n_pad = L.round_up(Nn, 256)
    sfb = 4096 if fmt == 4 else 2048
    ws = []
    for _ in range(copies):
        t = torch.randint(0, 255, (n_pad // 256, K // 256, 32768 + sfb), dtype=torch.uint8, device=DEV)
        t[..., 32768:] = torch.randint(0x30, 0x40, t[..., 32768:].shape, dtype=torch.uint8, device=DEV) if fmt == 4 else 127
        ws.append(F.QuantWeight(t, torch.full((n_pad,), 1e-3, device=DEV), Nn, K, True, fp4=fmt))
    m_pad = L.padded_rows(M)
    q = torch.randint(0, 255, (K // 256, m_pad, 128), dtype=torch.uint8, device=DEV)
    sf = torch.full((K // 256, (m_pad + 127) // 128, sfb // 2), 0x38 if fmt == 4 else 127, dtype=torch.uint8, device=DEV)
    qa = F.QuantAct(q, torch.ones(m_pad, device=DEV), M, K, fp4=fmt, sf=sf)
    out = torch.empty(M, Nn, dtype=torch.bfloat16, device=DEV)
    sc = F.scratch(DEV)
    ps = [F.gemm_params(w, qa, out, sc, splits=splits) for w in ws]
    lib = N.lib()
    fns = [lambda p=p: N.check(lib.saber_gemm_i8_launch(C.byref(p), 0, N.stream_handle()), "gemm") for p in ps]
    _time(fns, f"gemm_fp4 ({'nvfp4' if fmt == 4 else 'mxfp4'}) N={Nn} K={K} M={M} splits={ps[0].splits}", n_pad * K * 0.5 + n_pad * K // (16 if fmt == 4 else 32))
    return ws, qa, out


def _attn(nseq, n, ctx, splits, copies=3, impl=0):
    nq, nkv, D = 24, 4, 256
    M = nseq * n
    pages = (ctx + n + 15) // 16
    nblocks = nseq * pages + 1
    kvs = [(torch.randn(nblocks, nkv, 2, 16, D, device=DEV) * 0.5).to(torch.float8_e4m3fn).view(torch.uint8)
           for _ in range(copies)]
    q = torch.randn(M, nq, D, device=DEV).to(torch.bfloat16)
    bt = torch.arange(1, 1 + nseq * pages, dtype=torch.int32, device=DEV).view(nseq, pages)
    cu = torch.arange(0, M + 1, n, dtype=torch.int32, device=DEV)
    kvl = torch.full((nseq,), ctx + n, dtype=torch.int32, device=DEV)
    out = torch.empty_like(q)
    po = torch.empty(nseq, nq, splits, 16, D, device=DEV) if splits > 1 else None
    pm = torch.empty(nseq, nq, splits, 16, 2, device=DEV) if splits > 1 else None
    q_tiles = (n + 15) // 16
    ps = [F.attn_params(q, kv, bt, cu, kvl, out, po, pm, nkv, splits, q_tiles, pack_rows=n, impl=impl) for kv in kvs]
    torch.cuda.synchronize()
    lib = N.lib()
    fns = [lambda p=p: N.check(lib.saber_attn_launch(C.byref(p), N.stream_handle()), "attn") for p in ps]
    _time(fns, f"attn_{'tc' if impl else 'paged'} nseq={nseq} rows={n} ctx={ctx} splits={splits}", nseq * (ctx + n) * nkv * 2 * D)
    return kvs, q, out, po, pm


def _gdn(nseq, n, shift, vs=2, copies=3):
    HV, HK, d = 48, 16, 128
    M = nseq * n
    C_ = 2 * HK * d + HV * d
    qkv = torch.randn(M, C_, device=DEV) * 0.1
    ba = torch.randn(M, 2 * HV, device=DEV).to(torch.bfloat16)
    A_log, dtb = torch.randn(HV, device=DEV) * 0.5, torch.randn(HV, device=DEV) * 0.5
    states = [torch.randn(nseq + 1, HV, d, d, device=DEV) * 0.01 for _ in range(copies)]
    stashes = [torch.randn(nseq + 1, 9, HV, vs, F.gdn_stash_stride(vs), device=DEV) * 0.1 for _ in range(copies)]
    cu = torch.arange(0, M + 1, n, dtype=torch.int32, device=DEV)
    slots = torch.arange(1, nseq + 1, dtype=torch.int32, device=DEV)
    sh = torch.full((nseq,), shift, dtype=torch.int32, device=DEV)
    out = torch.empty(M, HV * d, device=DEV)
    ps = [F.gdn_rec_params(qkv, ba, A_log, dtb, states[i], stashes[i], cu, slots, sh, out, HK * d, HK * d, HV, HK, False)
          for i in range(copies)]
    torch.cuda.synchronize()
    lib = N.lib()
    fns = [lambda p=p: N.check(lib.saber_gdn_recurrent_launch(C.byref(p), nseq, vs, N.stream_handle()), "gdn") for p in ps]
    _time(fns, f"gdn_recurrent nseq={nseq} rows={n} replay={shift}", 2.0 * nseq * HV * d * d * 4)
    return states, stashes, out


def _gdn_step(nseq, n, shift, copies=3):
    """One DeltaNet layer of a decode step: the fused launch, and the three launches it replaces."""
    HV, HK, d = 48, 16, 128
    M = nseq * n
    K = HV * d
    C_ = 2 * HK * d + K
    ld = C_ + K + 2 * HV
    x = (torch.randn(M, ld, device=DEV) * 0.5).to(torch.bfloat16)
    conv_w = torch.randn(C_, 4, device=DEV) * 0.5
    A_log, dtb = torch.randn(HV, device=DEV) * 0.5, torch.randn(HV, device=DEV) * 0.5
    norm_w = torch.ones(d, device=DEV)
    states = [torch.randn(nseq + 1, HV, d, d, device=DEV) * 0.01 for _ in range(copies)]
    stashes = [torch.randn(nseq + 1, 9, HV, 1, 260, device=DEV) * 0.1 for _ in range(copies)]
    hists = [F.gdn_hist_alloc(nseq + 1, 3 + 9, C_, DEV) for _ in range(copies)]
    cu = torch.arange(0, M + 1, n, dtype=torch.int32, device=DEV)
    slots = torch.arange(1, nseq + 1, dtype=torch.int32, device=DEV)
    sh = torch.full((nseq,), shift, dtype=torch.int32, device=DEV)
    qa = F.QuantAct.alloc(M, K, DEV)
    scr = F.GdnStepScratch(M, HV, nseq, DEV)
    lib = N.lib()
    ps = [F.gdn_step_params(x, x[:, C_:], x[:, C_ + K:], conv_w, A_log, dtb, norm_w, hists[i], states[i], stashes[i],
                            cu, slots, sh, scr, qa, HK * d, HK * d, HV, HK, n) for i in range(copies)]
    fns = [lambda p=p: N.check(lib.saber_gdn_step_launch(C.byref(p), nseq, N.stream_handle()), "gdn_step") for p in ps]
    nbytes = 2.0 * nseq * HV * d * d * 4
    _time(fns, f"gdn fused step nseq={nseq} rows={n} replay={shift}", nbytes)
    conv_out = torch.empty(M, C_, device=DEV)
    o = torch.empty(M, K, device=DEV)
    trio = []
    for i in range(copies):
        cp = F.gdn_conv_params(x, conv_w, hists[i], cu, slots, sh, conv_out, HK * d, HK * d, False, dual=True)
        rp = F.gdn_rec_params(conv_out, x[:, C_ + K:], A_log, dtb, states[i], stashes[i], cu, slots, sh, o, HK * d, HK * d, HV, HK, False)
        np_ = F.row_params(M, K, a_f32=o, b=x[:, C_:], w=norm_w, qa=qa, ldb=ld)
        def f(cp=cp, rp=rp, np_=np_):
            N.check(lib.saber_gdn_conv_launch(C.byref(cp), nseq, N.stream_handle()), "conv")
            N.check(lib.saber_gdn_recurrent_launch(C.byref(rp), nseq, 1, N.stream_handle()), "rec")
            N.check(lib.saber_row_producer_launch(N.ROW_GDN_NORM, C.byref(np_), N.stream_handle()), "norm")
        trio.append(f)
    _time(trio, f"gdn conv + recurrence (one slice per head) + norm_quant, three launches nseq={nseq} rows={n} replay={shift}", nbytes)
    return states, stashes, hists, x, qa, scr, conv_out, o


def _gdn_prefill(n, copies=3, form=1, chunk_impl=-1):
    """One sequence of n rows through the committing row-by-row form the prefill rungs use
    (chunk_impl >= 0: the 64-row chunked form instead, 0 = fp32, 1 = tensor cores)."""
    HV, HK, d = 48, 16, 128
    C_ = 2 * HK * d + HV * d
    qkv = torch.randn(n, C_, device=DEV) * 0.1
    ba = torch.randn(n, 2 * HV, device=DEV).to(torch.bfloat16)
    A_log, dtb = torch.randn(HV, device=DEV) * 0.5, torch.randn(HV, device=DEV) * 0.5
    states = [torch.randn(2, HV, d, d, device=DEV) * 0.01 for _ in range(copies)]
    stash = torch.zeros(2, 9, HV, 2, F.gdn_stash_stride(2), device=DEV)
    cu = torch.tensor([0, n], dtype=torch.int32, device=DEV)
    slots = torch.tensor([1], dtype=torch.int32, device=DEV)
    sh = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.empty(n, HV * d, device=DEV)
    ps = [F.gdn_rec_params(qkv, ba, A_log, dtb, st, stash, cu, slots, sh, out, HK * d, HK * d, HV, HK, True,
                           prefill_rows=form, chunk_impl=max(chunk_impl, 0)) for st in states]
    torch.cuda.synchronize()
    lib = N.lib()
    if chunk_impl >= 0:
        scr = F.gdn_chunk_scratch(n, 1, HV, DEV)
        fns = [lambda p=p: N.check(lib.saber_gdn_chunk_launch(C.byref(p), 1, n, scr.data_ptr(), N.stream_handle()), "gdn") for p in ps]
        _time(fns, f"gdn prefill chunked n={n} impl={chunk_impl}", n * (2 * HK * d + HV * d) * 4.0 + n * HV * d * 4.0)
        F.scratch(DEV).check()
        return states, out, scr
    fns = [lambda p=p: N.check(lib.saber_gdn_recurrent_launch(C.byref(p), 1, 2, N.stream_handle()), "gdn") for p in ps]
    _time(fns, f"gdn prefill rows n={n} form={form}", n * (2 * HK * d + HV * d) * 4.0 + n * HV * d * 4.0)
    return states, out


def _row(M, K, copies=3):
    xs = [torch.randn(M, K, device=DEV).to(torch.bfloat16) for _ in range(copies)]
    res = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = torch.randn(K, device=DEV) * 0.1
    qa = F.QuantAct.alloc(M, K, DEV)
    lib = N.lib()
    ps = [F.row_params(M, K, a=x, res=res, w=w, w_offset=1.0, qa=qa) for x in xs]
    fns = [lambda p=p: N.check(lib.saber_row_producer_launch(N.ROW_ADD_RMS, C.byref(p), N.stream_handle()), "row") for p in ps]
    _time(fns, f"row add_rms_quant M={M} K={K}", M * K * 7.0)
    return xs, res, qa


def _moe(M):
    from ..models import config as MC
    from ..models.moe_block import MoeWorkspace, add_moe_ops
    from ..models.moe_weights import random_moe_layer
    cfg = MC.flashnext_moe()
    g = torch.Generator(device=DEV).manual_seed(1)
    layers = [random_moe_layer(cfg, 1, 0, torch.device(DEV), g, 0.02) for _ in range(2)]
    qa = F.plain_quant(torch.randn(M, cfg.hidden, device=DEV).to(torch.bfloat16))
    ws = MoeWorkspace(cfg, cfg.moe.n_experts, M, DEV, layers[0]["shared_inter"])
    out = torch.zeros(M, cfg.hidden, dtype=torch.bfloat16, device=DEV)
    progs = []
    for i, moe in enumerate(layers):
        prog = N.Program(f"moe{i}")
        add_moe_ops(prog, ws, cfg, moe, qa, out, F.scratch(DEV), "moe")
        progs.append(prog)
    torch.cuda.synchronize()
    _time([p.run for p in progs] * 2, f"moe block (12 launches) M={M} experts={cfg.moe.n_experts} top_k={cfg.moe.top_k}")
    return layers, ws, out, progs


def _vision(side):
    """The full 27-block tower on one side x side image (side / 16 squared patch rows)."""
    from ..vision.tower import VisionConfig, VisionWeights
    from ..vision.tower_gpu import VisionTowerGPU
    cfg = VisionConfig.qwen38()
    tower = VisionTowerGPU(cfg, VisionWeights.random(cfg, seed=0), DEV, max_patches=(side // 16) ** 2)
    g = side // 16
    px = torch.randn(g * g, cfg.patch_row).pin_memory()
    out = torch.empty(g * g // 4, cfg.out_hidden, dtype=torch.bfloat16, device=DEV)
    tower.forward(px, [(1, g, g)], out=out)
    n0 = tower.launches
    _time([lambda: tower.forward(px, [(1, g, g)], out=out)] * 3,
          f"vision tower {side}x{side}: {g * g} patch rows -> {g * g // 4} tokens, {n0} launches")
    tower.forward(px, [(1, g, g)], out=out, graph=True)
    _time([lambda: tower.forward(px, [(1, g, g)], out=out, graph=True)] * 3, f"vision tower {side}x{side}, graph replay")
    return tower, out


CASES = {
    "gemm_w4_gate_up_m72": lambda: _gemm(34816, 5120, 72, 1, 1),
    "gemm_w4_down_m72_split": lambda: _gemm(5120, 17408, 72, 1, 7, copies=4),
    "gemm_w4_in_proj_m9_split": lambda: _gemm(10496, 5120, 9, 1, 3, copies=6),
    "gemm_w8_lm_head_m72": lambda: _gemm(248320, 5120, 72, 0, 1, copies=2),
    "gemm_nvfp4_gate_up_m64": lambda: _gemm_fp4(34816, 5120, 64, 4, 1),
    "gemm_nvfp4_down_m64_split": lambda: _gemm_fp4(5120, 17408, 64, 4, 7, copies=4),
    "gemm_nvfp4_in_proj_m64_split": lambda: _gemm_fp4(16640, 5120, 64, 4, 2, copies=4),
    "gemm_mxfp4_gate_up_m64": lambda: _gemm_fp4(34816, 5120, 64, 5, 1),
    "gemm_nvfp4_gate_up_m2048": lambda: _gemm_fp4(34816, 5120, 2048, 4, 1, copies=2),
    "gemm_w4_gate_up_m64": lambda: _gemm(34816, 5120, 64, 1, 1),
    "gemm_w4_gate_up_m2048": lambda: _gemm(34816, 5120, 2048, 1, 1, copies=2),
    "attn_decode_b8_ctx4096": lambda: _attn(8, 9, 4096, 4),
    "attn_decode_b1_ctx32768": lambda: _attn(1, 9, 32768, 32, copies=2),
    "attn_decode_b8_w8_ctx4096": lambda: _attn(8, 8, 4096, 9),
    "attn_decode_b8_w1_ctx4096": lambda: _attn(8, 1, 4096, 9),
    "attn_decode_b8_w5_ctx4096": lambda: _attn(8, 5, 4096, 4),
    "attn_tc_decode_b8_w8_ctx4096": lambda: _attn(8, 8, 4096, 4, impl=1),
    "attn_tc_decode_b8_w8_ctx4096_s2": lambda: _attn(8, 8, 4096, 2, impl=1),
    "attn_tc_decode_b8_w8_ctx4096_s1": lambda: _attn(8, 8, 4096, 1, impl=1),
    "attn_tc_decode_b1_w8_ctx32768": lambda: _attn(1, 8, 32768, 32, copies=2, impl=1),
    "attn_tc_decode_b1_w8_ctx131072": lambda: _attn(1, 8, 131072, 32, copies=2, impl=1),
    "attn_tc_prefill_2048_ctx4096": lambda: _attn(1, 2048, 2048, 1, impl=1),
    "gdn_rec_b8": lambda: _gdn(8, 9, 5),
    "gdn_step_b8_w8": lambda: _gdn_step(8, 8, 4),
    "gdn_step_b1_w8": lambda: _gdn_step(1, 8, 4),
    "gdn_prefill_2048": lambda: _gdn_prefill(2048),
    "gdn_prefill_2048_one_row": lambda: _gdn_prefill(2048, form=2),
    "gdn_prefill_2048_chunk_tc": lambda: _gdn_prefill(2048, chunk_impl=1),
    "gdn_prefill_512_chunk_tc": lambda: _gdn_prefill(512, chunk_impl=1),
    "gdn_prefill_512": lambda: _gdn_prefill(512),
    "gdn_prefill_512_one_row": lambda: _gdn_prefill(512, form=2),
    "gemm_w8_2sm_gate_up_m2048": lambda: _gemm_2sm(34816, 5120, 2048),
    "gemm_w8_2sm_down_m2048": lambda: _gemm_2sm(5120, 17408, 2048),
    "row_add_rms_m72": lambda: _row(72, 5120),
    "row_add_rms_m2048": lambda: _row(2048, 5120),
    "moe_block_m72": lambda: _moe(72),
    "vision_tower_512": lambda: _vision(512),
    "vision_tower_1024": lambda: _vision(1024),
}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True, choices=sorted(CASES) + ["all"])
    args = ap.parse_args(argv)
    for name in (sorted(CASES) if args.case == "all" else [args.case]):
        keep = CASES[name]()        # keep the operands alive until the launches have finished
        torch.cuda.synchronize()
        del keep
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
