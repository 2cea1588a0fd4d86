"""`saber tune` body for the integer GEMM: sweeps (split-K, ring depth) per (N, K, M, w4) shape of a
model and records the winners in a TuneTable.

Each candidate is timed over a ring of weight copies larger than L2 (126 MB), because in the model
every layer streams its own weights: a single 16 MB weight timed alone would sit in L2 and lie.

    python -m saber_engine_b200.plan.tune_gemm --model qwen38-27b --tp 1 --rows 9,72 --out tune.json
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import math

import torch

from ..models import config as MC
from ..ops import functional as F
from ..ops import layouts as L
from ..ops import native as N
from .autotune import Sweeper, TuneTable, build_hash, make_key

L2_BYTES = 126 * 1024 * 1024


def model_gemm_shapes(cfg, tp: int) -> list:
    """(name, N, K, w4) of every distinct linear of one rank."""
    sh = MC.shard(cfg, tp, 0)
    H = cfg.hidden
    out = [("gdn.in_proj", sh.gdn_in_n, H, 1), ("gdn.out_proj", H, sh.gdn_out_k, 1),
           ("attn.qkv", sh.qkv_n, H, 1), ("attn.o_proj", H, sh.o_k, 1)]
    if cfg.moe is None:
        out += [("mlp.gate_up", 2 * sh.ffn_inter, H, 1), ("mlp.down", H, sh.ffn_inter, 1)]
    out += [("lm_head", sh.vocab, H, 0 if cfg.lm_head_bits == 8 else 1)]
    return out


def candidates(n_tiles: int, m_tiles: int, kb: int, nt: int, w4: int = 1) -> dict:
    out = {}
    for s in (1, 2, 3, 4, 5, 6, 7, 8):          # the kernel's split-K ceiling is 8
        if s > kb or (s - 1) * math.ceil(kb / s) >= kb:
            continue
        if n_tiles * m_tiles * s > 148 * 24 or (s > 1 and n_tiles * m_tiles * s > 148):
            continue
        for st in ((4, 8) if w4 else (3, 5)):
            if N.lib().saber_gemm_i8_smem_bytes_w(nt, st, w4) > 224 * 1024:
                continue
            out[f"s{s}_st{st}"] = {"splits": s, "stages": st, "halves": 1}
    if w4 == 1 and 148 // 4 < n_tiles * m_tiles <= 148 // 2:
        out["halves_st8"] = {"splits": 1, "stages": 8, "halves": 2}     # two CTAs per weight tile instead of split-K
    return out


def tune_shape(Nn: int, K: int, M: int, w4: int, sweeper: Sweeper, dev) -> "TuneRecord":
    n_pad = L.round_up(Nn, L.TILE_N)
    wbytes = n_pad * K // (2 if w4 else 1)
    copies = max(2, min(24, math.ceil(2.2 * L2_BYTES / wbytes)))
    tiles = [torch.randint(0, 255, (n_pad // L.TILE_N, K // 128, 16384 if w4 else 32768), dtype=torch.uint8, device=dev)
             for _ in range(copies)]
    scale = torch.rand(n_pad, device=dev) * 1e-3
    ws = [F.QuantWeight(t, scale, Nn, K, bool(w4)) for t in tiles]
    x = torch.randn(M, K, device=dev).to(torch.bfloat16)
    qa = F.plain_quant(x)
    out = torch.empty(M, (Nn + 7) // 8 * 8, dtype=torch.bfloat16, device=dev)[:, :Nn]      # rows 16-byte aligned, as the model's buffers are
    nt = L.token_tile(M)
    m_tiles = (M + nt - 1) // nt
    cands = candidates(n_pad // L.TILE_N, m_tiles, K // 128, nt, w4)
    sc = F.scratch(dev)
    lib = N.lib()

    stream = torch.cuda.Stream()

    def make_runner(v):
        """A captured graph holding one launch per weight copy: replaying it times the kernel
        back to back without any host gap inside the measured interval."""
        prog = N.Program(f"tune-s{v['splits']}-st{v['stages']}")
        for w in ws:
            prog.gemm(F.gemm_params(w, qa, out, sc, splits=v["splits"], halves=v.get("halves", 1)), v["stages"], tag="gemm")
        prog.keep(ws, qa, out)
        with torch.cuda.stream(stream):
            prog.capture(stream)
        stream.synchronize()

        def run():
            prog.replay()
        run.launches = len(ws)
        return run

    # one checked launch per candidate first: a variant whose bounded waits run out is dropped
    for name in list(cands):
        make_runner(cands[name])()
        torch.cuda.synchronize()
        code = int(sc.err.item())
        if code != 0:
            sc.err.zero_()
            sc.ws.zero_()
            sc.counters.zero_()
            print(f"  dropped {name} (N={Nn} K={K} M={M} w4={w4}): {N.ERR_NAMES.get(code, code)}", flush=True)
            del cands[name]
    default_s = F.pick_splits(n_pad // L.TILE_N, m_tiles, K // 128)
    ref = next((k for k, v in cands.items() if v["splits"] == default_s), next(iter(cands)))
    rec = sweeper.sweep(make_key("gemm_i8", N=n_pad, K=K, M=M, w4=w4), cands, make_runner, ref)
    sc.check()
    rec.measured_us /= len(ws)                 # a sample is one replay = one launch per weight copy
    if rec.runner_up_us is not None:
        rec.runner_up_us /= len(ws)
    rec.variant["gbps"] = wbytes / rec.measured_us / 1e3
    return rec


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen38-27b")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--rows", default="9,72")
    ap.add_argument("--out", default="tune.json")
    ap.add_argument("--samples", type=int, default=7)
    ap.add_argument("--one", default="", help="N,K,M,w4,splits,stages: launch that one variant a few "
                    "times over rotating weight copies and exit (the small case profilers capture)")
    args = ap.parse_args(argv)
    dev = torch.device("cuda")
    if args.one:
        Nn, K, M, w4, splits, stages = [int(x) for x in args.one.split(",")]
        n_pad = L.round_up(Nn, L.TILE_N)
        ws = [F.QuantWeight(torch.randint(0, 255, (n_pad // L.TILE_N, K // 128, 16384 if w4 else 32768),
                                          dtype=torch.uint8, device=dev),
                            torch.rand(n_pad, device=dev) * 1e-3, Nn, K, bool(w4)) for _ in range(4)]
        qa = F.plain_quant(torch.randn(M, K, device=dev).to(torch.bfloat16))
        out = torch.empty(M, (Nn + 7) // 8 * 8, dtype=torch.bfloat16, device=dev)[:, :Nn]      # rows 16-byte aligned, as the model's buffers are
        for i in range(6):
            pr = F.gemm_params(ws[i % 4], qa, out, F.scratch(dev), splits=splits)
            N.check(N.lib().saber_gemm_i8_launch(C.byref(pr), stages, N.stream_handle()), "gemm")
        torch.cuda.synchronize()
        F.scratch(dev).check()
        print("ok")
        return 0
    cfg = MC.by_name(args.model)
    table = TuneTable(torch.cuda.get_device_name(dev), build_hash())
    sw = Sweeper(samples=args.samples, batch=1)
    for name, Nn, K, w4 in model_gemm_shapes(cfg, args.tp):
        for M in [int(r) for r in args.rows.split(",")]:
            rec = tune_shape(Nn, K, M, w4, sw, dev)
            table.put(rec)
            print(f"{name:14s} N={Nn:6d} K={K:5d} M={M:4d} w4={w4}: {rec.variant['name']:10s} "
                  f"{rec.measured_us:8.1f} us  {rec.variant['gbps']:7.0f} GB/s  runner-up {(rec.runner_up_us if rec.runner_up_us is not None else float('nan')):.1f} us"
                  f"{'' if rec.stable else '  UNSTABLE'}", flush=True)
    table.save(args.out)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
