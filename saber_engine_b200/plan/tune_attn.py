"""Measured KV-split counts for the decode attention: `python -m saber_engine_b200.plan.tune_attn`.

One record per (sequences, rows per sequence, context) of the model's head geometry: the sweep times the
tcgen05 attention over a paged fp8 cache with each candidate split count (interleaved, the first sample
of each variant discarded: `plan.autotune.Sweeper`) and keeps the fastest; the launch rules' choice is the
reference variant, which a winner within 1 % loses to.  Records go into the same table file as the GEMM
records (`--into`), under the op name `attn_tc_decode`; `HybridModel.attn_splits` looks them up for the
context length it is given (the bucket's context hint) and falls back to the rules.

What the sweep can and cannot tell: it times the kernel alone, every launch streaming its own pages from
memory.  Measured on a B200 for the 27B geometry (24 query heads on 4 KV heads, 4096 keys): one sequence 24
splits (35-37 us), eight sequences 4 splits (77-82 us).  Inside the decode step the eight-sequence case runs in
41 us with the rules' 9 splits -- the streams of the benchmark share a 2048-token prefix, so most pages come
from L2 and more, smaller CTAs win -- and with the swept value the step got slower (10.65 -> 11.6 ms).  The
committed tables therefore carry no attention records; the tool is for workloads without shared prefixes.

Parity: the reference's autotune cache holds attention records beside its GEMM records
(`examples/autotune-gfx1201-210w.json`, `crates/saber-plan/src/autotune.rs:1-16`).
"""
from __future__ import annotations

import argparse
import ctypes as C

import torch

from ..models import config as MC
from ..models.config import shard
from ..ops import functional as F
from ..ops import layouts as L
from ..ops import native as N
from .autotune import Sweeper, TuneTable, build_hash, make_key

OP = "attn_tc_decode"


def candidates(nseq: int, nkv: int, group: int, width: int, ctx: int) -> dict:
    """Split counts worth timing: powers of two and the rules' pick, none with fewer than 128 keys per split."""
    from ..rules import default_rules
    ruled = default_rules().attn_decode_splits("tc", nseq, nkv, group, width)
    cands = sorted({s for s in (1, 2, 3, 4, 6, 8, 9, 12, 16, 24, 32, ruled) if s == 1 or ctx // s >= 128})
    return {f"s{s}": {"splits": s} for s in cands}, f"s{ruled}" if ruled in cands else "s1"


def tune_shape(nseq: int, width: int, ctx: int, nq: int, nkv: int, sweeper: Sweeper, dev):
    page = 16
    max_blocks = (ctx + width + page - 1) // page
    nblocks = nseq * max_blocks + 1
    page_bytes = nblocks * nkv * 2 * page * 256
    copies = max(2, min(16, -(-int(2.2 * 126e6) // page_bytes)))      # rotate caches: every launch streams its pages from memory
    # (keys and values of unit scale: random bytes would be e4m3 values up to 240, scores that leave the range
    # of the probabilities, and a kernel that repeats its probability pass on every tile)
    caches = [(torch.randn(nblocks, nkv, 2, page, 256, device=dev) * 0.7).to(torch.float8_e4m3fn).view(torch.uint8)
              for _ in range(copies)]
    bt = (torch.arange(nseq * max_blocks, dtype=torch.int32, device=dev) + 1).reshape(nseq, max_blocks)
    M = nseq * width
    q = (torch.randn(M, nq, 256, device=dev) * 0.7).to(torch.bfloat16)
    out = torch.empty_like(q)
    cu = torch.arange(0, M + 1, width, dtype=torch.int32, device=dev)
    kv_len = torch.full((nseq,), ctx + width, dtype=torch.int32, device=dev)
    cands, ref = candidates(nseq, nkv, nq // nkv, width, ctx)
    stream = torch.cuda.Stream()

    def make_runner(v):
        """A captured graph with one launch per cache copy: a replay times the kernel back to back, no host gap inside."""
        s = v["splits"]
        po = torch.empty(nseq, nq, s, 16, 256, dtype=torch.float32, device=dev) if s > 1 else None
        pm = torch.empty(nseq, nq, s, 16, 2, dtype=torch.float32, device=dev) if s > 1 else None
        prog = N.Program(f"tune-attn-s{s}")
        for c in caches:
            prog.attn(F.attn_params(q, c, bt, cu, kv_len, out, po, pm, nkv, s, 1, pack_rows=width, impl=1), tag="attn")
        prog.keep(caches, q, out, bt, cu, kv_len, po, pm)
        with torch.cuda.stream(stream):
            prog.capture(stream)
        stream.synchronize()

        def run():
            prog.replay()
        return run

    rec = sweeper.sweep(make_key(OP, nseq=nseq, width=width, ctx=ctx, nq=nq, nkv=nkv), cands, make_runner, ref)
    F.scratch(dev).check()
    rec.measured_us /= copies
    if rec.runner_up_us is not None:
        rec.runner_up_us /= copies
    rec.variant["gbps"] = nseq * nkv * (ctx + width) * 512 / rec.measured_us / 1e3
    return rec


def lookup(table, nseq: int, width: int, ctx: int, nq: int, nkv: int):
    """The measured split count for this shape at the nearest tuned context not above `ctx` (or None)."""
    if table is None:
        return None
    best = None
    for c in (1024, 4096, 16384, 65536, 262144):
        if c <= max(ctx, 1024):
            hit = table.lookup(OP, nseq=nseq, width=width, ctx=c, nq=nq, nkv=nkv)
            if hit is not None:
                best = int(hit.get("splits", 1))
    return best


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen38-27b")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--batches", default="1,8")
    ap.add_argument("--widths", default="1,5,8")
    ap.add_argument("--contexts", default="4096,65536")
    ap.add_argument("--into", default="", help="an existing table file to add the records to (else --out is written alone)")
    ap.add_argument("--out", default="tune_attn.json")
    ap.add_argument("--samples", type=int, default=7)
    args = ap.parse_args(argv)
    dev = torch.device("cuda")
    cfg = MC.by_name(args.model)
    sh = shard(cfg, args.tp, 0)
    table = TuneTable.load(args.into) if args.into else TuneTable(torch.cuda.get_device_name(dev), build_hash())
    sw = Sweeper(samples=args.samples, batch=1)
    ints = lambda s: [int(x) for x in s.split(",") if x]      # noqa: E731
    for ctx in ints(args.contexts):
        for b in ints(args.batches):
            for w in ints(args.widths):
                rec = tune_shape(b, w, ctx, sh.n_q_heads, sh.n_kv_heads, sw, dev)
                table.put(rec)
                print(f"attn b={b} w={w} ctx={ctx:6d}: {rec.variant['name']:4s} {rec.measured_us:8.1f} us  "
                      f"{rec.variant['gbps']:6.0f} GB/s  runner-up {(rec.runner_up_us or float('nan')):.1f} us"
                      f"{'' if rec.stable else '  UNSTABLE'}", flush=True)
    table.save(args.into or args.out)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
