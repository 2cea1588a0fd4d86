"""Per-op device timing of a bucket (the role of the reference's per-op timing arms,
`crates/saber-engine/src/host_trace.rs:5-12` device attribution): walks the program eagerly, one op
at a time, with CUDA events around each launch, and aggregates by op family.  Numbers are for
attribution (shares), never published as step times: an eager walk serialises launches."""
from __future__ import annotations

import re
from collections import defaultdict

import torch

from ..models.hybrid import Bucket, HybridModel, fill_blob


def profile_bucket(model: HybridModel, b: Bucket, seqs: list, repeats: int = 3) -> dict:
    fill_blob(b, seqs, model.cfg.page_tokens)
    st = model.stream
    prog = b.program
    tags = prog.tags()
    n = len(tags)
    acc = [0.0] * n
    with torch.cuda.stream(st):
        b.blob_dev.copy_(b.blob_host, non_blocking=True)
        for rep in range(repeats + 1):
            evs = [torch.cuda.Event(enable_timing=True) for _ in range(n + 1)]
            evs[0].record(st)
            for i in range(n):
                prog.run(st, i, i + 1)
                evs[i + 1].record(st)
            st.synchronize()
            if rep == 0:
                continue            # warm-up walk
            for i in range(n):
                acc[i] += evs[i].elapsed_time(evs[i + 1]) / repeats
    fam = defaultdict(lambda: [0.0, 0])
    for t, ms in zip(tags, acc):
        key = re.sub(r"^L\d+\.", "", t)
        key = re.sub(r"^draft\.L\d+\.", "draft.", key)
        fam[key][0] += ms
        fam[key][1] += 1
    total = sum(acc)
    rows = sorted(((k, v[0], v[1]) for k, v in fam.items()), key=lambda r: -r[1])
    return {"total_ms": total, "families": [{"op": k, "ms": ms, "count": c, "share": ms / total}
                                             for k, ms, c in rows]}


def format_profile(p: dict) -> str:
    lines = [f"eager per-op walk: {p['total_ms']:.3f} ms total"]
    for r in p["families"]:
        lines.append(f"  {r['op']:28s} {r['ms']:9.3f} ms  x{r['count']:<4d} {100 * r['share']:5.1f}%"
                     f"  ({1e3 * r['ms'] / r['count']:8.1f} us each)")
    return "\n".join(lines)


def main(argv=None) -> int:
    """`python -m saber_engine_b200.runtime.profile --batch 8`: build the model, replay the decode
    bucket a few times and bracket ONE replay with cudaProfilerStart/Stop (for
    `ncu --profile-from-start off`), or print the eager per-op walk with --walk."""
    import argparse
    from ..models import config as C
    from ..models.hybrid import SeqStep, run_bucket
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen38-27b")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--width", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--walk", action="store_true")
    ap.add_argument("--prefill", type=int, default=0, help="profile a prefill bucket of this many rows instead")
    args = ap.parse_args(argv)
    import os
    cfg = C.by_name(args.model)
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    comm = None
    torch.cuda.set_device(local)
    if world > 1:       # under torchrun: the tensor-parallel shard of every rank, walked in lock step
        import torch.distributed as dist
        from ..parallel.symm import SymmetricComm
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        rows_max = max(args.prefill, args.batch * args.width, 128)
        comm = SymmetricComm(rank, world, torch.device("cuda", local), max_elems=rows_max * cfg.hidden,
                             rows_max=rows_max, hidden=cfg.hidden)
    model = HybridModel(cfg, tp=world, rank=rank, device=torch.device("cuda", local), max_seqs=args.batch,
                        max_ctx=args.ctx + 512, max_width=args.width, seed=1, oracle_p=0.75, comm=comm)
    bp = (args.ctx + 512) // cfg.page_tokens
    b = model.build_bucket("decode", args.batch, args.width)
    g = torch.Generator().manual_seed(3)
    seqs = [SeqStep(torch.randint(0, cfg.vocab, (args.width,), generator=g).tolist(), args.ctx, j + 1, 3,
                    list(range(1 + j * bp, 1 + (j + 1) * bp)), uid=j) for j in range(args.batch)]
    if args.prefill:
        b = model.build_bucket("prefill", 1, args.prefill)
        seqs = [SeqStep(torch.randint(0, cfg.vocab, (args.prefill,), generator=g).tolist(), args.ctx - args.prefill, 1, 0,
                        list(range(1, 1 + bp)), uid=0)]
    if args.walk:
        prof = profile_bucket(model, b, seqs)
        if rank == 0:
            print(format_profile(prof))
        if world > 1:
            torch.distributed.barrier()
            torch.distributed.destroy_process_group()
        return 0
    for _ in range(2):
        run_bucket(model, b, seqs)
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    run_bucket(model, b, seqs)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print("profiled one replay:", b.n_launches, "launches")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
