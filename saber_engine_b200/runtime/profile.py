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
