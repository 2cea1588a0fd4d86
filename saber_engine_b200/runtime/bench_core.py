"""Benchmark body shared by `bench.py` and `saber bench`: builds the model (random-init pack
layouts), prefills the streams, then times decode steps on the device.

Timing rules: warm-up steps first; CUDA events on the launching stream around the whole timed
region with a barrier + synchronize on both sides; the max over ranks is reported; clocks are
sampled with nvidia-smi while the region runs.  Every timed step streams the full weight set
(several GB, far beyond the 126 MB L2), so no explicit L2 flush is needed between iterations.
"""
from __future__ import annotations

import os
import time

import torch

from ..models import config as C
from ..models.hybrid import HybridModel, SeqStep, run_bucket


def _dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if n_gpus > 1 and world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} needs torchrun with {n_gpus} ranks (WORLD_SIZE={world})")
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, local, world


def _barrier(world: int):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def _max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def timed_decode(model: HybridModel, bucket, seqs_state: list, steps: int, warmup: int, world: int):
    """Runs warmup + steps decode steps over the given live sequences; returns (ms, tokens)."""
    def one_step():
        seqs = [SeqStep([s["last"]] + s["drafts"][: bucket.width - 1], s["pos"], s["slot"], s["shift"],
                        s["blocks"], uid=s["uid"], step_no=s["step"], blocks_key=("bench", s["uid"])) for s in seqs_state]
        res = run_bucket(model, bucket, seqs)
        n = 0
        for j, s in enumerate(seqs_state):
            c = res.n_commit[j]
            s["last"] = res.tokens[j][-1]
            s["drafts"] = res.drafts[j] if res.drafts[j] else [0] * (bucket.width - 1)
            s["pos"] += c
            s["shift"] = c
            s["step"] += 1
            n += c
        return n
    for _ in range(warmup):
        one_step()
    _barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record(model.stream)
    tokens = 0
    for _ in range(steps):
        tokens += one_step()
    e1.record(model.stream)
    _barrier(world)
    wall_ms = (time.perf_counter() - t0) * 1e3
    return e0.elapsed_time(e1), wall_ms, tokens


def e2e_through_engine(model: HybridModel, prompts: list, steps: int, warmup: int, world: int, W: int, rung: int,
                       max_ctx: int) -> dict:
    """The same decode metric through the public engine API: requests are submitted to a
    `Scheduler` over a `HybridExecutor` (continuous batching, prefix cache on, paged KV allocation)
    and `Scheduler.step()` is what is timed -- by wall clock, with a barrier and a device
    synchronize on both sides.  Every step builds the index tables on the host, copies them from
    pinned memory to the device, replays the captured bucket and reads the step's result back.
    All ranks run the same deterministic scheduler in lock step."""
    from ..sched.scheduler import Scheduler, SchedulerConfig
    from ..sched.width import WidthByBatch
    from ..serve.engine_api import EngineRequest, SamplingParams
    from .hybrid_executor import HybridExecutor
    n = len(prompts)
    ex = HybridExecutor(model, decode_batches=(n,), decode_widths=(1, W), prefill_rungs=(rung,))
    sched = Scheduler(ex, SchedulerConfig(max_seqs=n, max_ctx=max_ctx, prefix_cache=True,
                                          width_table=WidthByBatch({1: W}, captured=(1, W))))
    budget = (steps + warmup + 8) * W
    subs = [sched.submit(EngineRequest(p, SamplingParams(max_tokens=budget, ignore_eos=True))) for p in prompts]
    t_pre = time.perf_counter()
    while any(s.prefilling for s in sched.running) or sched.waiting:
        sched.step()
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t_pre
    for _ in range(warmup):
        sched.step()
    before = sched.counters["generation_tokens"]
    _barrier(world)
    t0 = time.perf_counter()
    for _ in range(steps):
        sched.step()
    _barrier(world)
    wall = time.perf_counter() - t0
    tokens = sched.counters["generation_tokens"] - before
    b = model.buckets[("decode", n, W)]
    import dataclasses
    hits = dataclasses.asdict(sched.prefix.stats) if dataclasses.is_dataclass(sched.prefix.stats) else {}
    for sub in subs:
        sched.abort(sub.seq_id)
    sched.step()
    return {"tokens": tokens, "wall_ms": wall * 1e3, "h2d": b.last_h2d_bytes, "d2h": b.out_host.numel() * 4,
            "prefill_s": prefill_s, "prefix_cache": hits, "live": n,
            "mixed_steps": sched.counters["mixed_steps"], "deferred_for_prefix": sched.counters["deferred_for_prefix"]}


def run_benchmark(args, ClockSampler):
    rank, local, world = _dist_setup(args.gpus)
    if getattr(args, "pdl", -1) >= 0:
        from ..ops import native as _N
        _N.set_pdl(args.pdl)
    dev = torch.device("cuda", local)
    cfg = C.by_name(args.model)
    streams, W = args.streams, args.width
    decode_budget = (args.warmup + args.steps + 8) * W * 2 + 64
    # the pool and every block table are sized for the model's full context (262,144 tokens per
    # sequence) unless --max-ctx says otherwise; the workload itself uses prompt + decode budget
    max_ctx = max(int(getattr(args, "max_ctx", 0) or cfg.max_ctx), args.prompt + decode_budget)
    comm = None
    if world > 1:
        from ..parallel.symm import SymmetricComm
        rows_max = max(args.rung, streams * W, 128)
        comm = SymmetricComm(rank, world, dev, max_elems=rows_max * cfg.hidden, rows_max=rows_max, hidden=cfg.hidden)
    t_build = time.perf_counter()
    model = HybridModel(cfg, tp=world, rank=rank, device=dev, max_seqs=streams, max_ctx=max_ctx,
                        max_width=W, seed=1234, comm=comm, oracle_p=args.accept_p, oracle_seed=99,
                        gdn_fused=(None if getattr(args, "gdn_fused", -1) < 0 else bool(args.gdn_fused)),
                        fuse=bool(getattr(args, "fuse", 1)), gdn_prefill=getattr(args, "gdn_prefill", "tc"),
                        prefill_w8=(None if getattr(args, "prefill_w8", -1) < 0 else bool(args.prefill_w8)),
                        sp_prefill=(None if getattr(args, "sp_prefill", -1) < 0 else bool(args.sp_prefill)))
    tuned = None
    table_path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                              "examples", f"autotune-b200-{cfg.name}-tp{world}.json")
    if os.path.exists(table_path) and not getattr(args, "no_tune_table", False):
        from ..plan.autotune import TuneTable
        model.tune_table = TuneTable.load(table_path)        # the committed device table of this model and degree
        tuned = os.path.basename(table_path)
    torch.cuda.synchronize()
    build_s = time.perf_counter() - t_build
    page = cfg.page_tokens
    blocks_per = (max_ctx + page - 1) // page
    g = torch.Generator().manual_seed(7)
    prefix = torch.randint(0, cfg.vocab, (args.shared_prefix,), generator=g).tolist()
    prompts = [prefix + torch.randint(0, cfg.vocab, (args.prompt - args.shared_prefix,), generator=g).tolist()
               for _ in range(streams)]

    # ---- prefill (device-timed per stream: TTFT of a cold 4k prompt, prefill tok/s)
    rung = min(args.rung, args.prompt)
    pb = model.build_bucket("prefill", 1, rung)
    state, ttft_ms = [], []
    for j in range(streams):
        blocks = list(range(1 + j * blocks_per, 1 + (j + 1) * blocks_per))
        slot = j + 1
        model.reset_slot(slot)
        _barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(model.stream)
        pos, res = 0, None
        while pos < args.prompt:
            n = min(rung, args.prompt - pos)
            res = run_bucket(model, pb, [SeqStep(prompts[j][pos:pos + n], pos, slot, 0, blocks)])
            pos += n
        e1.record(model.stream)
        torch.cuda.synchronize()
        ttft_ms.append(_max_over_ranks(e0.elapsed_time(e1), world))
        state.append(dict(last=res.tokens[0][0], drafts=res.drafts[0] or [0] * (W - 1), pos=args.prompt,
                          slot=slot, shift=0, blocks=blocks, uid=j, step=0))
    model.scratch.check()
    # first prefill includes lazy initialisation; report the median
    ttft_sorted = sorted(ttft_ms)
    ttft_p50 = ttft_sorted[len(ttft_sorted) // 2]
    prefill_tok_s = args.prompt / (ttft_p50 / 1e3)

    # ---- TTFT of a short prompt (512 tokens, one rung): the reference's TTFT p50 is a short-prompt figure
    short_ms = None
    if args.prompt >= 512:
        sbk = model.build_bucket("prefill", 1, 512)
        spare = list(range(1, 1 + blocks_per))
        samples = []
        for _ in range(3):
            model.reset_slot(streams)            # the last stream's slot; its state is rebuilt below
            _barrier(world)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(model.stream)
            run_bucket(model, sbk, [SeqStep(prompts[0][:512], 0, streams, 0, spare)])
            e1.record(model.stream)
            torch.cuda.synchronize()
            samples.append(_max_over_ranks(e0.elapsed_time(e1), world))
        short_ms = sorted(samples)[1]
        # put the borrowed slot and pages back: re-prefill stream 0 and the last stream
        for j in sorted({0, streams - 1}):
            blocks = list(range(1 + j * blocks_per, 1 + (j + 1) * blocks_per))
            model.reset_slot(j + 1)
            pos, res = 0, None
            while pos < args.prompt:
                n = min(rung, args.prompt - pos)
                res = run_bucket(model, pb, [SeqStep(prompts[j][pos:pos + n], pos, j + 1, 0, blocks)])
                pos += n
            state[j].update(last=res.tokens[0][0], drafts=res.drafts[0] or [0] * (W - 1), pos=args.prompt, shift=0, step=0)

    # ---- decode, all streams
    db = model.build_bucket("decode", streams, W)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    dev_ms, wall_ms, tokens = timed_decode(model, db, state, args.steps, args.warmup, world)
    clocks = sampler.stop() if rank == 0 else {}
    dev_ms = _max_over_ranks(dev_ms, world)
    wall_ms = _max_over_ranks(wall_ms, world)
    model.scratch.check()
    value = tokens / (dev_ms / 1e3)

    # ---- single stream side measurement (the reference's other headline)
    single = None
    if not args.no_single:
        sb = model.build_bucket("decode", 1, W)
        s_ms, s_wall, s_tok = timed_decode(model, sb, state[:1], args.steps, args.warmup, world)
        s_ms = _max_over_ranks(s_ms, world)
        single = dict(tok_s=s_tok / (s_ms / 1e3), ms_per_step=s_ms / args.steps, tokens=s_tok,
                      launches_per_step=sb.n_launches)
    # ---- end to end through the public engine API (fresh KV / state, same model and buckets)
    e2e = e2e_through_engine(model, prompts, args.steps, args.warmup, world, W, rung, max_ctx)
    kv_tokens = (model.kv_blocks - 1) * page
    e2e_wall = _max_over_ranks(e2e["wall_ms"], world)
    model.scratch.check()
    if rank != 0:
        return None
    lay = db.layout
    names = {"qwen38-27b": ("decode_tok_s_8streams_27b_w4a8", 642.0, 230.0, 5200.0),
             "flashnext-moe": ("decode_tok_s_8streams_flashnext_moe_w4a8", 420.2, 166.9, None),
             "flashnext-moe-mxfp4": ("decode_tok_s_8streams_flashnext_moe_mxfp4_experts", 420.2, 166.9, None),
             "flashnext-ref": ("decode_tok_s_8streams_flashnext_moe_w4a8", 420.2, 166.9, None)}
    dtype = {"iu8": "w4a8-int8 (bf16 activations)", "mxfp4": "mxfp4 weights x fp8 activations (bf16 residual stream)",
             "nvfp4": "nvfp4 weights x nvfp4 activations, block-scaled tensor-core MMA (bf16 residual stream)"}.get(
                 getattr(cfg, "weight_format", "iu8"), "w4a8-int8 (bf16 activations)")
    if cfg.moe is not None and getattr(cfg.moe, "expert_format", "iu8") == "mxfp4":
        dtype = "routed experts mxfp4 x fp8 rows; " + dtype + " elsewhere"
    metric, base8, base1, base_pre = names.get(cfg.name, (f"decode_tok_s_{streams}streams_{cfg.name}", None, None, None))
    return {
        "metric": metric, "value": value, "unit": "tok/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": (value / base8) if base8 and streams == 8 else None, "dtype": dtype, "data": "synthetic",
        "impl": "ours",
        "config": {"model": cfg.name, "global_batch": streams, "seq_len": args.prompt,
                   "parallelism": f"tp{world}", "verify_width": W, "accept_p": args.accept_p,
                   "decode_tokens_timed": tokens, "l2": "inputs larger than L2 (weights re-streamed every step)",
                   "shared_prefix": args.shared_prefix, "max_ctx": max_ctx, "kv_pool_tokens": kv_tokens,
                   "autotune_table": tuned},
        "clocks": clocks,
        "e2e": {"value": e2e["tokens"] / (e2e_wall / 1e3), "unit": "tok/s",
                "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                "ms_per_step": e2e_wall / args.steps, "tokens": e2e["tokens"],
                "api": "sched.Scheduler.submit/step over runtime.HybridExecutor (prefix cache on)",
                "prefill_s_all_streams": e2e["prefill_s"], "prefix_cache": e2e["prefix_cache"],
                "mixed_steps": e2e["mixed_steps"], "deferred_for_prefix": e2e["deferred_for_prefix"],
                "bucket_loop_tok_s": tokens / (wall_ms / 1e3)},
        "gpu_launches": db.n_launches * args.steps,
        "extra": {"single_stream": single, "ttft_p50_ms": ttft_p50, "ttft_512_tokens_ms": short_ms,
                  "ttft_512_vs_baseline_38ms": (38.0 / short_ms) if short_ms and cfg.name == "qwen38-27b" else None, "ttft_ms_all": ttft_ms,
                  "prefill_tok_s": prefill_tok_s, "prefill_vs_baseline": (prefill_tok_s / base_pre) if base_pre else None,
                  "single_stream_vs_baseline": (single["tok_s"] / base1) if single and base1 else None,
                  "launches_per_step": db.n_launches, "build_s": build_s,
                  "state_bytes": model.state_bytes()},
    }
