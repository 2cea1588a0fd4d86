"""The `saber` command: models | serve | engine | explain | tune | pack | probe | bench | tp-gate | gate.

Everything the engine needs arrives as explicit flags or in the plan: no environment variables on
the engine path (only the model front door reads HOME / XDG_* / SABER_PACKS / HF_ENDPOINT).

Parity: `crates/saber-cli/src/main.rs:153-3603` (subcommands), `:22-28` (no env on the engine path),
`docs/MODELS.md:8-17` (front door), `crates/saber-cli/src/explain.rs`.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def _ints(s: str) -> tuple:
    return tuple(int(x) for x in s.split(",") if x)


# ------------------------------------------------------------------------------------------ models
def cmd_models(a) -> int:
    from ..registry import registry as R
    try:
        reg = R.load()
        if a.action == "list":
            rows = []
            for m in reg.models.values():
                rows.append({"name": m.name, "kind": m.kind, "aliases": m.aliases, "tp": sorted(m.tp),
                             "present": {t: (R.pack_dir(m, t, a.packs_dir) / "manifest.json").exists() for t in m.tp},
                             "default": m.name == reg.default})
            if a.json:
                print(json.dumps(rows, indent=1))
            else:
                for r in rows:
                    have = ",".join(f"tp{t}" for t, ok in r["present"].items() if ok) or "-"
                    print(f"{'*' if r['default'] else ' '} {r['name']:34s} {r['kind']:8s} tp {r['tp']}  on disk: {have}  aliases: {', '.join(r['aliases'])}")
        elif a.action == "info":
            m = reg.resolve(a.name)
            d = {"name": m.name, "kind": m.kind, "description": m.description, "repo": m.repo, "license": m.license,
                 "requires_tag": m.requires_tag, "drafter": m.drafter,
                 "tp": {t: vars(e) | {"pack_dir": str(R.pack_dir(m, t, a.packs_dir))} for t, e in m.tp.items()}}
            print(json.dumps(d, indent=1, default=str) if a.json else "\n".join(f"{k}: {v}" for k, v in d.items()))
        elif a.action == "pull":
            print(json.dumps(R.pull(reg, a.name, a.tp, a.packs_dir, a.dry_run), indent=1))
        elif a.action == "rm":
            for p in R.remove(reg, a.name, a.tp, a.packs_dir, a.dry_run):
                print(("would remove " if a.dry_run else "removed ") + p)
        return 0
    except R.RegistryError as exc:
        for p in exc.problems:
            print(f"saber: {p}", file=sys.stderr)
        return 2


# ------------------------------------------------------------------------------------------ serve
def cmd_serve(a, extra) -> int:
    from ..registry import registry as R
    try:
        plan = R.plan_serve(R.load(), a.model, a.tp, a.port, a.packs_dir, extra)
    except R.RegistryError as exc:
        for p in exc.problems:
            print(f"saber: {p}", file=sys.stderr)
        return 2
    if a.print_argv:
        print(" ".join(plan["argv"]))
        return 0
    if a.dry_run:
        print(json.dumps(plan, indent=1))
        return 0
    argv = plan["argv"][1:]
    if not plan["pack_present"] and not a.random_init:
        print(f"saber: no pack at {plan['pack_dir']} (pull it, or pass --random-init to serve seeded random weights)",
              file=sys.stderr)
        return 2
    if a.random_init:
        argv += ["--random-init"]
    return main(argv)


def build_engine(a):
    """Executor + scheduler for `saber engine` (also used by tests)."""
    from ..sched.scheduler import Scheduler, SchedulerConfig
    from ..serve.sampler import HostSampler
    if a.engine == "mock":
        from ..sched.mock import NullExecutor
        ex = NullExecutor(vocab=a.mock_vocab, max_seqs=a.engine_max_seqs, decode_widths=_ints(a.engine_decode_widths),
                          decode_batches=_ints(a.engine_decode_batches))
    elif a.engine == "tiny":
        from ..models.tiny_qwen3 import TinyExecutor
        ex = TinyExecutor(max_seqs=a.engine_max_seqs)
    else:
        import torch
        from ..models import config as MC
        from ..models.hybrid import HybridModel
        from ..runtime.hybrid_executor import HybridExecutor
        cfg = MC.by_name(a.engine_config)
        widths = _ints(a.engine_decode_widths)
        # several GPUs: one process per GPU (torchrun or the self-launch in cmd_engine); rank 0 plans
        # and serves, the other ranks follow its executor calls (parallel/tp_serve.py)
        rank, comm, dev = 0, None, "cuda"
        if a.engine_tp > 1:
            import os
            import torch.distributed as dist
            from ..parallel.symm import SymmetricComm
            from ..parallel.tp_serve import init_control_group
            rank, local = int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", os.environ["RANK"]))
            if int(os.environ["WORLD_SIZE"]) != a.engine_tp:
                raise SystemExit(f"--engine-tp {a.engine_tp} needs {a.engine_tp} ranks, got {os.environ['WORLD_SIZE']}")
            torch.cuda.set_device(local)
            dev = torch.device("cuda", local)
            dist.init_process_group("nccl", device_id=dev)
            a._tp_group = init_control_group(timeout_s=7 * 86400.0)   # followers idle between requests
            rows_max = max(max(_ints(a.engine_prefill_rows)), a.engine_max_seqs * max(widths), 128)
            comm = SymmetricComm(rank, a.engine_tp, dev, max_elems=rows_max * cfg.hidden, rows_max=rows_max, hidden=cfg.hidden)
            if getattr(a, "vision", False):
                raise SystemExit("--vision serves from one GPU only")
        a._tp_rank = rank
        # ---- one resolved plan drives the engine: buckets, the KV pool (budget - billed), tuned routes
        from ..plan import launch_plan as LP
        from ..utils.host_trace import StartupLedger
        boot = StartupLedger()
        with boot.phase("plan"):
            if getattr(a, "manifest", None):
                man = LP.Manifest.from_toml(Path(a.manifest).read_text())
                if man.tp != a.engine_tp:
                    raise SystemExit(f"saber: the manifest is for tp {man.tp} but the engine runs tp {a.engine_tp}")
            else:
                man = LP.Manifest(model=a.engine_config, pack=a.pack, tp=a.engine_tp, max_ctx=a.engine_max_ctx,
                                  max_seqs=a.engine_max_seqs, decode_batches=tuple(_ints(a.engine_decode_batches)),
                                  decode_widths=tuple(widths), prefill_rows=tuple(_ints(a.engine_prefill_rows)),
                                  draft_block=a.engine_draft_block, budget_mib=a.engine_budget_mib,
                                  prefix_cache_mib=a.prefix_cache_host_mib, autotune=a.autotune,
                                  allow_untuned=not getattr(a, "require_tuned", False))
            try:
                plan = LP.bind(LP.resolve(man, LP.DeviceProfile.measured()))
            except LP.PlanError as exc:
                for prob in exc.problems:
                    print(f"saber: {prob}", file=sys.stderr)
                raise SystemExit(2)
            a._plan = plan
            cfg = MC.by_name(man.model)
            widths = list(man.decode_widths)
        weights = None
        with boot.phase("weights"):
            if a.pack and not a.random_init:
                from ..pack.build import load_weights
                weights = load_weights(a.pack, cfg, a.engine_tp, rank, dev)
        with boot.phase("model"):
            kv_blocks = a.engine_kv_blocks or plan.kv_blocks            # the ledger's pool unless a count is forced
            model = HybridModel(cfg, tp=a.engine_tp, rank=rank, device=dev, max_seqs=man.max_seqs, comm=comm,
                                max_ctx=man.max_ctx, kv_blocks=kv_blocks, max_width=max(widths),
                                weights=weights, seed=a.seed, race_check=a.engine_race_check,
                                gdn_prefill=getattr(a, "engine_gdn_prefill", "tc"),
                                prefill_w8=bool(getattr(man, "prefill_w8", True)),
                                image_rows=(getattr(a, "vision_arena_patches", 0) // 4 if getattr(a, "vision", False) else 0))
            if man.autotune:
                from ..plan.autotune import TuneTable
                model.tune_table = TuneTable.load(man.autotune)
        with boot.phase("buckets"):
            ex = HybridExecutor(model, list(man.decode_batches), widths, list(man.prefill_rows), prebuild=a.prebuild)
        ex.startup = boot
        ex.plan_hash = plan.plan_hash
        if a.engine_tp > 1:
            from ..parallel.tp_serve import TpLeaderExecutor, follower_loop
            if rank != 0:                # a follower never returns from here until the leader stops it
                import os
                channel = alive = None
                if getattr(a, "ctrl_line", None):
                    from ..parallel.control_frames import ShmChannel
                    from ..parallel.launcher import parent_alive
                    channel, alive = ShmChannel(a.ctrl_line, a.engine_tp, rank, create=False), parent_alive(os.getppid())
                follower_loop(ex, a._tp_group, channel=channel, alive=alive)
                import torch.distributed as dist
                dist.destroy_process_group()
                raise SystemExit(0)
            ex = TpLeaderExecutor(ex, a._tp_group, channel=getattr(a, "_ctrl_channel", None))
    if a.engine_tp > 1 and getattr(a, "prompt_cache_dir", None):
        # (parked sessions work on several ranks: every rank keeps its shard under the leader's park id, in the
        # memory of the running process group; a prompt cache on a drive would outlive that group)
        raise SystemExit("saber: --prompt-cache-dir holds one rank's shard only: not available with --engine-tp > 1")
    from ..sched.width import WidthByBatch
    wt = WidthByBatch.parse(a.engine_width_table, captured=tuple(_ints(a.engine_decode_widths))) if getattr(a, "engine_width_table", "") else None
    cfg_s = SchedulerConfig(max_seqs=a.engine_max_seqs, max_ctx=a.engine_max_ctx, prefix_cache=not a.no_prefix_cache,
                            prefix_cache_bytes=a.prefix_cache_host_mib << 20, model_name=a.served_model_name,
                            width_table=wt, width_policy=getattr(a, "engine_width_policy", "table"),
                            lookup_drafts=bool(getattr(a, "engine_lookup_drafts", False)),
                            park_victims=bool(getattr(a, "engine_park_victims", False)),
                            mixed_steps=not getattr(a, "no_mixed_steps", False),
                            mixed_chunk_rows=getattr(a, "engine_mixed_chunk_rows", 512))
    if getattr(a, "engine_mem_valve", False):
        from ..sched.mem_valve import MemValve
        cfg_s.mem_valve = MemValve()
    sched = Scheduler(ex, cfg_s, sampler=HostSampler())
    from ..sched.park import ParkTier
    from ..utils.host_trace import HostTrace, StepLedger
    sched.trace = HostTrace(bool(getattr(a, "engine_host_trace", False)))
    sched.park_tier = ParkTier(getattr(a, "park_ram_mib", 8192) << 20, getattr(a, "park_dir", None))
    if getattr(a, "prompt_cache_dir", None):
        from ..sched.prompt_store import PromptStore
        sched.prompt_store = PromptStore(a.prompt_cache_dir, page=ex.page_tokens)
    ledger = StepLedger(getattr(a, "step_trace", None))
    sched.step_ledger = ledger
    fail = getattr(a, "fail_rank_after_steps", None)
    fail_rank, fail_n = (int(x) for x in fail.split(":")) if fail else (None, None)

    def on_step(info):
        ledger.record(info["kind"], info["live"], info["seconds"])
        if fail_n is not None and sched.counters["steps"] >= fail_n:     # host-side fault injection
            from ..serve import fatal
            sched.set_fatal(f"rank {fail_rank} failed after {fail_n} steps (injected)")
            fatal.set_fatal(fail_rank, f"failed after {fail_n} steps (injected)", exit_process=True,
                            watchdog_s=getattr(a, "fatal_watchdog_s", 10.0))
    sched.on_step = on_step
    poison = getattr(a, "poison_boot", None)
    if poison is not None and hasattr(ex, "model"):
        from ..runtime.race_check import poison_arenas
        build = ex.model.build_bucket

        def build_poisoned(*args, **kw):
            fresh = tuple(args[:3]) not in ex.model.buckets
            b = build(*args, **kw)
            if fresh:
                poison_arenas(b, poison & 0xFF)
            return b
        ex.model.build_bucket = build_poisoned
    return ex, sched


def cmd_engine(a) -> int:
    import os
    holder = {"sched": None}
    if getattr(a, "engine", "") == "real" and getattr(a, "engine_tp", 1) > 1 and "RANK" not in os.environ:
        # self-launch: this process is rank 0, one watched child per further GPU, rendezvous on the
        # loopback address; the control frames go over one shared-memory line per follower
        from ..parallel.control_frames import ShmChannel
        from ..parallel.launcher import launch_followers
        from ..serve import fatal
        port = 29400 + (os.getpid() % 500)
        a.ctrl_line = f"/saber-ctl-{os.getpid()}"
        a._ctrl_channel = ShmChannel(a.ctrl_line, a.engine_tp, 0, create=True)

        def follower_died(rank: int, why: str) -> None:
            if holder["sched"] is not None:
                holder["sched"].set_fatal(why)
            fatal.set_fatal(rank, why, exit_process=True, watchdog_s=getattr(a, "fatal_watchdog_s", 10.0))
        a._ranks = launch_followers([sys.executable, "-m", "saber_engine_b200", *sys.argv[1:], "--ctrl-line", a.ctrl_line],
                                    a.engine_tp, port, follower_died)
    import uvicorn
    from ..serve.server import ServerState, create_app
    from ..serve.tokenizer import ByteCodec, HfTokenizer
    ex, sched = build_engine(a)
    holder["sched"] = sched
    tok = HfTokenizer(str(Path(a.tokenizer).parent)) if a.tokenizer and Path(a.tokenizer).exists() else ByteCodec(ex.vocab)
    template = Path(a.chat_template).read_text() if a.chat_template and Path(a.chat_template).exists() else None
    vision = None
    if getattr(a, "vision", False) and hasattr(ex, "model") and getattr(ex.model, "image_rows", 0) > 0:
        # the tower (random-init unless a pack carries it), its arena clamps the processor's pixel ceiling
        from ..vision.engine import VisionFrontend
        from ..vision.tower import VisionConfig, VisionWeights
        from ..vision.tower_gpu import VisionTowerGPU
        vcfg = VisionConfig.qwen38(out_hidden=ex.model.cfg.hidden)
        tower = VisionTowerGPU(vcfg, VisionWeights.random(vcfg, seed=a.seed), "cuda", max_patches=a.vision_arena_patches)
        pad = getattr(tok, "special_ids", {}).get("<|image_pad|>") if hasattr(tok, "special_ids") else None
        if pad is None:
            pad = tok.encode("<|image_pad|>")[0]
        vision = VisionFrontend(ex, tower, pad)
    state = ServerState(sched, tok, a.served_model_name, api_keys=a.api_key or (), chat_template=template,
                        census_fn=(lambda: dict(getattr(ex, "census", {}))), vision=vision)
    for path in getattr(a, "warm_prompt", []):
        ids = tok.encode(Path(path).read_text())
        sched.warm([ids])
    if getattr(ex, "startup", None) is not None or getattr(getattr(ex, "inner", None), "startup", None) is not None:
        boot = getattr(ex, "startup", None) or ex.inner.startup
        print("saber: ready; startup phases\n" + boot.render(), file=sys.stderr)
    sched.spawn_step_loop()
    try:
        uvicorn.run(create_app(state), host=a.host, port=a.port, log_level="warning")
    finally:
        sched.shutdown()
        if getattr(a, "_ranks", None) is not None:
            a._ranks.expect_exit()
        if hasattr(ex, "stop_followers"):
            ex.stop_followers()
        if getattr(a, "_ranks", None) is not None:
            a._ranks.wait()
            a._ctrl_channel.close()
    return 0


# ------------------------------------------------------------------------------------------ plan
def cmd_explain(a) -> int:
    from ..plan import launch_plan as LP
    try:
        man = LP.Manifest.from_toml(Path(a.manifest).read_text()) if a.manifest else LP.Manifest(
            model=a.model, tp=a.tp, allow_untuned=True, autotune=a.autotune)
        plan = LP.resolve(man, LP.DeviceProfile.measured())
        print(plan.explain())
        if a.bind:
            LP.bind(plan)
        return 0
    except LP.PlanError as exc:
        for p in exc.problems:
            print(f"saber: {p}", file=sys.stderr)
        return 2


def cmd_tune(a) -> int:
    """GEMM records first (a new table), then the decode attention's split counts into the same file."""
    from ..plan import tune_attn, tune_gemm
    ops = set((getattr(a, "ops", "") or "gemm,attn").split(","))
    rc = 0
    if "gemm" in ops:
        rc = tune_gemm.main(["--model", a.model, "--tp", str(a.tp), "--rows", a.rows, "--out", a.out])
    if rc == 0 and "attn" in ops:
        import os
        rc = tune_attn.main(["--model", a.model, "--tp", str(a.tp)] + (["--into", a.out] if os.path.exists(a.out) else ["--out", a.out]))
    return rc


def cmd_pack(a) -> int:
    from ..pack import format as PF
    if a.action == "build":
        from ..models import config as MC
        from ..pack.build import write_pack
        d = write_pack(MC.by_name(a.model), a.out, a.tp, a.seed, a.device)
        print(d)
        return 0
    problems = PF.check_manifest(a.dir)
    for p in problems:
        print(f"saber: {p}", file=sys.stderr)
    print("pack ok" if not problems else f"{len(problems)} problems")
    return 1 if problems else 0


def cmd_probe(a) -> int:
    import torch
    info = {"cuda": torch.cuda.is_available(), "gpus": torch.cuda.device_count() if torch.cuda.is_available() else 0}
    if info["cuda"]:
        p = torch.cuda.get_device_properties(0)
        info.update(name=p.name, sms=p.multi_processor_count, mem_gib=round(p.total_memory / 2 ** 30, 1),
                    capability=f"{p.major}.{p.minor}")
    from ..ops import native
    info["native_library"] = native.available()
    print(json.dumps(info, indent=1))
    return 0


def cmd_gate(a) -> int:
    import pytest
    return pytest.main(["-q", "-m", "gpu", str(Path(__file__).resolve().parents[2] / "tests")] + (["-k", a.k] if a.k else []))


def cmd_console(a) -> int:
    """The console: supervises `saber engine ...` as a child, proxies /v1 to it, keeps usage, audit and config history."""
    import urllib.request
    import uvicorn
    from ..console.app import Console
    from ..console.supervisor import Supervisor
    Path(a.data_dir).mkdir(parents=True, exist_ok=True)

    def ready() -> bool:
        try:
            with urllib.request.urlopen(f"{a.engine_url}/health", timeout=1) as r:
                return r.status == 200
        except OSError:
            return False
    sup = Supervisor(ready_probe=ready, ready_timeout_s=a.ready_timeout, history_path=str(Path(a.data_dir) / "history.json"))
    con = Console(sup, a.data_dir, a.engine_url, admin_token=a.admin_token, engine_bearer=a.engine_key)
    if a.engine_argv:
        if not sup.apply(a.engine_argv, note="boot"):
            print("saber console: the engine never reached ready", file=sys.stderr)
    try:
        uvicorn.run(con.app(), host=a.host, port=a.port, log_level="warning")
    finally:
        sup.stop()
        con.usage.close()
    return 0


def make_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="saber")
    sub = ap.add_subparsers(dest="cmd", required=True)
    m = sub.add_parser("models")
    m.add_argument("action", nargs="?", default="list", choices=["list", "info", "pull", "rm"])
    m.add_argument("name", nargs="?")
    m.add_argument("--tp", type=int)
    m.add_argument("--json", action="store_true")
    m.add_argument("--dry-run", action="store_true")
    m.add_argument("--yes", action="store_true")
    m.add_argument("--packs-dir")
    s = sub.add_parser("serve")
    s.add_argument("--model")
    s.add_argument("--tp", type=int)
    s.add_argument("--port", type=int, default=8000)
    s.add_argument("--dry-run", action="store_true")
    s.add_argument("--print-argv", action="store_true")
    s.add_argument("--packs-dir")
    s.add_argument("--random-init", action="store_true")
    e = sub.add_parser("engine")
    e.add_argument("--engine", default="real", choices=["real", "mock", "tiny"])
    e.add_argument("--engine-tp", type=int, default=1)
    e.add_argument("--pack")
    e.add_argument("--engine-config", default="qwen38-27b")
    e.add_argument("--engine-max-ctx", type=int, default=262144)
    e.add_argument("--engine-max-seqs", type=int, default=8)
    e.add_argument("--engine-prefill-rows", default="128,512,2048")
    e.add_argument("--engine-decode-batches", default="1,2,3,4,8")
    e.add_argument("--engine-decode-widths", default="1,5,8")
    e.add_argument("--engine-draft-block", type=int, default=8)
    e.add_argument("--engine-budget-mib", type=int, default=160000)
    e.add_argument("--engine-kv-blocks", type=int, default=0, help="force the KV block count (0: what the plan's ledger derives from the budget)")
    e.add_argument("--manifest", help="typed TOML manifest: replaces the bucket / limit flags (see examples/)")
    e.add_argument("--require-tuned", action="store_true", help="refuse to boot when a route has no measurement in the autotune table")
    e.add_argument("--engine-width-table", default="", help="verify width by batch, e.g. 1:8,4:5")
    e.add_argument("--engine-width-policy", default="table", choices=["table", "ema"])
    e.add_argument("--engine-lookup-drafts", action="store_true", help="prompt-lookup drafts for sequences without model drafts")
    e.add_argument("--engine-park-victims", action="store_true", help="park a decoding sequence when a waiting request does not fit")
    e.add_argument("--engine-mem-valve", action="store_true", help="host-memory pressure valve: demote, park, refuse")
    e.add_argument("--no-mixed-steps", action="store_true")
    e.add_argument("--engine-mixed-chunk-rows", type=int, default=512)
    e.add_argument("--served-model-name", default="saber")
    e.add_argument("--host", default="127.0.0.1")
    e.add_argument("--port", type=int, default=8000)
    e.add_argument("--tokenizer")
    e.add_argument("--chat-template")
    e.add_argument("--api-key", action="append")
    e.add_argument("--no-prefix-cache", action="store_true")
    e.add_argument("--prefix-cache-host-mib", type=int, default=6144)
    e.add_argument("--autotune")
    e.add_argument("--random-init", action="store_true")
    e.add_argument("--prebuild", action="store_true")
    e.add_argument("--seed", type=int, default=0)
    e.add_argument("--mock-vocab", type=int, default=1024)
    e.add_argument("--vision", action="store_true", help="load the vision tower and accept image parts in chat requests")
    e.add_argument("--vision-arena-patches", type=int, default=16384, help="patch rows the tower arena holds (larger images are downscaled)")
    e.add_argument("--engine-host-trace", action="store_true", help="named host phases per step (an attribution, not a published time)")
    e.add_argument("--engine-race-check", default="off", choices=["off", "shadow"])
    e.add_argument("--engine-gdn-prefill", default="tc", choices=["tc", "rows", "chunked"],
                   help="DeltaNet prefill: 64-row chunks on the tensor cores (default), the exact fp32 row-by-row "
                        "recurrence, or the fp32 chunked form")
    e.add_argument("--poison-boot", type=lambda v: int(v, 0), default=None, metavar="BYTE",
                   help="fill every activation arena with this byte when a bucket is built (write-before-read proof)")
    e.add_argument("--warm-prompt", action="append", default=[], metavar="FILE",
                   help="text file whose content is prefilled at boot so its pages are in the prefix cache")
    e.add_argument("--step-trace", metavar="PATH", help="append one JSON line per engine step")
    e.add_argument("--park-dir", help="drive tier of parked sessions")
    e.add_argument("--prompt-cache-dir", help="keep prefilled prefixes on this drive across restarts")
    e.add_argument("--park-ram-mib", type=int, default=8192)
    e.add_argument("--fatal-watchdog-s", type=float, default=10.0)
    e.add_argument("--ctrl-line", default=None, help=argparse.SUPPRESS)      # set by the self-launch for its followers
    e.add_argument("--fail-rank-after-steps", default=None, metavar="R:N", help=argparse.SUPPRESS)
    x = sub.add_parser("explain")
    x.add_argument("--manifest")
    x.add_argument("--model", default="qwen38-27b")
    x.add_argument("--tp", type=int, default=1)
    x.add_argument("--autotune")
    x.add_argument("--bind", action="store_true")
    t = sub.add_parser("tune")
    t.add_argument("--model", default="qwen38-27b")
    t.add_argument("--tp", type=int, default=1)
    t.add_argument("--rows", default="9,72")
    t.add_argument("--out", default="autotune.json")
    t.add_argument("--ops", default="gemm,attn", help="what to measure: gemm (a new table), attn (decode attention splits, added to the table)")
    p = sub.add_parser("pack")
    p.add_argument("action", choices=["build", "check"])
    p.add_argument("--model", default="hybrid-mini")
    p.add_argument("--tp", type=int, default=1)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--out", default="packs")
    p.add_argument("--dir")
    p.add_argument("--device", default="cpu")
    sub.add_parser("probe")
    c = sub.add_parser("console", help="supervisor + /v1 proxy + usage, audit and config history (then `--` and the engine's argv)")
    c.add_argument("--data-dir", required=True)
    c.add_argument("--engine-url", default="http://127.0.0.1:8090")
    c.add_argument("--host", default="127.0.0.1")
    c.add_argument("--port", type=int, default=8080)
    c.add_argument("--admin-token", default=None)
    c.add_argument("--engine-key", default=None)
    c.add_argument("--ready-timeout", type=float, default=600.0)
    c.add_argument("engine_argv", nargs=argparse.REMAINDER)
    g = sub.add_parser("gate")
    g.add_argument("-k")
    return ap


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    ap = make_parser()
    if argv and argv[0] == "serve":
        a, extra = ap.parse_known_args(argv)
        return cmd_serve(a, extra)
    if argv and argv[0] == "bench":
        import runpy
        sys.argv = ["bench.py"] + argv[1:]
        runpy.run_path(str(Path(__file__).resolve().parents[2] / "bench.py"), run_name="__main__")
        return 0
    if argv and argv[0] == "shadow":
        from ..shadow.__main__ import main as shadow_main
        return shadow_main(argv[1:])
    if argv and argv[0] == "tp-gate":
        from ..parallel import tp_gate
        return tp_gate.main(argv[1:])
    a = ap.parse_args(argv)
    return {"models": cmd_models, "engine": cmd_engine, "explain": cmd_explain, "tune": cmd_tune,
            "pack": cmd_pack, "probe": cmd_probe, "gate": cmd_gate, "console": cmd_console}[a.cmd](a)


if __name__ == "__main__":
    sys.exit(main())
