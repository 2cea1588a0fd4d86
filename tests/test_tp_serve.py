"""Leader / follower executors over a gloo group: two CPU processes, the device mock on both."""
import os
import sys

import pytest

_CHILD = r'''
import json, os, sys
import torch.distributed as dist
from saber_engine_b200.parallel.tp_serve import TpLeaderExecutor, follower_loop, init_control_group
from saber_engine_b200.sched.mock import NullExecutor
from saber_engine_b200.sched.scheduler import Scheduler, SchedulerConfig
from saber_engine_b200.serve.engine_api import EngineRequest, SamplingParams

rank = int(os.environ["RANK"])
dist.init_process_group("gloo", init_method=os.environ["INIT"], rank=rank, world_size=2)
group = init_control_group(60)
ex = NullExecutor(seed=3, vocab=500, max_seqs=4)
if rank == 0:
    lead = TpLeaderExecutor(ex, group)
    s = Scheduler(lead, SchedulerConfig(max_seqs=4, max_ctx=2048, prefix_cache_min_tokens=32, prefix_cache_interval=64))
    shared = list(range(100, 260))
    subs = [s.submit(EngineRequest(shared + [7, 8, 9 + i], SamplingParams(max_tokens=12))) for i in range(3)]
    s.run_until_idle()
    late = s.submit(EngineRequest(shared + [1, 2, 3], SamplingParams(max_tokens=5)))     # a prefix-cache hit: restore on both ranks
    s.run_until_idle()
    # park a decoding sequence and bring it back: every rank exports and imports its own shard
    from saber_engine_b200.sched.mock import reference_generation
    pp = list(range(300, 340))
    psub = s.submit(EngineRequest(pp, SamplingParams(max_tokens=20)))
    for _ in range(4):
        s.step()
    key = s.park(psub.seq_id)
    other = s.submit(EngineRequest(list(range(50, 90)), SamplingParams(max_tokens=6)))    # the slot is used meanwhile
    s.run_until_idle()
    s.restore(key)
    s.run_until_idle()
    pt = []
    while True:
        ev = psub.events.get(timeout=10)
        pt += ev.new_token_ids
        if ev.finished:
            break
    park_ok = pt == reference_generation(pp, 20, 500)
    # an image of another process group is refused before any rank is asked to import it
    from saber_engine_b200.sched.park import ParkError
    try:
        lead.import_session(1, [1, 2], {"tp_park": {"id": 1, "epoch": lead.epoch + 1}}, b"")
        foreign = "imported"
    except ParkError:
        foreign = "refused"
    toks = []
    for sub in subs + [late]:
        t = []
        while True:
            ev = sub.events.get(timeout=10)
            t += ev.new_token_ids
            if ev.finished:
                break
        toks.append(t)
    lead.stop_followers()
    print(json.dumps({"rank": 0, "log": ex.launch_log, "tokens": toks, "cast": lead.calls_cast, "park_ok": park_ok,
                      "foreign": foreign, "hits": s.prefix.stats.hits, "state": sorted((k, v[1]) for k, v in ex._state.items())}))
else:
    n = follower_loop(ex, group)
    print(json.dumps({"rank": 1, "log": ex.launch_log, "served": n,
                      "state": sorted((k, v[1]) for k, v in ex._state.items())}))
dist.destroy_process_group()
'''


def test_follower_rank_runs_the_leaders_calls(tmp_path):
    import json
    import subprocess
    init = f"file://{tmp_path}/rdv"
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), INIT=init, PYTHONPATH=os.pathsep.join([os.getcwd()] + sys.path))
        procs.append(subprocess.Popen([sys.executable, "-c", _CHILD], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = []
    try:
        for p in procs:
            try:
                so, se = p.communicate(timeout=120)
            except subprocess.TimeoutExpired:
                p.kill()
                pytest.fail("rank process did not finish")
            assert p.returncode == 0, se[-2000:]
            outs.append(json.loads(so.strip().splitlines()[-1]))
    finally:
        for p in procs:               # no rank may outlive the test
            if p.poll() is None:
                p.kill()
    lead, fol = (outs[0], outs[1]) if outs[0]["rank"] == 0 else (outs[1], outs[0])
    assert lead["log"] == fol["log"] and len(lead["log"]) > 5          # the same launches, in the same order
    assert fol["served"] == lead["cast"] - 1                           # every call but the stop
    assert lead["state"] == fol["state"]                               # slots hold the same committed lengths
    assert lead["hits"] >= 1 and all(len(t) > 0 for t in lead["tokens"])
    assert lead["park_ok"] and lead["foreign"] == "refused"            # parked and restored on both ranks, same ids as unparked


_CHILD_SHM = r'''
import json, os, sys
from saber_engine_b200.parallel.control_frames import ShmChannel
from saber_engine_b200.parallel.tp_serve import TpLeaderExecutor, follower_loop
from saber_engine_b200.sched.mock import NullExecutor
from saber_engine_b200.sched.scheduler import Scheduler, SchedulerConfig
from saber_engine_b200.serve.engine_api import EngineRequest, SamplingParams

rank, line = int(os.environ["RANK"]), os.environ["LINE"]
ex = NullExecutor(seed=3, vocab=500, max_seqs=4)
if rank == 0:
    ch = ShmChannel(line, 3, 0, create=True)
    print("lines ready", flush=True)
    sys.stdin.readline()                       # the test starts the followers, then lets the leader go
    lead = TpLeaderExecutor(ex, None, channel=ch)
    s = Scheduler(lead, SchedulerConfig(max_seqs=4, max_ctx=8192, prefix_cache_min_tokens=32, prefix_cache_interval=64))
    shared = list(range(100, 260))
    subs = [s.submit(EngineRequest(shared + [7, 8, 9 + i], SamplingParams(max_tokens=12))) for i in range(3)]
    subs.append(s.submit(EngineRequest([j % 400 for j in range(3000)], SamplingParams(max_tokens=40))))   # multi-part frames, many pages
    s.run_until_idle()
    # a session parked and restored through the frames: its page list rides in one export / import frame
    ps = s.submit(EngineRequest(list(range(20, 420)), SamplingParams(max_tokens=400)))
    while not any(x.seq_id == ps.seq_id and not x.prefilling and x.output for x in s.running):
        s.step()                             # (the prompt is prefilled in pieces, one per prefix-cache cut point)
    key = s.park(ps.seq_id)
    s.run_until_idle()
    s.restore(key)
    s.run_until_idle()
    lead.stop_followers()
    print(json.dumps({"rank": 0, "log": ex.launch_log, "cast": lead.calls_cast, "bytes": lead.bytes_cast,
                      "state": sorted((k, v[1]) for k, v in ex._state.items())}))
    ch.close()
else:
    ch = ShmChannel(line, 3, rank, create=False)
    from saber_engine_b200.parallel.launcher import parent_alive
    n = follower_loop(ex, None, channel=ch, alive=parent_alive(os.getppid()))
    print(json.dumps({"rank": rank, "log": ex.launch_log, "served": n,
                      "state": sorted((k, v[1]) for k, v in ex._state.items())}))
    ch.close()
'''


def test_followers_run_the_leaders_calls_from_fixed_layout_frames_over_shared_memory(tmp_path):
    """Three processes, no process group at all: the control frames carry everything, block tables as
    deltas, a 3000-token prompt chunk in several parts."""
    import json
    import subprocess
    pytest.importorskip("saber_engine_b200.ops.native")
    from saber_engine_b200.ops import native
    if not native.available():
        pytest.skip("native library not built")
    line = f"/saber-test-{os.getpid()}"
    env = lambda r: dict(os.environ, RANK=str(r), LINE=line, PYTHONPATH=os.pathsep.join([os.getcwd()] + sys.path))
    lead = subprocess.Popen([sys.executable, "-c", _CHILD_SHM], env=env(0), stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                            stderr=subprocess.PIPE, text=True)
    assert "lines ready" in lead.stdout.readline()
    fols = [subprocess.Popen([sys.executable, "-c", _CHILD_SHM], env=env(r), stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
            for r in (1, 2)]
    lead.stdin.write("go\n")
    lead.stdin.flush()
    outs = []
    try:
        for p in [lead] + fols:
            try:
                so, se = p.communicate(timeout=120)
            except subprocess.TimeoutExpired:
                p.kill()
                pytest.fail("rank process did not finish")
            assert p.returncode == 0, se[-2000:]
            outs.append(json.loads(so.strip().splitlines()[-1]))
    finally:
        for p in [lead] + fols:       # a leader that failed leaves followers polling their lines: none may outlive the test
            if p.poll() is None:
                p.kill()
    l, f1, f2 = outs
    assert l["log"] == f1["log"] == f2["log"] and len(l["log"]) > 8
    assert f1["served"] == f2["served"] == l["cast"] - 1
    assert l["state"] == f1["state"] == f2["state"]
    # a decode step that crosses no page sends its record and tokens only: far below a pickled SeqRun with 190 blocks
    assert l["bytes"] / l["cast"] < 1500


def test_a_follower_that_dies_ends_in_the_fatal_law(tmp_path):
    """The self-launch's watcher: a child rank that exits while the engine is up sets the fatal (the
    reason names the rank and what it printed), an expected exit at shutdown does not; a follower
    whose parent is gone stops waiting on its line."""
    import subprocess
    from saber_engine_b200.parallel.launcher import launch_followers, parent_alive
    deaths = []
    import io
    tee = io.StringIO()
    code = "import sys, time, os\nr = os.environ['RANK']\nassert os.environ['WORLD_SIZE'] == '3' and os.environ['MASTER_ADDR'] == '127.0.0.1'\n" \
           "time.sleep(0.2 if r == '2' else 30)\nprint('saber: FATAL rank 2: device lost (injected on the host)', file=sys.stderr)\nsys.exit(86)\n"
    saved = {k: os.environ.get(k) for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT")}
    try:
        rs = launch_followers([sys.executable, "-c", code], 3, 29999, lambda r, why: deaths.append((r, why)), tee=tee)
        assert os.environ["RANK"] == "0" and os.environ["WORLD_SIZE"] == "3"
        for _ in range(200):
            if deaths:
                break
            import time
            time.sleep(0.02)
        assert deaths == [(2, "saber: FATAL rank 2: device lost (injected on the host)")]
        assert "device lost" in tee.getvalue()                      # the child's log is passed on, not swallowed
        rs.expect_exit()
        rs.procs[0].terminate()
        rs.wait(timeout=5)
        import time
        time.sleep(0.1)
        assert len(deaths) == 1                                        # rank 1's exit at shutdown is not a failure
    finally:
        for k, v in saved.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    assert parent_alive(os.getppid())() and not parent_alive(1 if os.getppid() != 1 else 2)()


def test_export_and_import_frames_carry_the_page_list():
    """Parking across ranks rides on two small-integer frames: slot, token count, park id and the session's pages."""
    from saber_engine_b200.parallel.control_frames import FrameDecoder, FrameEncoder
    enc, dec = FrameEncoder(), FrameDecoder()
    blocks = list(range(7, 7 + 700))                       # more than one 4 KiB part
    parts = enc.encode("export_session", 3, 11000, 42, *blocks)
    assert len(parts) == 2
    got = None
    for p in parts:
        got = dec.feed(p)
    assert got == ("export_session", (3, 11000, 42, *blocks))
    (part,) = enc.encode("import_session", 1, 42, *blocks[:5])
    assert dec.feed(part) == ("import_session", (1, 42, 7, 8, 9, 10, 11))
