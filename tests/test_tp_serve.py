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
    print(json.dumps({"rank": 0, "log": ex.launch_log, "tokens": toks, "cast": lead.calls_cast,
                      "hits": s.prefix.stats.hits, "state": sorted((k, v[1]) for k, v in ex._state.items())}))
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
    for p in procs:
        try:
            so, se = p.communicate(timeout=120)
        except subprocess.TimeoutExpired:
            p.kill()
            pytest.fail("rank process did not finish")
        assert p.returncode == 0, se[-2000:]
        outs.append(json.loads(so.strip().splitlines()[-1]))
    lead, fol = (outs[0], outs[1]) if outs[0]["rank"] == 0 else (outs[1], outs[0])
    assert lead["log"] == fol["log"] and len(lead["log"]) > 5          # the same launches, in the same order
    assert fol["served"] == lead["cast"] - 1                           # every call but the stop
    assert lead["state"] == fol["state"]                               # slots hold the same committed lengths
    assert lead["hits"] >= 1 and all(len(t) > 0 for t in lead["tokens"])
