"""Self-launch of the ranks of one node: the process the user started becomes rank 0 (it plans and
serves) and starts one child per further GPU.  Every child is watched (`serve.fatal.RankWatch`): a
child that exits while the engine is up, or that prints a FATAL line, sets the process-wide fatal
here, so queued and in-flight requests get 503 with the reason and the leader exits 86.  A follower
in turn watches its parent: when the leader is gone it leaves.

Parity: the reference's leader spawns its rank workers and a watcher ends the engine by the
teardown law when one of them dies (`crates/saber-serve/src/fatal.rs:1-30`, `README.md:602`).
"""
from __future__ import annotations

import os
import subprocess
import sys
from typing import Callable, Optional

from ..serve.fatal import RankWatch


class RankSet:
    def __init__(self):
        self.procs: list = []
        self.watches: list = []
        self.closing = False

    def expect_exit(self) -> None:
        """The leader is stopping its followers: their exits are not failures any more."""
        self.closing = True

    def wait(self, timeout: float = 10.0) -> None:
        for p in self.procs:
            try:
                p.wait(timeout=timeout)
            except subprocess.TimeoutExpired:
                p.terminate()


def rank_env(rank: int, world: int, port: int, base: Optional[dict] = None) -> dict:
    env = dict(os.environ if base is None else base)
    env.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), LOCAL_WORLD_SIZE=str(world),
               MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    return env


def launch_followers(argv: list, world: int, port: int, on_death: Callable[[int, str], None],
                     tee=sys.stderr) -> RankSet:
    """Start ranks 1 .. world-1 as children running `argv`; this process takes rank 0's environment.
    `on_death(rank, reason)` is called when a child ends before `expect_exit()`."""
    rs = RankSet()
    os.environ.update(rank_env(0, world, port, base={}))

    def died(rank: int, reason: str) -> None:
        if not rs.closing:
            on_death(rank, reason)
    for r in range(1, world):
        p = subprocess.Popen(argv, env=rank_env(r, world, port), stderr=subprocess.PIPE)
        rs.procs.append(p)
        rs.watches.append(RankWatch(p, r, died, tee=tee))
    return rs


def parent_alive(ppid: int) -> Callable[[], bool]:
    """For a follower: is the process that started it still there?"""
    return lambda: os.getppid() == ppid
