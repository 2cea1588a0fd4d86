"""Serving on several GPUs: rank 0 runs the scheduler and the HTTP plane, the other ranks follow.

Every rank owns a shard of the model and runs the SAME step programs; the fused collectives inside
the kernels keep the GPUs in step.  What the follower ranks lack is the scheduler's decisions, so
rank 0 wraps its executor in `TpLeaderExecutor`: every executor call (prefill, decode, slot reset,
state snapshot / restore) is first broadcast -- name and arguments, over a host-side (gloo) process
group -- and then run locally; `follower_loop` on the other ranks receives the calls and runs them on
its own executor, discarding the results (token picks are merged across ranks on the device and
equal everywhere).

    # one process per GPU, e.g. under torchrun
    group = init_control_group()                      # gloo, beside the NCCL group used for bootstrap
    if rank == 0:  scheduler = Scheduler(TpLeaderExecutor(executor, group), ...)
    else:          follower_loop(executor, group)

Parity: the reference's rank workers (`crates/saber-exec/src/peer.rs:140` `RankPeer::agree`, the
2-rank command line of `crates/saber-engine/src/device.rs`): one planning rank, lock-step followers.
"""
from __future__ import annotations

import itertools
from typing import Optional

FORWARDED = ("prefill", "decode", "reset_slot")
FOLLOWER_PARKS = 64          # parked images a follower keeps (host memory, newest first out last)


def init_control_group(timeout_s: float = 1800.0):
    """A gloo group over all ranks for the host-side command broadcast (the default group may be NCCL)."""
    import datetime

    import torch.distributed as dist
    return dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))


class TpLeaderExecutor:
    """Rank 0's executor: broadcasts each call to the followers, then runs it on the local shard."""

    def __init__(self, inner, group, src: int = 0, channel=None):
        """channel: a `control_frames.ShmChannel` (fixed-layout frames over shared memory, block tables
        as deltas); without one every call is pickled through the gloo group."""
        self.inner, self.group, self.src, self.channel = inner, group, src, channel
        self._snap_ids = itertools.count(1)
        import collections
        import os
        self.epoch = int.from_bytes(os.urandom(6), "little")
        self.world = int(getattr(getattr(inner, "model", None), "tp", 0)) or 0
        self._parks_made = collections.deque(maxlen=FOLLOWER_PARKS)
        self.calls_cast = 0
        self.bytes_cast = 0
        if channel is not None:
            from .control_frames import FrameEncoder
            self._enc = FrameEncoder()

    def __getattr__(self, name):                     # geometry, census, model, ...: the local executor's
        return getattr(self.inner, name)

    def _cast(self, name: str, *args) -> None:
        if self.channel is not None:
            parts = self._enc.encode(name, *args)
            self.channel.send(parts)
            self.bytes_cast += sum(len(p) for p in parts)
        else:
            import torch.distributed as dist
            dist.broadcast_object_list([(name, args)], src=self.src, group=self.group)
        self.calls_cast += 1

    def prefill(self, runs: list) -> list:
        self._cast("prefill", runs)
        return self.inner.prefill(runs)

    def decode(self, runs: list, width: int) -> list:
        self._cast("decode", runs, width)
        return self.inner.decode(runs, width)

    def reset_slot(self, slot: int) -> None:
        self._cast("reset_slot", slot)
        self.inner.reset_slot(slot)

    # prefix-cache snapshots: every rank keeps its own shard of a snapshot under the leader's id
    def snapshot_state(self, slot: int):
        sid = next(self._snap_ids)
        self._cast("snapshot_state", slot, sid)
        return {"id": sid, "local": self.inner.snapshot_state(slot)}

    def restore_state(self, slot: int, snap) -> None:
        self._cast("restore_state", slot, snap["id"])
        self.inner.restore_state(slot, snap["local"])

    def free_snapshot(self, snap) -> None:
        if isinstance(snap, dict) and "id" in snap:
            self._cast("free_snapshot", snap["id"])
            self.inner.free_snapshot(snap["local"])

    def snapshot_bytes(self) -> int:
        return self.inner.snapshot_bytes()

    # session parking: every rank exports its own shard (its KV heads, its DeltaNet heads) under the leader's
    # park id.  The leader's image travels through the park tiers as on one GPU; a follower keeps its shard
    # in host memory (the newest `FOLLOWER_PARKS` images), so an image can only come back into the process
    # group that made it: the header carries the group's epoch and an image of another epoch is refused
    # before any rank is asked to import.
    supports_parking = True

    def export_session(self, slot: int, blocks: list, n_tokens: int):
        pid = next(self._snap_ids)
        self._parks_made.append(pid)
        self._cast("export_session", slot, n_tokens, pid, *blocks)
        header, payload = self.inner.export_session(slot, blocks, n_tokens)
        header["tp_park"] = {"id": pid, "epoch": self.epoch, "ranks": self.world}
        return header, payload

    def import_session(self, slot: int, blocks: list, header: dict, payload: bytes) -> None:
        from ..sched.park import ParkError
        tag = header.get("tp_park")
        if not tag or tag.get("epoch") != self.epoch:
            raise ParkError("this image was parked by another process group: the follower ranks do not hold their shards of it")
        if tag["id"] < self._park_floor():
            raise ParkError("the follower ranks have dropped their shards of this image")
        self._cast("import_session", slot, tag["id"], *blocks)
        self.inner.import_session(slot, blocks, header, payload)

    def _park_floor(self) -> int:
        """Oldest park id the followers still hold (they keep the newest FOLLOWER_PARKS images; ids are shared
        with the snapshot counter, so this bound is conservative)."""
        return self._parks_made[0] if len(self._parks_made) == FOLLOWER_PARKS else 0

    def stop_followers(self) -> None:
        self._cast("stop")


def follower_loop(executor, group, src: int = 0, on_call=None, channel=None, alive=None) -> int:
    """Runs the leader's calls on this rank's executor until the leader says stop.  Returns the number
    of calls served.  With a channel the calls arrive as fixed-layout frames; `alive()` is asked while
    the line is idle, and a follower whose leader is gone leaves with ConnectionError."""
    snaps: dict = {}
    parks: dict = {}
    served = 0
    dec = None
    if channel is not None:
        from .control_frames import FrameDecoder
        dec = FrameDecoder()
    while True:
        if dec is not None:
            call = None
            while call is None:
                call = dec.feed(channel.recv(alive=alive))
            name, args = call
        else:
            import torch.distributed as dist
            box = [None]
            dist.broadcast_object_list(box, src=src, group=group)
            name, args = box[0]
        if name == "stop":
            return served
        if name == "prefill":
            executor.prefill(args[0])
        elif name == "decode":
            executor.decode(args[0], args[1])
        elif name == "reset_slot":
            executor.reset_slot(args[0])
        elif name == "snapshot_state":
            snaps[args[1]] = executor.snapshot_state(args[0])
        elif name == "restore_state":
            executor.restore_state(args[0], snaps[args[1]])
        elif name == "free_snapshot":
            s = snaps.pop(args[0], None)
            if s is not None:
                executor.free_snapshot(s)
        elif name == "export_session":
            slot, n_tokens, pid = int(args[0]), int(args[1]), int(args[2])
            parks[pid] = executor.export_session(slot, [int(b) for b in args[3:]], n_tokens)
            while len(parks) > FOLLOWER_PARKS:
                parks.pop(next(iter(parks)))
        elif name == "import_session":
            slot, pid = int(args[0]), int(args[1])
            header, payload = parks[pid]
            executor.import_session(slot, [int(b) for b in args[2:]], header, payload)
        else:
            raise RuntimeError(f"unknown call from the leader: {name!r}")
        served += 1
        if on_call is not None:
            on_call(name, args)
