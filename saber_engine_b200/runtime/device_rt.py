"""Two pieces of the device runtime the step loop stands on: a BOUNDED host-side wait (a step that
never finishes ends in the teardown law instead of a blocked thread) and a background copy lane (a
side stream with pinned staging for the bulk copies that are not part of a step: session images,
prefix snapshots, prompt-store pages), ordered against the step stream by events only.

Parity: the reference's device runtime gives every host wait a deadline and moves bulk copies on a
lane of their own (`crates/saber-hip/src/stream.rs`, `copy_lane.rs`; survey of the L1 runtime).
"""
from __future__ import annotations

import time
from typing import Optional

import torch


class DeviceWaitTimeout(RuntimeError):
    pass


def bounded_wait(ev, timeout_s: float, what: str = "device work", spin_s: float = 0.05) -> float:
    """Wait until `ev` (a CUDA event or stream: anything with query()) has completed, at most
    `timeout_s`.  Polls without sleeping for the first `spin_s` (steps take milliseconds), then with
    50 us naps.  Returns the seconds waited; raises DeviceWaitTimeout past the deadline (the work is
    still in flight: the caller ends the engine, it does not retry)."""
    t0 = time.perf_counter()
    while not ev.query():
        dt = time.perf_counter() - t0
        if dt > timeout_s:
            raise DeviceWaitTimeout(f"{what} did not complete within {timeout_s:g} s")
        if dt > spin_s:
            time.sleep(50e-6)
    return time.perf_counter() - t0


class CopyLane:
    """A side stream for bulk copies.  `after(stream)` makes the lane wait for what `stream` has
    queued so far (the data being copied out was produced there); `d2h` / `h2d` queue one copy through
    pinned memory and return an event; `before(stream)` makes `stream` wait for the lane (data copied
    in is about to be used there).  The step stream itself never blocks the host for these copies."""

    def __init__(self, device, staging_bytes: int = 64 << 20):
        self.device = torch.device(device)
        self.stream = torch.cuda.Stream(device=self.device)
        self.staging_bytes = staging_bytes
        self._pinned: dict = {}
        self.bytes_d2h = self.bytes_h2d = 0

    def pinned(self, nbytes: int, tag: str = "") -> torch.Tensor:
        """A pinned byte buffer of at least `nbytes` (kept and reused per tag)."""
        buf = self._pinned.get(tag)
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(max(nbytes, 1), dtype=torch.uint8).pin_memory()
            self._pinned[tag] = buf
        return buf[:nbytes]

    def after(self, stream) -> None:
        ev = torch.cuda.Event()
        ev.record(stream)
        self.stream.wait_event(ev)

    def before(self, stream) -> None:
        ev = torch.cuda.Event()
        ev.record(self.stream)
        stream.wait_event(ev)

    def d2h(self, dst_host: torch.Tensor, src_dev: torch.Tensor) -> "torch.cuda.Event":
        with torch.cuda.stream(self.stream):
            dst_host.copy_(src_dev, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        src_dev.record_stream(self.stream)
        self.bytes_d2h += src_dev.numel() * src_dev.element_size()
        return ev

    def h2d(self, dst_dev: torch.Tensor, src_host: torch.Tensor) -> "torch.cuda.Event":
        with torch.cuda.stream(self.stream):
            dst_dev.copy_(src_host, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        self.bytes_h2d += dst_dev.numel() * dst_dev.element_size()
        return ev

    def wait(self, timeout_s: float = 60.0) -> None:
        bounded_wait(self.stream, timeout_s, "the copy lane")
