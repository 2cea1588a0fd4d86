"""Memory pressure valve: escalates demote -> park -> refuse as available host memory falls, with
hysteresis so that it does not flap around a threshold.

Parity: `crates/saber-mem/src/mem_valve.rs:1-25` (MemAvailable-driven escalation with hysteresis).
The reader is injectable; the default reads /proc/meminfo.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

LEVELS = ("ok", "demote", "park", "refuse")


def mem_available_bytes() -> int:
    with open("/proc/meminfo") as fh:
        for line in fh:
            if line.startswith("MemAvailable:"):
                return int(line.split()[1]) * 1024
    return 1 << 62


@dataclass
class MemValve:
    demote_below: int = 16 << 30
    park_below: int = 8 << 30
    refuse_below: int = 4 << 30
    hysteresis: float = 0.25              # a level is left only above threshold * (1 + hysteresis)
    reader: Callable[[], int] = mem_available_bytes
    level: str = "ok"

    def poll(self) -> str:
        avail = self.reader()
        thresholds = {"demote": self.demote_below, "park": self.park_below, "refuse": self.refuse_below}
        want = "ok"
        for name in ("demote", "park", "refuse"):
            if avail < thresholds[name]:
                want = name
        cur = LEVELS.index(self.level)
        if LEVELS.index(want) >= cur:
            self.level = want                       # escalation is immediate
        else:                                       # relaxation needs head-room above the level being left
            while cur > LEVELS.index(want) and avail >= thresholds[LEVELS[cur]] * (1 + self.hysteresis):
                cur -= 1
            self.level = LEVELS[cur]
        return self.level

    def admits(self) -> bool:
        return self.level != "refuse"
