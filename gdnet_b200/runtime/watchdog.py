"""Host-side failure detection: per-rank step heartbeats and a monitor that names stragglers.

The reference has none (its only protection is the 30-minute NCCL timeout,
gdnet/utils/distributed.py:59,90). Here every rank writes ``{rank, step, time}`` to a small file (or a
``torch.distributed`` store) after each step; a monitor thread on rank 0 compares them and reports
ranks that have not advanced within ``stall_s``. Device-side waits are bounded separately (every
kernel wait has a time budget and reports through the status word), so a lost peer surfaces as a
``KernelTimeout`` on its neighbours rather than a hang. Recovery is restart from the last
checkpoint, on any world size (sharded checkpoints re-slice on load).
"""

from __future__ import annotations

import json
import os
import threading
import time
from pathlib import Path


class Heartbeat:
    """Writes this rank's progress; cheap enough to call every step."""

    def __init__(self, directory: str, rank: int):
        self.path = Path(directory) / f"rank_{rank:05d}.json"
        self.path.parent.mkdir(parents=True, exist_ok=True)
        self.rank = rank

    def beat(self, step: int, **extra) -> None:
        tmp = self.path.with_suffix(".tmp")
        tmp.write_text(json.dumps({"rank": self.rank, "step": int(step), "time": time.time(), **extra}))
        os.replace(tmp, self.path)


def read_heartbeats(directory: str) -> dict[int, dict]:
    out = {}
    for f in sorted(Path(directory).glob("rank_*.json")):
        try:
            rec = json.loads(f.read_text())
            out[int(rec["rank"])] = rec
        except (ValueError, KeyError, OSError):
            continue  # a file being replaced right now
    return out


def find_stalled(beats: dict[int, dict], world: int, stall_s: float, now: float | None = None) -> list[int]:
    """Ranks that are missing or whose last beat is older than ``stall_s`` seconds."""
    now = time.time() if now is None else now
    return [r for r in range(world) if r not in beats or now - beats[r]["time"] > stall_s]


def find_stragglers(beats: dict[int, dict], max_lag: int = 2) -> list[int]:
    """Ranks more than ``max_lag`` steps behind the fastest rank."""
    if not beats:
        return []
    top = max(b["step"] for b in beats.values())
    return [r for r, b in beats.items() if top - b["step"] > max_lag]


class Watchdog(threading.Thread):
    """Rank-0 monitor. Calls ``on_failure(stalled_ranks)`` once when ranks stall; never kills anything."""

    def __init__(self, directory: str, world: int, stall_s: float = 120.0, period_s: float = 5.0, on_failure=None):
        super().__init__(daemon=True)
        self.directory, self.world, self.stall_s, self.period_s = directory, world, stall_s, period_s
        self.on_failure = on_failure
        self.failed: list[int] = []
        self._halt = threading.Event()

    def run(self) -> None:
        while not self._halt.wait(self.period_s):
            stalled = find_stalled(read_heartbeats(self.directory), self.world, self.stall_s)
            if stalled and not self.failed:
                self.failed = stalled
                if self.on_failure is not None:
                    self.on_failure(stalled)

    def stop(self) -> None:
        self._halt.set()
