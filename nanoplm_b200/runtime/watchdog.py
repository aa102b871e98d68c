"""Host-side failure detection: per-rank heartbeat files and a watchdog.

The reference has no failure detection: a lost rank shows up as a collective that never returns
(src/nanoplm/pretraining/pure_pipeline.py has no timeout handling). Here every rank touches
`<run>/heartbeat/rank-<r>` from a background thread; `find_stalled` (used by the launcher and by
rank 0 before a collective-heavy phase) names the ranks whose heartbeat is older than the limit so
the job can be torn down and restarted from the last complete checkpoint instead of hanging.
All of it is host code: nothing here touches the GPU.
"""
from __future__ import annotations

import os
import threading
import time
from pathlib import Path
from typing import Optional


class RankFailure(RuntimeError):
    def __init__(self, ranks: list[int]):
        super().__init__(f"ranks without a recent heartbeat: {ranks}")
        self.ranks = ranks


class Heartbeat:
    def __init__(self, directory: str | Path, rank: int, interval: float = 5.0):
        self.path = Path(directory) / f"rank-{rank}"
        self.interval = float(interval)
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.step = 0

    def beat(self) -> None:
        self.path.parent.mkdir(parents=True, exist_ok=True)
        tmp = self.path.with_suffix(".tmp")
        tmp.write_text(f"{time.time()} {self.step} {os.getpid()}")
        os.replace(tmp, self.path)

    def start(self) -> "Heartbeat":
        self.beat()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            try:
                self.beat()
            except OSError:
                pass

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=self.interval + 1)


def read_heartbeat(path: Path) -> Optional[tuple[float, int, int]]:
    try:
        t, step, pid = path.read_text().split()
        return float(t), int(step), int(pid)
    except (OSError, ValueError):
        return None


def find_stalled(directory: str | Path, world_size: int, max_age: float,
                 now: Optional[float] = None) -> list[int]:
    """Ranks whose heartbeat file is missing or older than max_age seconds."""
    now = time.time() if now is None else now
    stalled = []
    for r in range(world_size):
        hb = read_heartbeat(Path(directory) / f"rank-{r}")
        if hb is None or now - hb[0] > max_age:
            stalled.append(r)
    return stalled


def check_or_raise(directory: str | Path, world_size: int, max_age: float) -> None:
    stalled = find_stalled(directory, world_size, max_age)
    if stalled:
        raise RankFailure(stalled)
