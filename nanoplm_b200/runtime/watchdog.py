"""Host-side failure detection: per-rank heartbeat files and a watchdog.

The reference has no failure detection: a lost rank shows up as a collective that never returns
(src/nanoplm/pretraining/pure_pipeline.py has no timeout handling). Here every rank touches
`<run>/heartbeat/rank-<r>` from a background thread, recording the wall-clock time of the beat and of
the last optimizer step it completed; `find_stalled` names the ranks whose file is missing or old
(process gone) or whose step has not advanced for too long (process alive but stuck, e.g. inside a
collective a peer never joined: the beat thread keeps running then, so the file age alone says
nothing). `Watchdog` runs that check periodically on rank 0 and ends the process with a clear
message, so the launcher tears the job down and it can restart from the last complete checkpoint
instead of hanging. All of it is host code: nothing here touches the GPU.
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
        self._step = 0
        self._progress_time = time.time()

    @property
    def step(self) -> int:
        return self._step

    @step.setter
    def step(self, value: int) -> None:
        if value != self._step:
            self._step = value
            self._progress_time = time.time()

    def beat(self) -> None:
        self.path.parent.mkdir(parents=True, exist_ok=True)
        tmp = self.path.with_suffix(".tmp")
        tmp.write_text(f"{time.time()} {self._step} {os.getpid()} {self._progress_time}")
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
        try:
            self.beat()                 # the file ends with the last step this rank completed
        except OSError:
            pass


def read_heartbeat(path: Path) -> Optional[tuple[float, int, int, float]]:
    """(time of the beat, step, pid, time the step last advanced); None if unreadable."""
    try:
        parts = path.read_text().split()
        t, step, pid = float(parts[0]), int(parts[1]), int(parts[2])
        progress = float(parts[3]) if len(parts) > 3 else t
        return t, step, pid, progress
    except (OSError, ValueError, IndexError):
        return None


def find_stalled(directory: str | Path, world_size: int, max_age: float,
                 now: Optional[float] = None, max_step_age: Optional[float] = None) -> list[int]:
    """Ranks whose heartbeat file is missing or older than max_age seconds, or (with max_step_age)
    whose step counter has not advanced for more than max_step_age seconds."""
    now = time.time() if now is None else now
    stalled = []
    for r in range(world_size):
        hb = read_heartbeat(Path(directory) / f"rank-{r}")
        if hb is None or now - hb[0] > max_age:
            stalled.append(r)
        elif max_step_age is not None and now - hb[3] > max_step_age:
            stalled.append(r)
    return stalled


class Watchdog:
    """Periodic `find_stalled` on one rank. on_stall(ranks) defaults to ending the process with
    exit code 75 after logging, which makes torchrun stop the other ranks."""

    def __init__(self, directory: str | Path, world_size: int, max_age: float, max_step_age: Optional[float],
                 interval: float = 5.0, on_stall=None):
        self.directory, self.world_size = Path(directory), world_size
        self.max_age, self.max_step_age, self.interval = max_age, max_step_age, float(interval)
        self.on_stall = on_stall or self._abort
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.fired: Optional[list[int]] = None

    @staticmethod
    def _abort(ranks: list[int]) -> None:
        import sys
        sys.stderr.write(f"[watchdog] ranks without progress: {ranks}; ending the job\n")
        sys.stderr.flush()
        os._exit(75)

    def start(self) -> "Watchdog":
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            stalled = find_stalled(self.directory, self.world_size, self.max_age, max_step_age=self.max_step_age)
            if stalled:
                self.fired = stalled
                self.on_stall(stalled)
                return

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=self.interval + 1)


def check_or_raise(directory: str | Path, world_size: int, max_age: float) -> None:
    stalled = find_stalled(directory, world_size, max_age)
    if stalled:
        raise RankFailure(stalled)
