"""Job supervisor: launches the ranks of a pretraining job, ends all of them when one fails or
stalls, and starts the job again from the latest complete checkpoint.

The reference leaves recovery to the user: a lost rank is a collective that never returns, and the
run is continued by hand with `resume.is_resume: true` (src/nanoplm/cli/pretrain.py:885-924). Here
`nanoplm pretrain supervise pretrain.yaml --nproc N` (and `nanoplm distill supervise distill.yaml`)
does that loop:

  1. start N rank processes of `nanoplm pretrain from-yaml` (one per GPU, or CPU ranks over gloo), each
     in a process group of its own, with RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR=127.0.0.1 and a
     fresh MASTER_PORT per attempt;
  2. watch them: all exit 0 -> done. A rank that exits non-zero (an exception, a kill, the in-process
     watchdog's exit code 75), or whose heartbeat step stops advancing for `stall_seconds` when
     heartbeats are on, ends the attempt: the remaining ranks get SIGTERM, then SIGKILL after a grace
     period, by the exact process groups that were started;
  3. look for the newest `checkpoint-N` with a complete state file in the run directory the attempt
     created (checkpoints are written under a temporary name and renamed, so a directory that exists
     is complete), write the attempt's YAML with `resume: {is_resume: true, checkpoint_dir: ...}`
     and go to 1, at most `max_restarts` times. Without a checkpoint the job starts over.

Ranks leave only between steps or die on the host; the survivors are ended by signal while they wait
in a collective. Nothing here touches a GPU.
"""
from __future__ import annotations

import os
import signal
import socket
import subprocess
import sys
import tempfile
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional, Sequence

import yaml

from nanoplm_b200.runtime.checkpoint import latest_checkpoint
from nanoplm_b200.runtime.watchdog import find_stalled
from nanoplm_b200.utils.logging import logger


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return int(s.getsockname()[1])


@dataclass
class Attempt:
    index: int
    exit_codes: list = field(default_factory=list)
    reason: str = ""
    resumed_from: Optional[str] = None
    run_dir: Optional[str] = None


class Supervisor:
    def __init__(self, config: str | Path, nproc: int = 1, max_restarts: int = 3, stall_seconds: float = 0.0,
                 grace_seconds: float = 10.0, poll_seconds: float = 0.5, extra_env: Optional[dict] = None,
                 command: Optional[Sequence[str]] = None, log_dir: Optional[str | Path] = None,
                 section: str = "pretraining"):
        self.config = Path(config).resolve()
        if not self.config.exists():
            raise FileNotFoundError(f"Config file not found: {self.config}")
        self.nproc, self.max_restarts = int(nproc), int(max_restarts)
        if self.nproc < 1:
            raise ValueError("nproc must be at least 1")
        self.stall_seconds, self.grace, self.poll = float(stall_seconds), float(grace_seconds), float(poll_seconds)
        self.extra_env = dict(extra_env or {})
        # the rank command; the attempt's YAML path is appended
        if section not in ("pretraining", "distillation"):
            raise ValueError("section must be 'pretraining' or 'distillation'")
        self.section = section
        group = "pretrain" if section == "pretraining" else "distill"
        self.command = list(command) if command else [sys.executable, "-m", "nanoplm_b200", group, "from-yaml"]
        self.raw = yaml.safe_load(self.config.read_text(encoding="utf-8")) or {}
        pre = self.raw.get(section) or {}
        self.ckp_dir = Path(pre.get("ckp_dir", "output/" + section))
        if not self.ckp_dir.is_absolute():
            self.ckp_dir = Path.cwd() / self.ckp_dir
        self.log_dir = Path(log_dir) if log_dir else None
        self.attempts: list[Attempt] = []
        self.run_dir: Optional[Path] = None
        self._work = Path(tempfile.mkdtemp(prefix="nplm-supervise-"))

    # ---- one attempt -------------------------------------------------------------------------
    def _attempt_config(self, k: int, resume_from: Optional[Path]) -> Path:
        raw = {key: (dict(v) if isinstance(v, dict) else v) for key, v in self.raw.items()}
        pre = raw.setdefault(self.section, {})
        if self.nproc > 1:
            pre["multi_gpu"] = True
            pre["world_size"] = self.nproc
        if resume_from is not None:
            raw["resume"] = {"is_resume": True, "checkpoint_dir": str(resume_from),
                             "extra_epochs": (self.raw.get("resume") or {}).get("extra_epochs")
                             if (self.raw.get("resume") or {}).get("is_resume") else None}
        self._work.mkdir(parents=True, exist_ok=True)
        path = self._work / f"attempt-{k}.yaml"
        path.write_text(yaml.safe_dump(raw), encoding="utf-8")
        return path

    def _run_dirs(self) -> set:
        return {p for p in self.ckp_dir.glob("run-*") if p.is_dir()} if self.ckp_dir.exists() else set()

    def _launch(self, k: int, cfg_path: Path) -> list[subprocess.Popen]:
        port = _free_port()
        procs = []
        for r in range(self.nproc):
            env = dict(os.environ)
            env.update(RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(self.nproc), MASTER_ADDR="127.0.0.1",
                       MASTER_PORT=str(port), NPLM_ATTEMPT=str(k))
            env.update({key: str(v) for key, v in self.extra_env.items()})
            out = None
            if self.log_dir is not None:
                self.log_dir.mkdir(parents=True, exist_ok=True)
                out = open(self.log_dir / f"attempt-{k}-rank-{r}.log", "wb")
            procs.append(subprocess.Popen(self.command + [str(cfg_path)], env=env, stdout=out,
                                          stderr=subprocess.STDOUT if out else None, start_new_session=True))
            if out is not None:
                out.close()
        return procs

    def _end(self, procs: list[subprocess.Popen]) -> None:
        """SIGTERM to the process group of every rank that is still running, SIGKILL after the
        grace period. Only the groups started by `_launch` are signalled."""
        for sig, wait in ((signal.SIGTERM, self.grace), (signal.SIGKILL, 5.0)):
            alive = [p for p in procs if p.poll() is None]
            if not alive:
                return
            for p in alive:
                try:
                    os.killpg(p.pid, sig)          # start_new_session: the group id is the child's pid
                except ProcessLookupError:
                    pass
            deadline = time.time() + wait
            while time.time() < deadline and any(p.poll() is None for p in alive):
                time.sleep(0.05)

    def _watch(self, procs: list[subprocess.Popen], before: set) -> str:
        """Returns "" when every rank exited 0, else the reason the attempt ended."""
        started = time.time()
        while True:
            codes = [p.poll() for p in procs]
            bad = [(r, c) for r, c in enumerate(codes) if c not in (None, 0)]
            if bad:
                return "rank " + ", ".join(f"{r} exited with code {c}" for r, c in bad)
            if all(c == 0 for c in codes):
                return ""
            if self.run_dir is None:
                new = self._run_dirs() - before
                if new:
                    self.run_dir = max(new, key=lambda p: p.stat().st_mtime)
            if self.stall_seconds > 0 and self.run_dir is not None and (self.run_dir / "heartbeat").exists() \
                    and time.time() - started > self.stall_seconds:
                hb = self.run_dir / "heartbeat"
                stalled = find_stalled(hb, self.nproc, max_age=self.stall_seconds, max_step_age=self.stall_seconds)
                # a rank that already left with code 0 no longer beats: not a stall. Neither is a file
                # left by an earlier attempt in the same run directory while this attempt is still
                # starting up (imports, dataset set-up), within a generous allowance
                starting = time.time() - started < max(120.0, 5 * self.stall_seconds)

                def stale(r: int) -> bool:
                    f = hb / f"rank-{r}"
                    return (not f.exists()) or f.stat().st_mtime < started
                stalled = [r for r in stalled if codes[r] is None and not (starting and stale(r))]
                if stalled:
                    return f"no progress on ranks {stalled} for {self.stall_seconds:.0f} s"
            time.sleep(self.poll)

    # ---- the loop ----------------------------------------------------------------------------
    def run(self) -> int:
        # the ranks live in sessions of their own, so a SIGTERM to the supervisor would orphan them:
        # turn it into an exit that runs the `finally` blocks (which end the ranks)
        import threading
        previous = None
        if threading.current_thread() is threading.main_thread():
            def _terminate(signum, frame):
                raise SystemExit(128 + signum)
            previous = signal.signal(signal.SIGTERM, _terminate)
        try:
            return self._run()
        finally:
            import shutil
            shutil.rmtree(self._work, ignore_errors=True)      # the per-attempt YAML files
            if previous is not None:
                signal.signal(signal.SIGTERM, previous)

    def _run(self) -> int:
        resume_from: Optional[Path] = None
        user_resume = self.raw.get("resume") or {}
        if user_resume.get("is_resume") and user_resume.get("checkpoint_dir"):
            resume_from = Path(user_resume["checkpoint_dir"])
            self.run_dir = resume_from.parent
        for k in range(self.max_restarts + 1):
            before = self._run_dirs()
            cfg_path = self._attempt_config(k, resume_from)
            att = Attempt(k, resumed_from=str(resume_from) if resume_from else None)
            self.attempts.append(att)
            logger.info(f"[supervisor] attempt {k}: {self.nproc} rank(s)"
                        + (f", resuming from {resume_from}" if resume_from else ""))
            procs = self._launch(k, cfg_path)
            try:
                att.reason = self._watch(procs, before)
            finally:
                self._end(procs)
            att.exit_codes = [p.returncode for p in procs]
            if self.run_dir is None:
                new = self._run_dirs() - before
                if new:
                    self.run_dir = max(new, key=lambda p: p.stat().st_mtime)
            att.run_dir = str(self.run_dir) if self.run_dir else None
            if not att.reason:
                logger.info(f"[supervisor] job finished after {k} restart(s)")
                return 0
            logger.info(f"[supervisor] attempt {k} ended: {att.reason}")
            ck = latest_checkpoint(self.run_dir) if self.run_dir is not None else None
            if ck is not None:
                resume_from = ck
            elif resume_from is None:
                self.run_dir = None                 # nothing saved yet: the next attempt starts a new run
        logger.info(f"[supervisor] giving up after {self.max_restarts} restart(s)")
        return 1

    @property
    def restarts(self) -> int:
        return max(0, len(self.attempts) - 1)
