"""Host-side fault injection for recovery tests.

`NPLM_INJECT_FAULT="rank:step:mode[:attempt]"` makes rank `rank` fail right after optimizer step
`step`, between steps, with none of its kernels or collectives in flight:

  * `raise`  raises `InjectedFault` (the rank leaves through the normal exception path),
  * `exit`   ends the process at once with exit code 17 (a killed process),
  * `stall`  stops making progress but stays alive (a rank stuck on the host; the heartbeat's step
             stops advancing), until the supervisor or the watchdog ends it.

`attempt` (default 0) is compared with `NPLM_ATTEMPT`, which the supervisor sets for every launch, so
that a restarted job does not fail again at the same step. Everything happens on the host: no GPU is
faulted, trapped or hung by this module, and nothing is injected unless the variable is set.
"""
from __future__ import annotations

import os
import time


class InjectedFault(RuntimeError):
    pass


def maybe_inject(rank: int, step: int) -> None:
    spec = os.environ.get("NPLM_INJECT_FAULT")
    if not spec:
        return
    parts = spec.split(":")
    if len(parts) < 3:
        raise ValueError(f"NPLM_INJECT_FAULT must be rank:step:mode[:attempt], got {spec!r}")
    want_rank, want_step, mode = int(parts[0]), int(parts[1]), parts[2]
    attempt = int(parts[3]) if len(parts) > 3 else 0
    if rank != want_rank or step != want_step or int(os.environ.get("NPLM_ATTEMPT", "0")) != attempt:
        return
    if mode == "raise":
        raise InjectedFault(f"injected failure on rank {rank} after step {step}")
    if mode == "exit":
        os._exit(17)
    if mode == "stall":
        while True:
            time.sleep(0.5)
    raise ValueError(f"unknown fault mode {mode!r} (raise, exit, stall)")
