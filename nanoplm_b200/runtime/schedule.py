"""Learning-rate schedules.

`WarmupLinearSchedule` is the reference pretraining schedule (pure_pipeline.py:150-172): linear
warm-up over `warmup_steps`, then linear decay to zero at `total_steps`; a warm-up value >= 1 is an
absolute step count, a value < 1 a ratio (rounded up). `make_distill_schedule` covers the four
schedules of the distillation pipeline (distillation/pipeline.py:396-446). State dicts carry
`last_epoch` / `base_lrs` like torch's LambdaLR, so `scheduler.pt` files are interchangeable.
"""
from __future__ import annotations

import math
from typing import Callable, Optional, Sequence


def get_warmup_steps(total_steps: int, warmup_value: float) -> int:
    if warmup_value >= 1:
        return int(warmup_value)
    return math.ceil(total_steps * warmup_value)


def num_update_steps_per_epoch(loader_len: int, grad_accum: int) -> int:
    if loader_len <= 0:
        return 1
    return max(1, math.ceil(loader_len / max(1, grad_accum)))


class LambdaSchedule:
    """A learning-rate multiplier over optimizer steps with the state-dict layout of torch's LambdaLR.

    `group_lrs` lists the base rate of every parameter group of the optimizer whose `optimizer.pt`
    is written next to this schedule (decay / no-decay for AdamW, Muon / AdamW for Muon), because
    torch's scheduler refuses a state whose lists are shorter than its optimizer's groups;
    `primary` is the group whose rate `get_lr()` returns."""

    def __init__(self, base_lr: float, fn: Callable[[int], float], group_lrs: Optional[Sequence[float]] = None,
                 primary: int = 0):
        self.base_lrs = [float(x) for x in group_lrs] if group_lrs else [float(base_lr), float(base_lr)]
        self.primary = primary if 0 <= primary < len(self.base_lrs) else 0
        self.base_lrs[self.primary] = float(base_lr)
        self.fn = fn
        self.last_epoch = 0

    def get_lr(self) -> float:
        return self.base_lrs[self.primary] * self.fn(self.last_epoch)

    def get_last_lr(self) -> list[float]:
        m = self.fn(self.last_epoch)
        return [b * m for b in self.base_lrs]

    def step(self) -> None:
        self.last_epoch += 1

    def state_dict(self) -> dict:
        return {"base_lrs": list(self.base_lrs), "last_epoch": self.last_epoch,
                "_step_count": self.last_epoch + 1, "_is_initial": False, "_get_lr_called_within_step": False,
                "_last_lr": self.get_last_lr(), "lr_lambdas": [None] * len(self.base_lrs)}

    def load_state_dict(self, sd: dict) -> None:
        self.last_epoch = int(sd.get("last_epoch", 0))
        saved = [float(x) for x in (sd.get("base_lrs") or [])]
        if len(saved) == len(self.base_lrs):
            self.base_lrs = saved
        elif saved:                                 # a file with another number of groups: one rate for all
            self.base_lrs = [saved[0]] * len(self.base_lrs)


class WarmupLinearSchedule(LambdaSchedule):
    def __init__(self, base_lr: float, warmup_steps: int, total_steps: int,
                 group_lrs: Optional[Sequence[float]] = None, primary: int = 0):
        def fn(step: int) -> float:
            if step < warmup_steps:
                return step / max(1, warmup_steps)
            return max(0.0, (total_steps - step) / max(1, total_steps - warmup_steps))
        super().__init__(base_lr, fn, group_lrs, primary)
        self.warmup_steps, self.total_steps = warmup_steps, total_steps


def make_distill_schedule(name: str, base_lr: float, warmup_steps: int, total_steps: int,
                          **kwargs) -> LambdaSchedule:
    name = name.lower()
    # an explicit warm-up length among the scheduler arguments wins (reference:
    # distillation/pipeline.py:415-419)
    warmup_steps = int(kwargs.get("num_warmup_steps", warmup_steps))

    def warm(step: int):
        return step / max(1, warmup_steps) if step < warmup_steps else None

    if name == "cosine":
        cycles = float(kwargs.get("num_cycles", 0.5))

        def fn(step):
            w = warm(step)
            if w is not None:
                return w
            prog = (step - warmup_steps) / max(1, total_steps - warmup_steps)
            return max(0.0, 0.5 * (1.0 + math.cos(math.pi * cycles * 2.0 * prog)))
    elif name == "linear":
        def fn(step):
            w = warm(step)
            if w is not None:
                return w
            return max(0.0, (total_steps - step) / max(1, total_steps - warmup_steps))
    elif name == "polynomial":
        power = float(kwargs.get("power", 1.0))
        lr_end = float(kwargs.get("lr_end", 1e-7))

        def fn(step):
            w = warm(step)
            if w is not None:
                return w
            if step > total_steps:
                return lr_end / base_lr
            rem = 1 - (step - warmup_steps) / max(1, total_steps - warmup_steps)
            return ((base_lr - lr_end) * rem ** power + lr_end) / base_lr
    elif name == "constant":
        def fn(step):
            w = warm(step)
            return 1.0 if w is None else w
    else:
        raise ValueError(f"Unknown lr_scheduler: {name}. Supported: cosine, linear, polynomial, constant")
    # the distillation optimizer has one parameter group (reference: distillation/pipeline.py:669)
    return LambdaSchedule(base_lr, fn, group_lrs=[base_lr])
