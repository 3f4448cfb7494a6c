"""Warmup / stable / decay learning-rate schedule with the reference trainer's conventions.

Linear warm-up over ``warmup_steps`` (0-indexed, so step 0 already has a non-zero rate), an optional
stable phase, then linear / sqrt / cosine decay towards ``lr_min`` (a fraction of the peak); a virtual
extra step keeps the last rate above the floor.  ``lr_min_absolute`` is converted to that fraction and
``anneal_begin_step`` re-times the decay for a resumed run, as flame/train.py:413-452 does.
"""
from __future__ import annotations

import math
from dataclasses import dataclass


@dataclass
class LRSchedule:
    peak_lr: float
    training_steps: int
    warmup_steps: int = 200
    decay_ratio: float | None = None
    decay_type: str = "linear"
    lr_min: float = 0.0            # fraction of the peak

    def __post_init__(self):
        self.warmup_steps = min(int(self.warmup_steps), int(self.training_steps))
        if self.decay_ratio is not None:
            decay_steps = round(self.training_steps * self.decay_ratio)
            if self.warmup_steps + decay_steps > self.training_steps:
                decay_steps = self.training_steps - self.warmup_steps
        else:
            decay_steps = self.training_steps - self.warmup_steps
        self.decay_steps = max(0, decay_steps)
        self.stable_steps = self.training_steps - self.warmup_steps - self.decay_steps

    def factor(self, step: int) -> float:
        """Multiplier of the peak rate for 0-indexed optimizer step ``step``."""
        if step < self.warmup_steps:
            return float(step + 1) / float(self.warmup_steps + 1)
        warm_stable = self.warmup_steps + self.stable_steps
        if step < warm_stable:
            return 1.0
        progress = min(1.0, float(step + 1 - warm_stable) / float(self.decay_steps + 1))
        if self.decay_type == "linear":
            curr = 1.0 - progress
        elif self.decay_type == "sqrt":
            curr = 1.0 - math.sqrt(progress)
        elif self.decay_type == "cosine":
            curr = 0.5 * (1.0 + math.cos(math.pi * progress))
        else:
            raise ValueError(f"unknown decay_type {self.decay_type!r}")
        return self.lr_min + (1.0 - self.lr_min) * curr

    def lr(self, step: int) -> float:
        return self.peak_lr * self.factor(step)


def build_lr_schedule(job_config, logger=None) -> LRSchedule:
    """Apply the lr_min_absolute and anneal_begin_step rewrites, then build the schedule."""
    sched, opt, training = job_config.lr_scheduler, job_config.optimizer, job_config.training
    lr_min = sched.lr_min
    if sched.lr_min_absolute is not None:
        if opt.lr <= 0:
            raise ValueError("optimizer.lr must be > 0 when lr_min_absolute is given")
        lr_min = sched.lr_min_absolute / opt.lr
        if logger:
            logger.info(f"lr_min_absolute={sched.lr_min_absolute:g} -> lr_min ratio {lr_min:g}")
    steps, decay_ratio, warmup = training.steps, sched.decay_ratio, sched.warmup_steps
    if sched.anneal_begin_step is not None:
        begin = int(sched.anneal_begin_step)
        if not 0 <= begin < steps:
            raise ValueError("anneal_begin_step must lie inside the run")
        decay_ratio = (steps - begin) / steps
        warmup = min(warmup, begin)
        if logger:
            logger.info(f"anneal from step {begin}: decay_ratio {decay_ratio:.4f}")
    return LRSchedule(opt.lr, steps, warmup, decay_ratio, sched.decay_type, lr_min)
