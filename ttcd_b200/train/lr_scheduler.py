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
    """Apply the lr_min_absolute and anneal_begin_step rewrites, then build the schedule.

    Both rewrites change ``job_config`` in place, as flame/train.py:413-452 does, so that the train loop and the
    metrics read the rewritten ``training.steps``: with ``anneal_begin_step = B`` and ``decay_ratio = r`` the run
    ends after ``B + round(B r)`` steps and decays over exactly those last ``round(B r)`` steps.
    """
    sched, opt, training = job_config.lr_scheduler, job_config.optimizer, job_config.training
    if sched.lr_min_absolute is not None:
        if sched.lr_min_absolute >= opt.lr:
            if logger:
                logger.warning(f"lr_min_absolute ({sched.lr_min_absolute:g}) >= optimizer.lr ({opt.lr:g}): "
                               "lr_min set to 1.0 (no decay)")
            sched.lr_min = 1.0
        else:
            sched.lr_min = sched.lr_min_absolute / opt.lr
            if logger:
                logger.info(f"lr_min_absolute={sched.lr_min_absolute:g} -> lr_min ratio {sched.lr_min:g}")
    if sched.anneal_begin_step is not None:
        begin, ratio = int(sched.anneal_begin_step), sched.decay_ratio
        if ratio is None or ratio <= 0:
            raise ValueError(f"anneal_begin_step={begin} requires a positive decay_ratio, got {ratio}")
        anneal_steps = round(begin * ratio)
        new_total = begin + anneal_steps
        if new_total <= 0:
            raise ValueError("anneal_begin_step must be positive")
        if logger:
            logger.info(f"anneal from step {begin}: {anneal_steps} decay steps, training.steps "
                        f"{training.steps} -> {new_total}, decay_ratio {ratio} -> {anneal_steps / new_total:.6f}")
        training.steps = new_total
        sched.decay_ratio = anneal_steps / new_total
    return LRSchedule(opt.lr, training.steps, sched.warmup_steps, sched.decay_ratio, sched.decay_type, sched.lr_min)
