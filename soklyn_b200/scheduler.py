"""Learning-rate schedulers of the reference (src/util/scheduler.rs), host scalars in f32."""
from __future__ import annotations

import math
from enum import Enum

import numpy as np

_f = np.float32


class CosineDecayLR:
    """Linear warm-up from min_lr to max_lr, then cosine decay back to min_lr (scheduler.rs:3-78)."""

    def __init__(self, min_lr: float, max_lr: float, total_step: int, warmup_steps: int):
        self.min_lr, self.max_lr = _f(min_lr), _f(max_lr)
        self.cur_lr = _f(min_lr)
        self.cur_step, self.total_step, self.warmup_steps = 0, total_step, warmup_steps
        self._update()

    def _update(self):
        if self.cur_step < self.warmup_steps:
            progress = _f(self.cur_step) / _f(self.warmup_steps)
            self.cur_lr = _f(self.min_lr + progress * (self.max_lr - self.min_lr))
            return
        decay_total = self.total_step - self.warmup_steps
        if decay_total == 0:
            self.cur_lr = self.min_lr
            return
        progress = _f(self.cur_step - self.warmup_steps) / _f(decay_total)
        self.cur_lr = _f(self.min_lr + _f(0.5) * (self.max_lr - self.min_lr) * (_f(1.0) + np.cos(progress * _f(math.pi))))

    def reset(self):
        self.cur_step = 0
        self._update()

    def get_learning_rate(self) -> float:
        return float(self.cur_lr)

    def step(self) -> float:
        self.cur_step += 1
        self._update()
        return float(self.cur_lr)


class ExponentialLR:
    """lr *= factor each step (scheduler.rs:81-123)."""

    def __init__(self, lr_initial: float, lr_factor: float):
        self.ori_lr = self.cur_lr = _f(lr_initial)
        self.lr_factor = _f(lr_factor)

    def reset(self):
        self.cur_lr = self.ori_lr

    def get_learning_rate(self) -> float:
        return float(self.cur_lr)

    def step(self) -> float:
        self.cur_lr = _f(self.cur_lr * self.lr_factor)
        return float(self.cur_lr)


class SchedulerMode(Enum):
    Minimize = 0
    Maximize = 1


class ReduceLROnPlateauScheduler:
    """Multiply the rate by lr_factor after `patience` steps without improvement (scheduler.rs:127-231)."""

    def __init__(self, patience: int, mode: SchedulerMode, lr_factor: float, min_lr: float):
        assert patience != 0, "Patience must be non-zero."
        self.mode, self.patience = mode, patience
        self.lr_factor, self.min_lr, self.cur_lr = _f(lr_factor), _f(min_lr), _f(0.0)
        self.timer = 0
        self.best_val = self._worst()

    def _worst(self):
        m = np.finfo(np.float32).max
        return _f(-m) if self.mode == SchedulerMode.Maximize else _f(m)

    def reset(self, learning_rate: float):
        self.cur_lr, self.timer, self.best_val = _f(learning_rate), 0, self._worst()

    def get_learning_rate(self) -> float:
        return float(self.cur_lr)

    def step(self, test_val: float) -> float:
        if math.isnan(test_val):
            return float(self.cur_lr)
        v = _f(test_val)
        improved = v > self.best_val if self.mode == SchedulerMode.Maximize else v < self.best_val
        if improved:
            self.best_val, self.timer = v, 0
        else:
            self.timer += 1
            if self.timer == self.patience:
                self.timer = 0
                self.cur_lr = max(_f(self.cur_lr * self.lr_factor), self.min_lr)
        return float(self.cur_lr)
