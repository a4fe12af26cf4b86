"""Learning-rate schedules (choice registry ``diffuser`` / ``vqbet`` / ``cosine_decay_with_warmup`` /
``constant``).  ``lr_lambda`` is exposed so the B200 engine can evaluate the multiplier itself.

Formulas follow the reference (OpenTau ``src/opentau/optim/schedulers.py:44-129``).
"""

from __future__ import annotations

import abc
import math
from dataclasses import dataclass

from torch.optim.lr_scheduler import LambdaLR

from ..configs.codec import ChoiceRegistry


@dataclass
class LRSchedulerConfig(ChoiceRegistry, abc.ABC):
    num_warmup_steps: int = 0

    @property
    def type(self) -> str:
        return self.get_choice_name()

    @abc.abstractmethod
    def lr_lambda(self, num_training_steps: int): ...

    def build(self, optimizer, num_training_steps: int) -> LambdaLR:
        return LambdaLR(optimizer, self.lr_lambda(num_training_steps), -1)


@LRSchedulerConfig.register_subclass("constant")
@dataclass
class ConstantSchedulerConfig(LRSchedulerConfig):
    num_warmup_steps: int = 0

    def lr_lambda(self, num_training_steps: int):
        w = self.num_warmup_steps

        def f(step: int) -> float:
            if w > 0 and step < w:
                return (step + 1) / (w + 1)
            return 1.0
        return f


@LRSchedulerConfig.register_subclass("diffuser")
@dataclass
class DiffuserSchedulerConfig(LRSchedulerConfig):
    name: str = "cosine"
    num_warmup_steps: int = 0

    def lr_lambda(self, num_training_steps: int):
        w = self.num_warmup_steps

        def f(step: int) -> float:
            if step < w:
                return step / max(1, w)
            if self.name == "constant":
                return 1.0
            prog = (step - w) / max(1, num_training_steps - w)
            if self.name == "linear":
                return max(0.0, 1.0 - prog)
            return max(0.0, 0.5 * (1.0 + math.cos(math.pi * min(1.0, prog))))
        return f


@LRSchedulerConfig.register_subclass("vqbet")
@dataclass
class VQBeTSchedulerConfig(LRSchedulerConfig):
    num_warmup_steps: int = 0
    num_vqvae_training_steps: int = 0
    num_cycles: float = 0.5

    def lr_lambda(self, num_training_steps: int):
        def f(step: int) -> float:
            if step < self.num_vqvae_training_steps:
                return 1.0
            s = step - self.num_vqvae_training_steps
            if s < self.num_warmup_steps:
                return s / max(1, self.num_warmup_steps)
            prog = (s - self.num_warmup_steps) / max(1, num_training_steps - self.num_warmup_steps)
            return max(0.0, 0.5 * (1.0 + math.cos(math.pi * self.num_cycles * 2.0 * prog)))
        return f


@LRSchedulerConfig.register_subclass("cosine_decay_with_warmup")
@dataclass
class CosineDecayWithWarmupSchedulerConfig(LRSchedulerConfig):
    """Linear warmup ``1/(W+1) -> 1`` over ``W`` steps, then cosine decay to ``decay_lr/peak_lr``."""

    num_warmup_steps: int = 1000
    num_decay_steps: int = 30000
    peak_lr: float = 2.5e-5
    decay_lr: float = 2.5e-6

    def lr_lambda(self, num_training_steps: int):
        W, D = self.num_warmup_steps, self.num_decay_steps
        alpha = self.decay_lr / self.peak_lr

        def f(step: int) -> float:
            if step < W:
                if step <= 0:
                    return 1.0 / (W + 1)
                frac = 1.0 - step / W
                return (1.0 / (W + 1) - 1.0) * frac + 1.0
            s = min(step, D)
            return (1.0 - alpha) * 0.5 * (1.0 + math.cos(math.pi * s / D)) + alpha
        return f
