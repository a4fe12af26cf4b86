"""Optimizer configurations (choice registry ``adam`` / ``adamw`` / ``sgd``).

Defaults follow the reference (OpenTau ``src/opentau/optim/optimizers.py:54-110``).  ``build`` returns a
``torch.optim`` optimizer for the generic path; the B200 training engine instead reads these
hyper-parameters and runs its own fused flat AdamW (``parallel/engine.py``).
"""

from __future__ import annotations

import abc
from dataclasses import asdict, dataclass
from pathlib import Path

import torch

from ..configs.codec import ChoiceRegistry


@dataclass
class OptimizerConfig(ChoiceRegistry, abc.ABC):
    lr: float = 1e-4
    weight_decay: float = 0.0
    grad_clip_norm: float = 10.0

    @property
    def type(self) -> str:
        return self.get_choice_name()

    @abc.abstractmethod
    def build(self, params) -> torch.optim.Optimizer: ...


@OptimizerConfig.register_subclass("adam")
@dataclass
class AdamConfig(OptimizerConfig):
    lr: float = 1e-3
    betas: tuple[float, float] = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 0.0
    grad_clip_norm: float = 10.0

    def build(self, params):
        kw = asdict(self)
        kw.pop("grad_clip_norm")
        return torch.optim.Adam(params, **kw)


@OptimizerConfig.register_subclass("adamw")
@dataclass
class AdamWConfig(OptimizerConfig):
    lr: float = 1e-3
    betas: tuple[float, float] = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 1e-2
    grad_clip_norm: float = 10.0
    fused: bool = True

    def build(self, params):
        kw = asdict(self)
        kw.pop("grad_clip_norm")
        fused = kw.pop("fused")
        params = list(params)
        on_cuda = any((p.is_cuda if isinstance(p, torch.Tensor) else any(q.is_cuda for q in p["params"]))
                      for p in params)
        return torch.optim.AdamW(params, fused=bool(fused and on_cuda), **kw)


@OptimizerConfig.register_subclass("sgd")
@dataclass
class SGDConfig(OptimizerConfig):
    lr: float = 1e-3
    momentum: float = 0.0
    dampening: float = 0.0
    nesterov: bool = False
    weight_decay: float = 0.0
    grad_clip_norm: float = 10.0

    def build(self, params):
        kw = asdict(self)
        kw.pop("grad_clip_norm")
        return torch.optim.SGD(params, **kw)


def save_optimizer_state(optimizer: torch.optim.Optimizer, save_dir: Path) -> None:
    """Tensors go to safetensors, param-group scalars to JSON (reference ``optimizers.py:113-134``)."""
    import json

    from safetensors.torch import save_file

    from ..constants import OPTIMIZER_PARAM_GROUPS, OPTIMIZER_STATE
    state = optimizer.state_dict()
    flat = {}
    for pid, st in state["state"].items():
        for k, v in st.items():
            flat[f"state/{pid}/{k}"] = v.detach().cpu().contiguous() if isinstance(v, torch.Tensor) else torch.tensor(v)
    save_dir.mkdir(parents=True, exist_ok=True)
    save_file(flat, str(save_dir / OPTIMIZER_STATE))
    with open(save_dir / OPTIMIZER_PARAM_GROUPS, "w") as f:
        json.dump(state["param_groups"], f, indent=2)


def load_optimizer_state(optimizer: torch.optim.Optimizer, save_dir: Path) -> torch.optim.Optimizer:
    import json

    from safetensors.torch import load_file

    from ..constants import OPTIMIZER_PARAM_GROUPS, OPTIMIZER_STATE
    flat = load_file(str(save_dir / OPTIMIZER_STATE))
    with open(save_dir / OPTIMIZER_PARAM_GROUPS) as f:
        groups = json.load(f)
    cur = optimizer.state_dict()
    st: dict = {}
    for key, v in flat.items():
        _, pid, name = key.split("/", 2)
        st.setdefault(int(pid), {})[name] = v
    for g_new, g_old in zip(groups, cur["param_groups"]):
        g_new["params"] = g_old["params"]
    optimizer.load_state_dict({"state": st, "param_groups": groups})
    return optimizer
