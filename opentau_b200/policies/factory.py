"""Policy registry: ``get_policy_class(name)``, ``make_policy_config``, ``make_policy``.

Mirrors the reference factory surface (OpenTau ``src/opentau/policies/factory.py:60-438``).
"""

from __future__ import annotations

import importlib
from typing import Any

from ..configs.policies import PreTrainedConfig
from .pretrained import PreTrainedPolicy

_POLICIES: dict[str, tuple[str, str, str]] = {
    # name: (module, policy class, config module)
    "pi05": ("opentau_b200.policies.pi05.modeling_pi05", "PI05Policy",
             "opentau_b200.policies.pi05.configuration_pi05"),
    "pi05_continuous_state": ("opentau_b200.policies.pi05.modeling_pi05", "PI05Policy",
                              "opentau_b200.policies.pi05.configuration_pi05"),
    "pi0": ("opentau_b200.policies.pi0.modeling_pi0", "PI0Policy", "opentau_b200.policies.pi0.configuration_pi0"),
    "cosmos3": ("opentau_b200.policies.cosmos3.modeling_cosmos3", "Cosmos3Policy",
                "opentau_b200.policies.cosmos3.configuration_cosmos3"),
    "cosmos3_nano": ("opentau_b200.policies.cosmos3_nano.modeling_cosmos3_nano", "Cosmos3NanoPolicy",
                     "opentau_b200.policies.cosmos3_nano.configuration_cosmos3_nano"),
    "pi07_low_level": ("opentau_b200.policies.pi07.low_level.modeling_pi07_low_level", "PI07LowLevelPolicy",
                       "opentau_b200.policies.pi07.low_level.configuration_pi07_low_level"),
    "pi07_high_level": ("opentau_b200.policies.pi07.high_level_planner.modeling_pi07_high_level",
                        "PI07HighLevelPlannerPolicy",
                        "opentau_b200.policies.pi07.high_level_planner.configuration_pi07_high_level"),
    "pi06": ("opentau_b200.policies.pi06.modeling_pi06", "PI06Policy",
             "opentau_b200.policies.pi06.configuration_pi06"),
    "pi05_mem": ("opentau_b200.policies.pi05_mem.modeling_pi05_mem", "PI05MemPolicy",
                 "opentau_b200.policies.pi05_mem.configuration_pi05_mem"),
    "pi07_paligemma_low_level": ("opentau_b200.policies.pi07_paligemma.low_level.modeling_pi07_low_level",
                                 "PI07PaligemmaLowLevelPolicy",
                                 "opentau_b200.policies.pi07_paligemma.low_level.configuration_pi07_low_level"),
    "pi07_paligemma_high_level_planner": (
        "opentau_b200.policies.pi07_paligemma.high_level_planner.modeling_pi07_high_level",
        "PI07PaligemmaHighLevelPlannerPolicy",
        "opentau_b200.policies.pi07_paligemma.high_level_planner.configuration_pi07_high_level"),
    "value": ("opentau_b200.policies.value.modeling_value", "ValueFunction",
              "opentau_b200.policies.value.configuration_value"),
}


def register_policy(name: str, module: str, cls: str, config_module: str) -> None:
    _POLICIES[name] = (module, cls, config_module)


def _import_all_configs() -> None:
    for _, _, cfgmod in _POLICIES.values():
        try:
            importlib.import_module(cfgmod)
        except ModuleNotFoundError:
            pass


def get_policy_class(name: str) -> type[PreTrainedPolicy]:
    if name not in _POLICIES:
        raise NotImplementedError(f"Policy with name {name} is not implemented.")
    module, cls, _ = _POLICIES[name]
    return getattr(importlib.import_module(module), cls)


def make_policy_config(policy_type: str, **kwargs) -> PreTrainedConfig:
    _import_all_configs()
    try:
        cls = PreTrainedConfig.get_choice_class(policy_type)
    except KeyError:
        raise ValueError(f"Policy type '{policy_type}' is not available.") from None
    return cls(**kwargs)


def make_policy(cfg: PreTrainedConfig, ds_meta: Any | None = None, per_dataset_stats: list[dict] | None = None,
                dataset_names: list[str] | None = None, **kwargs) -> PreTrainedPolicy:
    """Builds (or loads, when ``cfg.pretrained_path`` is set) a policy.

    ``ds_meta`` is a dataset-mixture metadata object exposing ``features``, ``per_dataset_stats`` and
    ``dataset_names``; its statistics fill the normalization heads and its features complete the
    config's ``input_features`` / ``output_features`` when those are empty.
    """
    _import_all_configs()
    policy_cls = get_policy_class(cfg.type)
    if ds_meta is not None:
        if per_dataset_stats is None:
            per_dataset_stats = getattr(ds_meta, "per_dataset_stats", None)
            if per_dataset_stats is None and getattr(ds_meta, "stats", None) is not None:
                per_dataset_stats = [ds_meta.stats]
        if dataset_names is None:
            dataset_names = getattr(ds_meta, "dataset_names", None)
        feats = getattr(ds_meta, "policy_features", None)
        if feats and not cfg.input_features and not cfg.output_features:
            from ..configs.types import FeatureType
            cfg.output_features = {k: f for k, f in feats.items() if f.type is FeatureType.ACTION}
            cfg.input_features = {k: f for k, f in feats.items() if f.type is not FeatureType.ACTION}
    if dataset_names is not None:
        cfg.dataset_names = list(dataset_names)
        cfg.dataset_to_norm_index = {n: i for i, n in enumerate(dataset_names)}
    cfg.validate_input_resolution(strict=True)
    if cfg.pretrained_path:
        policy = policy_cls.from_pretrained(cfg.pretrained_path, config=cfg, **kwargs)
        if per_dataset_stats is not None and cfg.skip_normalization_weights:
            policy._inject_stats(per_dataset_stats, dataset_names)
    else:
        policy = policy_cls(cfg, per_dataset_stats=per_dataset_stats, dataset_names=dataset_names, **kwargs)
    return policy
