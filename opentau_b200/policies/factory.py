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


def load_norm_stats_override(path: str, num_heads: int) -> list[dict]:
    """An openpi-style ``norm_stats.json`` (``{"norm_stats": {"state": {...}, "actions": {...}}}`` with ``mean`` / ``std``
    and optionally ``min`` / ``max`` / ``q01`` / ``q99``), replicated over every head.  Meant for replaying a teacher
    checkpoint under the statistics it was trained with; every head then shares one scale, hence the warning
    (reference ``src/opentau/policies/factory.py:186-233``)."""
    import json
    import logging

    import numpy as np
    logging.warning("norm_stats_override_path=%s: the dataset-derived statistics are REPLACED by this file for all %d "
                    "head(s); per-dataset normalisation is lost.  Prefer a converted checkpoint with the right "
                    "statistics stored in it.", path, num_heads)
    with open(path) as f:
        raw = json.load(f)["norm_stats"]

    def feature(name: str) -> dict:
        if name not in raw:
            raise KeyError(f"norm_stats_override_path={path!r} has no '{name}' entry under 'norm_stats' (found {sorted(raw)})")
        return {k: np.asarray(raw[name][k], np.float32) for k in ("mean", "std", "min", "max", "q01", "q99") if k in raw[name]}

    head = {"state": feature("state"), "actions": feature("actions")}
    return [{k: dict(v) for k, v in head.items()} for _ in range(num_heads)]      # rows must not alias each other


def make_policy(cfg: PreTrainedConfig, ds_meta: Any | None = None, per_dataset_stats: list[dict] | None = None,
                dataset_names: list[str] | None = None, *, features: dict | None = None,
                stats: dict | list[dict] | None = None, execution_target: str | None = None,
                **kwargs) -> PreTrainedPolicy:
    """Builds (or loads, when ``cfg.pretrained_path`` is set) a policy
    (reference ``src/opentau/policies/factory.py:236-438``).

    Statistics come, in this order of precedence, from ``cfg.norm_stats_override_path`` (one file for every head),
    ``stats`` / ``per_dataset_stats`` (caller-supplied, no dataset identity: inference must then use ``dataset_index``
    or the head names), or ``ds_meta``: a mixture's metadata (``per_norm_key_stats`` / ``norm_keys`` /
    ``dataset_to_norm_index``, pooled per ``(robot_type, control_mode)``) or one dataset's (``stats`` + ``info``: a
    single head keyed by its tags).  The head keys go to ``cfg.dataset_names`` (one per row of the stacked buffers) and
    the dataset-name table to ``cfg.dataset_to_norm_index``, so a saved checkpoint can resolve ``dataset_repo_id`` also
    where several datasets share a head.  ``features`` (or ``ds_meta``'s) complete empty ``input_features`` /
    ``output_features``.  A mixture's delta-action map is stored on the config (pi05 inverts it in ``sample_actions``);
    a policy type without that field refuses such a mixture.  ``execution_target``: ``None`` (training), ``"robot"``
    (action decoder only) or ``"cloud"`` (VLM only), forwarded to policies that split.

    After a load, buffers that are still ``+inf`` (a checkpoint saved without statistics) are filled from the supplied
    statistics; buffers that did load are kept, so ``skip_normalization_weights=False`` really keeps the checkpoint's."""
    from ..configs.policies import CURRENT_CONFIG_VERSION
    from ..configs.types import FeatureType
    _import_all_configs()
    if execution_target not in ("robot", "cloud", None):
        raise ValueError(f"execution_target must be one of ['robot', 'cloud', None], got {execution_target!r}")
    policy_cls = get_policy_class(cfg.type)
    norm_keys: list[str] | None = list(dataset_names) if dataset_names is not None else None
    dataset_to_norm_index: dict[str, int] | None = None
    head_stats: list[dict] | None = list(per_dataset_stats) if per_dataset_stats is not None else None
    if ds_meta is not None:
        if head_stats is None:
            if hasattr(ds_meta, "per_norm_key_stats") and hasattr(ds_meta, "norm_keys"):
                head_stats = list(ds_meta.per_norm_key_stats)
                norm_keys = norm_keys or list(ds_meta.norm_keys)
                dataset_to_norm_index = dict(ds_meta.dataset_to_norm_index)
            elif getattr(ds_meta, "per_dataset_stats", None) is not None:
                head_stats = list(ds_meta.per_dataset_stats)
                norm_keys = norm_keys or (list(ds_meta.dataset_names) if getattr(ds_meta, "dataset_names", None) else None)
                dataset_to_norm_index = dict(getattr(ds_meta, "dataset_to_norm_index", None) or {}) or None
            elif getattr(ds_meta, "stats", None) is not None:
                from ..datasets.dataset_mixture import compute_norm_key
                repo_id = getattr(ds_meta, "repo_id", "default")
                info = getattr(ds_meta, "info", None) or {}
                key, _ = compute_norm_key(info.get("robot_type"), info.get("control_mode"), repo_id)
                head_stats, norm_keys, dataset_to_norm_index = [ds_meta.stats], norm_keys or [key], {repo_id: 0}
        if features is None:
            features = getattr(ds_meta, "policy_features", None)
    if not features and not cfg.input_features and not cfg.output_features and cfg.pretrained_path:
        # a pipeline config whose policy block names a checkpoint but binds no features (an eval / diagnosis run
        # started from the TRAINING config): the checkpoint knows what it was built with
        try:
            saved = PreTrainedConfig.from_pretrained(cfg.pretrained_path)
            features = {**(saved.input_features or {}), **(saved.output_features or {})} or None
            if features:
                import logging
                logging.info("policy features taken from the checkpoint's configuration (%s)", cfg.pretrained_path)
                if not cfg.dataset_names and saved.dataset_names and norm_keys is None:
                    cfg.dataset_names, cfg.dataset_to_norm_index = saved.dataset_names, saved.dataset_to_norm_index
        except Exception:  # noqa: BLE001 - no readable configuration beside the weights: construction reports it
            features = None
    if features and not cfg.input_features and not cfg.output_features:
        cfg.output_features = {k: f for k, f in features.items() if f.type is FeatureType.ACTION}
        cfg.input_features = {k: f for k, f in features.items() if f.type is not FeatureType.ACTION}
    if stats is not None:
        head_stats = [stats] if isinstance(stats, dict) else list(stats)
        norm_keys = norm_keys or (["external"] if isinstance(stats, dict) else [f"external_{i}" for i in range(len(head_stats))])
        dataset_to_norm_index = None
    delta_map = getattr(ds_meta, "delta_action_state_map", None)
    if delta_map:
        if not hasattr(cfg, "delta_action_state_map"):
            raise ValueError(f"the dataset mixture uses delta joint actions (post-index map {dict(delta_map)}), but policy "
                             f"type '{cfg.type}' has no `delta_action_state_map` field and no inverse at inference: it "
                             "would emit displacements that are read as absolute actions.  Use policy.type=pi05, or take "
                             "`use_delta_joint_actions` out of the mixture.")
        cfg.delta_action_state_map = {int(a): int(b) for a, b in delta_map.items()}
    override = getattr(cfg, "norm_stats_override_path", None)
    if override:
        head_stats = load_norm_stats_override(override, num_heads=len(norm_keys) if norm_keys else 1)
        norm_keys = norm_keys or [f"override_{i}" for i in range(len(head_stats))]
    if norm_keys is not None:
        cfg.dataset_names = list(norm_keys)
        cfg.dataset_to_norm_index = dict(dataset_to_norm_index) if dataset_to_norm_index else (
            None if stats is not None else {n: i for i, n in enumerate(norm_keys)})
    if ds_meta is not None:
        cfg.validate_input_resolution(strict=True)       # training-shaped call: a double letterbox is an error
    if execution_target is not None:
        kwargs["execution_target"] = execution_target
    if cfg.pretrained_path:
        load_kw = dict(kwargs)
        if head_stats is not None:
            load_kw.update(per_dataset_stats=head_stats, dataset_names=norm_keys)
        policy = policy_cls.from_pretrained(cfg.pretrained_path, config=cfg, **load_kw)
        if head_stats is not None and policy._norm_buffers_have_inf():
            policy._inject_stats(head_stats, norm_keys)
        else:
            policy._check_norm_stats_loaded()
    else:
        policy = policy_cls(cfg, per_dataset_stats=head_stats, dataset_names=norm_keys, **kwargs)
    if cfg.config_version is None:
        cfg.config_version = CURRENT_CONFIG_VERSION      # a fresh policy is current: its saves must say so
    return policy
