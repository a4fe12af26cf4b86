"""``TrainPipelineConfig``: the root configuration of ``opentau-train`` / ``opentau-eval``.

Field names, defaults, the batch-size invariant, the pipeline->policy shape propagation and the
``train_config.json`` persistence follow the reference (OpenTau ``src/opentau/configs/train.py:83-668``).
The accelerate YAML surface is replaced by the ``distributed`` block.
"""

from __future__ import annotations

import json
import logging
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

from ..constants import TRAIN_CONFIG_NAME
from ..optim.optimizers import OptimizerConfig
from ..optim.schedulers import LRSchedulerConfig
from .codec import apply_overrides, decode, encode
from .default import DatasetMixtureConfig, DistributedConfig, EvalConfig, WandBConfig
from .deployment import PlannerConfig, ServerConfig
from .policies import PreTrainedConfig
from .refs import load_json_with_refs

# pipeline field -> policy field: the pipeline value overwrites the policy's
PIPELINE_TO_POLICY_SHAPE_FIELDS = {
    "max_state_dim": "max_state_dim",
    "max_action_dim": "max_action_dim",
    "action_chunk": "chunk_size",
}


@dataclass
class TrainPipelineConfig:
    dataset_mixture: DatasetMixtureConfig = field(default_factory=DatasetMixtureConfig)
    policy: PreTrainedConfig | None = None
    output_dir: str | None = None
    resume: bool = False
    seed: int | None = 1000
    resolution: tuple[int, int] = (224, 224)
    num_cams: int = 2
    max_state_dim: int = 32
    max_action_dim: int = 32
    action_chunk: int = 50
    loss_weighting: dict[str, float] = field(default_factory=lambda: {"MSE": 1.0, "CE": 1.0})
    num_workers: int = 4
    batch_size: int | None = None
    gradient_accumulation_steps: int = 1
    dataloader_batch_size: int | None = None
    prefetch_factor: int | None = None
    steps: int = 100_000
    log_freq: int = 200
    save_checkpoint: bool = True
    save_freq: int = 20_000
    use_policy_training_preset: bool = False
    optimizer: OptimizerConfig | None = None
    scheduler: LRSchedulerConfig | None = None
    wandb: WandBConfig = field(default_factory=WandBConfig)
    debug: bool = False
    trace_nans: bool = False
    env: Any | None = None
    eval: EvalConfig = field(default_factory=EvalConfig)
    eval_freq: int = 0
    val_freq: int = 0
    # None: a validation pass scores the WHOLE validation split (every sample once); a number caps the batches per rank
    val_max_batches: int | None = None
    last_checkpoint_only: bool = True
    running_best_count: int = 0
    running_best_metric: str = "auto"
    server: ServerConfig = field(default_factory=ServerConfig)
    planner: PlannerConfig = field(default_factory=PlannerConfig)
    distributed: DistributedConfig = field(default_factory=DistributedConfig)

    _deprecated_fields = ("job_name",)

    def __post_init__(self):
        self.checkpoint_path: Path | None = None
        self._resolve_batch_sizes()
        self._propagate_shape_fields()

    # -- invariants --------------------------------------------------------------------------------
    def _resolve_batch_sizes(self) -> None:
        ga = self.gradient_accumulation_steps
        if ga < 1:
            raise ValueError("gradient_accumulation_steps must be >= 1")
        if self.batch_size is None and self.dataloader_batch_size is None:
            self.dataloader_batch_size = 8
        if self.batch_size is None:
            self.batch_size = self.dataloader_batch_size * ga
        elif self.dataloader_batch_size is None:
            if self.batch_size % ga:
                raise ValueError(f"batch_size ({self.batch_size}) must be divisible by "
                                 f"gradient_accumulation_steps ({ga})")
            self.dataloader_batch_size = self.batch_size // ga
        if self.batch_size != self.dataloader_batch_size * ga:
            raise ValueError(f"batch_size ({self.batch_size}) must equal dataloader_batch_size "
                             f"({self.dataloader_batch_size}) * gradient_accumulation_steps ({ga})")

    def _propagate_shape_fields(self) -> None:
        if self.policy is None:
            return
        import dataclasses
        import logging
        declared = {f.name for f in dataclasses.fields(type(self.policy))} if dataclasses.is_dataclass(self.policy) else set()
        for src, dst in PIPELINE_TO_POLICY_SHAPE_FIELDS.items():
            if not hasattr(self.policy, dst):
                continue
            new, old = getattr(self, src), getattr(self.policy, dst, None)
            if dst in declared and old != new and old != type(self.policy).__dataclass_fields__[dst].default:
                # the data loader shapes every sample from the pipeline-level value, so it wins; say so when it
                # replaces a value that somebody set (a checkpoint's, say) rather than the class default
                logging.warning("overriding policy.%s=%s with %s=%s from the training config; to keep the policy's "
                                "value set %s=%s at the top level instead", dst, old, src, new, src, old)
            setattr(self.policy, dst, new)
        if hasattr(self.policy, "n_action_steps") and hasattr(self.policy, "chunk_size"):
            if self.policy.n_action_steps > self.policy.chunk_size:
                self.policy.n_action_steps = self.policy.chunk_size

    def _validate_loss_weighting(self) -> None:
        """Both terms must be named (a weight of exactly 0 drops that term from the backward pass, which is a supported
        way to train one head only), none may be negative, and at least one must be active
        (reference ``src/opentau/configs/train.py:435-465``)."""
        unknown = set(self.loss_weighting) - {"MSE", "CE"}
        if unknown:
            raise ValueError(f"unknown loss term(s) {sorted(unknown)} in loss_weighting (expected MSE / CE)")
        missing = {"MSE", "CE"} - set(self.loss_weighting)
        if missing:
            raise ValueError(f"loss_weighting must define weights for ['CE', 'MSE']; missing {sorted(missing)}. "
                             f"Got {self.loss_weighting}.")
        negative = {k: v for k, v in self.loss_weighting.items() if v < 0}
        if negative:
            raise ValueError(f"loss_weighting values must be >= 0; got negative entries {negative}.")
        if all(float(v) == 0.0 for v in self.loss_weighting.values()):
            raise ValueError("loss_weighting has all-zero weights; there is nothing to optimize")

    def _validate_data_matches_policy(self) -> None:
        """The loader delivers frames at ``resolution`` and ``n_obs_history`` steps of history: a policy that resizes to
        another size would letterbox every frame a second time, and one that expects another number of observation
        steps would meet the wrong time axis.  Training only (evaluation never calls ``validate``), so checkpoints
        trained with a mismatch stay evaluable; ``policy.skip_input_resolution_check`` downgrades the first to a warning
        (reference ``src/opentau/configs/train.py:395-433``)."""
        import logging
        resize = getattr(self.policy, "resize_imgs_with_padding", None)
        if resize is not None and tuple(resize) != tuple(self.resolution):
            msg = (f"policy.resize_imgs_with_padding={tuple(resize)} != resolution={tuple(self.resolution)} (both (H, W)): "
                   "the policy would resample and pad every frame a second time before the vision tower.  Set both to "
                   "the same value (Gemma-3 policies: the tower's image size), or policy.resize_imgs_with_padding=null "
                   "to pass frames through (PaliGemma-family policies only).")
            if getattr(self.policy, "skip_input_resolution_check", False):
                logging.warning("%s Proceeding because skip_input_resolution_check=true.", msg)
            else:
                raise ValueError(msg + " To resume a run trained with this mismatch set "
                                       "policy.skip_input_resolution_check=true.")
        if self.dataset_mixture is not None and self.dataset_mixture.datasets and hasattr(self.policy, "n_obs_steps"):
            want = self.dataset_mixture.n_obs_history if self.dataset_mixture.n_obs_history else 1
            if int(self.policy.n_obs_steps) != int(want):
                raise ValueError(f"policy.n_obs_steps ({self.policy.n_obs_steps}) != dataset_mixture.n_obs_history "
                                 f"({self.dataset_mixture.n_obs_history}; treated as 1 when unset): set "
                                 "dataset_mixture.n_obs_history to match")

    def validate(self) -> None:
        if self.policy is None:
            raise ValueError("a policy configuration is required (`policy.type=...` or `--policy.path=...`)")
        if not self.dataset_mixture.datasets and self.env is None:
            raise ValueError("at least one dataset (or an env for pure evaluation) is required")
        self._validate_loss_weighting()
        self._validate_data_matches_policy()
        self._validate_running_best()
        if self.use_policy_training_preset or self.optimizer is None:
            self.optimizer = self.optimizer if (self.optimizer and not self.use_policy_training_preset) \
                else self.policy.get_optimizer_preset()
            if self.scheduler is None or self.use_policy_training_preset:
                self.scheduler = self.policy.get_scheduler_preset()
        if self.output_dir is None:
            import datetime as dt
            now = dt.datetime.now()
            self.output_dir = str(Path("outputs/train") / f"{now:%Y-%m-%d}" / f"{now:%H-%M-%S}_{self.policy.type}")
        if not self.resume and Path(self.output_dir).is_dir() and any(Path(self.output_dir).iterdir()):
            ck = Path(self.output_dir) / "checkpoints"
            if ck.is_dir() and any(ck.iterdir()):
                raise FileExistsError(f"output directory {self.output_dir} already holds checkpoints and "
                                      "`resume` is False")
        self.policy.validate_action_horizon()

    def _validate_running_best(self) -> None:
        """``running_best_metric``: ``eval_success`` (keep the highest simulation success rates), ``val_loss`` (keep
        the lowest validation losses) or ``auto`` (success when an environment is evaluated during training, else
        validation loss).  The resolved choice is a runtime attribute, never saved: a resumed ``auto`` run stays
        ``auto`` (reference ``configs/train.py:438-516``)."""
        allowed = ("auto", "eval_success", "val_loss", "success")        # "success": accepted alias of eval_success
        if self.running_best_metric not in allowed:
            raise ValueError(f"running_best_metric must be one of {sorted(allowed[:3])}, got "
                             f"{self.running_best_metric!r}")
        if self.running_best_count < 0:
            raise ValueError(f"running_best_count must be >= 0, got {self.running_best_count}")
        self.running_best_metric_resolved = None
        if self.running_best_count == 0:
            return
        has_eval = self.env is not None and self.eval_freq > 0
        has_val = self.val_freq > 0
        metric = "eval_success" if self.running_best_metric == "success" else self.running_best_metric
        if metric == "eval_success" and not has_eval:
            raise ValueError("running_best_metric='eval_success' needs a simulation evaluation source: set env and "
                             "eval_freq > 0")
        if metric == "val_loss" and not has_val:
            raise ValueError("running_best_metric='val_loss' needs val_freq > 0")
        if metric == "auto" and not (has_eval or has_val):
            raise ValueError("running_best_count >= 1 but no metric source is configured: set eval_freq > 0 with an "
                             "env (success rate) or val_freq > 0 (validation loss)")
        self.running_best_metric_resolved = ("eval_success" if has_eval else "val_loss") if metric == "auto" else metric

    # -- persistence -------------------------------------------------------------------------------
    def to_dict(self) -> dict[str, Any]:
        return encode(self)

    def _save_pretrained(self, save_directory: str | Path) -> None:
        Path(save_directory).mkdir(parents=True, exist_ok=True)
        with open(Path(save_directory) / TRAIN_CONFIG_NAME, "w") as f:
            json.dump(self.to_dict(), f, indent=4)

    save_pretrained = _save_pretrained

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "TrainPipelineConfig":
        _import_policy_configs()
        return decode(cls, raw)

    @staticmethod
    def _locate_config_file(config_path: str | Path) -> Path:
        """A JSON file; a directory holding ``train_config.json`` or, failing that, ``hf_config.json`` (the name
        the publishing tools give the pipeline config of an uploaded checkpoint); or ``repo[@revision]`` in the local
        cache with the same two names (reference ``configs/train.py:596-640``).  A revision that is not cached is
        reported with the revisions that are."""
        from ..utils.hub import HF_OPENTAU_HOME, split_repo_revision
        names = (TRAIN_CONFIG_NAME, "hf_config.json")
        p = Path(str(config_path))
        if p.is_file():
            return p
        if p.is_dir():
            for n in names:
                if (p / n).is_file():
                    return p / n
            raise FileNotFoundError(f"neither {names[0]} nor {names[1]} found in {p.resolve()}")
        repo, rev = split_repo_revision(str(config_path))
        repo_dir = HF_OPENTAU_HOME / repo
        if not repo_dir.is_dir():
            raise FileNotFoundError(f"{config_path!r} is not a file, not a directory and not in the local cache "
                                    f"({repo_dir}); this installation does not download")
        from ..utils.hub import cached_revision_dir
        root = cached_revision_dir(repo_dir, rev)
        if rev and not root.is_dir():
            tags = sorted(d.name for d in repo_dir.iterdir() if d.is_dir())
            raise FileNotFoundError(f"revision {rev!r} does not exist in cached repository {repo!r}; training steps "
                                    f"are published as tags named by step number (cached: {tags or 'none'}).  Omit "
                                    "the '@<step>' suffix to load the latest step.")
        for n in names:
            if (root / n).is_file():
                return root / n
        raise FileNotFoundError(f"neither {names[0]} nor {names[1]} was found in {root}")

    @classmethod
    def from_pretrained(cls, config_path: str | Path, cli_overrides: list[str] | None = None) -> "TrainPipelineConfig":
        """Loads a JSON config (a file, a checkpoint directory holding ``train_config.json``, or a cached
        ``repo@rev``); ``$ref`` includes are resolved, then dotted CLI overrides applied.  With
        ``--resume=true`` the checkpoint's own ``train_config.json`` wins over the CLI for everything but
        ``steps``/``resume`` (reference ``configs/train.py:352-366``)."""
        p = cls._locate_config_file(config_path)
        raw = load_json_with_refs(p)
        overrides = list(cli_overrides or [])
        policy_path = None
        kept = []
        for a in overrides:
            if a.startswith("--policy.path="):
                policy_path = a.split("=", 1)[1]
            else:
                kept.append(a)
        raw = apply_overrides(raw, kept)
        if policy_path is not None:
            pcfg = PreTrainedConfig.from_pretrained(policy_path)
            merged = encode(pcfg)
            merged.update({k: v for k, v in (raw.get("policy") or {}).items() if k != "type"})
            merged["pretrained_path"] = policy_path
            raw["policy"] = merged
        cfg = cls.from_dict(raw)
        if cfg.resume:
            cfg.checkpoint_path = p.parent
        return cfg


def _import_policy_configs() -> None:
    from ..policies.factory import _import_all_configs
    _import_all_configs()
