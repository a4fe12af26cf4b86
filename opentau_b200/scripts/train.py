"""``opentau-train``: the training loop.

Same stages and user-visible behaviour as the reference trainer (``src/opentau/scripts/train.py:708-1609``) —
config validation, one process per GPU, rank-0 output directory broadcast, seeding with a per-rank offset, dataset
mixture (+ validation split), policy construction with normalisation heads from the mixture statistics, bf16
weights with fp32 masters, gradient accumulation, weighted loss assembly, clipping, cosine schedule, per-step
metric gathers, periodic logging / checkpoints (with pruning, running-best retention and an interrupted-save
tripwire) / validation (bucketed per normalisation head and per dataset) / simulated-environment evaluation, and
resume.  What differs is the machinery underneath: :class:`~opentau_b200.parallel.engine.TrainEngine` owns flat
bf16 parameter / gradient buffers, sharded fp32 masters and the fused gradient-reduce + AdamW + parameter-gather
kernels over peer memory, instead of accelerate's DDP / DeepSpeed / FSDP wrappers.

Run one process per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m opentau_b200.scripts.train --config_path=cfg.json --steps=1000
"""

from __future__ import annotations

import json
import logging
import os
import time
from pathlib import Path
from typing import Any

import torch
import torch.distributed as dist
from torch import Tensor

from ..configs import parser
from ..configs.train import TrainPipelineConfig
from ..datasets.factory import make_dataset_mixture, warn_if_resumed_split_differs
from ..datasets.utils import cycle
from ..parallel import control
from ..parallel.fsdp import make_engine
from ..parallel.engine import OptimHyper, TrainEngine, assemble_weighted_loss
from ..policies.factory import make_policy
from ..utils.logging_utils import AverageMeter, MetricsTracker, format_big_number, init_logging
from ..utils.random_utils import set_seed
from ..utils.train_utils import (RunningBestTracker, checkpoint_is_complete, get_step_checkpoint_dir,
                                 get_step_identifier, load_training_state, prune_checkpoints, save_checkpoint,
                                 update_last_checkpoint)

CHECKPOINTS_DIR = "checkpoints"
LAST_LINK = "last"


# ---------------------------------------------------------------------------------------------- helpers
def init_distributed() -> tuple[int, int, torch.device]:
    """Joins the process group described by the launcher's environment (``RANK`` / ``WORLD_SIZE`` / ...)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if torch.cuda.is_available():
        torch.cuda.set_device(local % torch.cuda.device_count())
        device = torch.device("cuda", local % torch.cuda.device_count())
    else:
        device = torch.device("cpu")
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if device.type == "cuda":
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world)
    return rank, world, device


def to_device(batch: dict[str, Any], device: torch.device) -> dict[str, Any]:
    return {k: (v.to(device, non_blocking=True) if isinstance(v, Tensor) else v) for k, v in batch.items()}


class WandBLogger:
    """Thin tracker: wandb when enabled and importable (offline mode works without network), else a JSONL file."""

    def __init__(self, cfg: TrainPipelineConfig, out_dir: Path, is_main: bool, resume_step: int | None = None):
        self.run = None
        self.file = None
        if not is_main:
            return
        self.file = open(out_dir / "metrics.jsonl", "a")
        w = cfg.wandb
        if getattr(w, "enable", False):
            try:
                import wandb
                os.environ.setdefault("WANDB_MODE", getattr(w, "mode", None) or "offline")
                # a resumed run forks from (or continues) its parent as `wandb.on_resume` says
                kw = w.to_wandb_kwargs(step=resume_step if cfg.resume else None)
                kw["name"] = kw.get("name") or out_dir.name
                self.run = wandb.init(project=w.project or "opentau", dir=str(out_dir), config=cfg.to_dict(), **kw)
            except Exception as e:  # noqa: BLE001 - logging must never stop a run
                logging.warning("wandb disabled: %s", e)

    def log(self, metrics: dict[str, float], step: int) -> None:
        if self.file is not None:
            import json
            self.file.write(json.dumps({"step": step, **{k: float(v) for k, v in metrics.items()}}) + "\n")
            self.file.flush()
        if self.run is not None:
            self.run.log(metrics, step=step, commit=True)

    def log_videos(self, videos: dict[str, str], step: int, enabled: bool = True) -> None:
        """Grid-summary videos go to the experiment tracker (never the per-episode clips); without a tracker the paths
        are noted in the metrics file so that they can be found later."""
        if not videos or not enabled:
            return
        if self.file is not None:
            import json
            self.file.write(json.dumps({"step": step, "videos": videos}) + "\n")
            self.file.flush()
        if self.run is not None:
            try:
                import wandb
                self.run.log({k: wandb.Video(v, format="mp4") for k, v in videos.items()}, step=step)
            except Exception as e:  # noqa: BLE001 - logging must never stop a run
                logging.warning("video logging skipped: %s", e)

    def finish(self) -> None:
        if self.file is not None:
            self.file.close()
        if self.run is not None:
            self.run.finish()


def bucket_per_sample(per_sample: dict[str, Tensor], dataset_index: Tensor, names: list[str]) -> dict[str, dict[str, float]]:
    """Groups per-sample ``(sum, count)`` losses by normalisation head: exact masked means per group."""
    out: dict[str, dict[str, float]] = {}
    for i, name in enumerate(names):
        sel = dataset_index == i
        if not bool(sel.any()):
            continue
        row = {}
        for key in ("MSE", "CE"):
            s, c = per_sample[f"{key}_sum"][sel].sum(), per_sample[f"{key}_count"][sel].sum()
            row[key] = float(s / c.clamp(min=1))
            row[f"{key}_count"] = float(c)
        row["n"] = float(sel.sum())
        out[name] = row
    return out


def mixture_weighted_aggregate(buckets: dict[str, dict[str, float]], weights: dict[str, float]) -> dict[str, float]:
    """Validation losses weighted like the training mixture, over the heads that actually occurred."""
    tot = sum(weights.get(k, 0.0) for k in buckets) or 1.0
    return {key: sum(weights.get(k, 0.0) * b[key] for k, b in buckets.items()) / tot for key in ("MSE", "CE")}


@torch.no_grad()
def run_validation(policy, loader, n_batches: int | None, device, names: list[str], weights: dict[str, float],
                   loss_weights: dict[str, float], dataset_names: list[str] | None = None) -> dict[str, float]:
    """One pass over ``loader`` (all of it, or ``n_batches`` per rank) without gradients.

    Policies whose ``forward`` takes ``return_per_sample`` report per-sample ``(sum, count)`` losses; those are
    gathered from all ranks (the ranks' last shards may differ in length) and split per normalisation head
    (``Validation/<head>/...``, the headline) and per source dataset (``Validation/by_dataset/<name>/...``: nothing is
    lost where datasets share a head).  The overall ``Validation/Loss`` weights the heads like the TRAINING mixture, so
    it is not dominated by whichever head has the most validation frames.  Other policies (planners, value heads) get
    the batch-mean aggregate only; their optional ``L1`` / ``Accuracy`` outputs are averaged
    (reference ``src/opentau/scripts/train.py:1225-1436``)."""
    import inspect
    was_training = policy.training
    policy.eval()
    per_sample_ok = "return_per_sample" in inspect.signature(policy.forward).parameters
    keys = ("MSE_sum", "MSE_count", "CE_sum", "CE_count", "idx", "src")
    acc: dict[str, list[Tensor]] = {k: [] for k in keys}
    plain: dict[str, list[Tensor]] = {"MSE": [], "CE": [], "L1": [], "Accuracy": []}
    src_of = {n: i for i, n in enumerate(dataset_names or [])}
    threshold = getattr(getattr(policy, "config", None), "warn_outlier_threshold", None)
    for bi, raw in enumerate(loader):
        if n_batches is not None and bi >= n_batches:
            break
        batch = to_device(raw, device)
        out = policy(batch, return_per_sample=True) if per_sample_ok else policy(batch)
        records = out.pop("outlier_records", []) if isinstance(out, dict) else []
        if threshold is not None and threshold > 0:
            from ..policies.outlier_utils import log_outlier_records_distributed
            log_outlier_records_distributed(records, threshold)
        B = next(v.shape[0] for v in batch.values() if isinstance(v, Tensor) and v.dim() > 0)
        for key in ("L1", "Accuracy"):
            if key in out:
                plain[key].append(out[key].detach().float().reshape(1))
        if per_sample_ok and out.get("MSE_per_sample") is not None:
            for key in ("MSE", "CE"):
                ps = out.get(f"{key}_per_sample")
                s_, c_ = ps if ps is not None else (torch.zeros(B, device=device), torch.zeros(B, device=device))
                acc[f"{key}_sum"].append(s_.float()), acc[f"{key}_count"].append(c_.float())
            acc["idx"].append(torch.as_tensor(batch.get("dataset_index", torch.zeros(B, dtype=torch.long)),
                                              device=device).long().reshape(-1))
            repo = batch.get("dataset_repo_id")
            acc["src"].append(torch.tensor([src_of.get(r, -1) for r in repo], dtype=torch.long, device=device)
                              if repo is not None and src_of else torch.full((B,), -1, dtype=torch.long, device=device))
        else:
            for key in ("MSE", "CE"):
                if key in out:
                    plain[key].append(out[key].detach().float().reshape(1))
    policy.train(was_training)
    metrics: dict[str, float] = {}
    for key, label in (("L1", "Validation/L1 Loss"), ("Accuracy", "Validation/Accuracy")):
        if plain[key]:
            metrics[label] = float(control.gather_ragged({"v": torch.cat(plain[key])})["v"].mean())
    if acc["idx"]:
        flat = control.gather_ragged({k: torch.cat(v) for k, v in acc.items()})
        buckets = bucket_per_sample(flat, flat["idx"], names)
        for name, row in buckets.items():
            metrics[f"Validation/{name}/MSE Loss"] = row["MSE"]
            metrics[f"Validation/{name}/CE Loss"] = row["CE"]
            metrics[f"Validation/{name}/Loss"] = loss_weights.get("MSE", 1.0) * row["MSE"] + loss_weights.get("CE", 1.0) * row["CE"]
        if dataset_names and bool((flat["src"] >= 0).any()):
            for name, row in bucket_per_sample(flat, flat["src"], dataset_names).items():
                metrics[f"Validation/by_dataset/{name}/MSE Loss"] = row["MSE"]
                metrics[f"Validation/by_dataset/{name}/CE Loss"] = row["CE"]
                metrics[f"Validation/by_dataset/{name}/Loss"] = (loss_weights.get("MSE", 1.0) * row["MSE"]
                                                                 + loss_weights.get("CE", 1.0) * row["CE"])
        agg = mixture_weighted_aggregate(buckets, weights)
        metrics["Validation/Num Samples"] = float(flat["idx"].shape[0])
    elif plain["MSE"] or plain["CE"]:
        agg = {k: (float(control.gather_ragged({"v": torch.cat(plain[k])})["v"].mean()) if plain[k] else 0.0)
               for k in ("MSE", "CE")}
    else:
        return metrics
    metrics["Validation/MSE Loss"], metrics["Validation/CE Loss"] = agg["MSE"], agg["CE"]
    metrics["Validation/Loss"] = loss_weights.get("MSE", 1.0) * agg["MSE"] + loss_weights.get("CE", 1.0) * agg["CE"]
    return metrics


def update_policy(engine: TrainEngine, batches: list[dict[str, Any]]) -> dict[str, Tensor]:
    """One optimizer step over ``len(batches)`` micro-batches (gradient accumulation)."""
    sums: dict[str, Tensor] = {}
    records: list[dict[str, Any]] = []
    for b in batches:
        out = engine.forward_backward(b)
        records += out.pop("outlier_records", [])
        for k, v in out.items():
            sums[k] = sums.get(k, 0) + v.float() / len(batches)
    sums["grad_norm"] = engine.optimizer_step().float()
    # State / action outliers found inside forward (policies with ``warn_outlier_threshold``): every rank takes part,
    # rank 0 warns once per offender, whichever rank held the sample (reference scripts/train.py:282-287, 350-425).
    threshold = getattr(getattr(engine.policy, "config", None), "warn_outlier_threshold", None)
    if threshold is not None and threshold > 0:
        from ..policies.outlier_utils import log_outlier_records_distributed
        log_outlier_records_distributed(records, threshold)
    return sums


# ---------------------------------------------------------------------------------------------- main
def train(cfg: TrainPipelineConfig) -> dict[str, float]:
    rank, world, device = init_distributed()
    is_main = rank == 0
    init_logging(rank)
    cfg.validate()
    out_dir = Path(control.broadcast_object(str(cfg.output_dir)))
    cfg.output_dir = str(out_dir)
    if is_main:
        out_dir.mkdir(parents=True, exist_ok=True)
    control.wait_for_everyone()
    if cfg.seed is not None:
        set_seed(cfg.seed, rank)
    resume_step = None
    if cfg.resume and (out_dir / CHECKPOINTS_DIR / LAST_LINK / "training_step.json").exists():
        from ..utils.train_utils import load_training_step
        resume_step = load_training_step((out_dir / CHECKPOINTS_DIR / LAST_LINK).resolve())
    tracker_wb = WandBLogger(cfg, out_dir, is_main, resume_step)

    # ---- data
    res = make_dataset_mixture(cfg)
    train_mix, val_mix = res if isinstance(res, tuple) else (res, None)
    if is_main and val_mix is not None:
        warn_if_resumed_split_differs(out_dir, {d.repo_id: list(getattr(d.dataset, "episodes", []))
                                                for d in val_mix.datasets})
    micro_bs = cfg.dataloader_batch_size or cfg.batch_size
    ga = cfg.gradient_accumulation_steps
    loader = train_mix.get_dataloader(micro_bs, cfg.num_workers, rank, world, cfg.prefetch_factor)
    dl_iter = cycle(loader)

    # ---- model
    policy = make_policy(cfg.policy, ds_meta=train_mix.meta)
    policy.to(device)
    if device.type == "cuda":
        policy.to(torch.bfloat16)
    policy.train()
    if cfg.distributed.tp > 1:
        if cfg.distributed.tp != world or not hasattr(policy, "enable_tensor_parallel"):
            raise ValueError("distributed.tp must equal the number of ranks and needs a policy with a frozen, "
                             "shardable backbone (cosmos3)")
        from ..parallel.tp import TensorParallel
        policy.enable_tensor_parallel(TensorParallel(device), free_replicated_weights=True)
    opt_cfg, sched_cfg = cfg.optimizer, cfg.scheduler
    dcfg = cfg.distributed
    clip = dcfg.gradient_clipping if dcfg.gradient_clipping is not None else getattr(opt_cfg, "grad_clip_norm", 10.0)
    hyper = OptimHyper(lr=opt_cfg.lr, betas=tuple(getattr(opt_cfg, "betas", (0.9, 0.999))),
                       eps=getattr(opt_cfg, "eps", 1e-8), weight_decay=getattr(opt_cfg, "weight_decay", 0.0),
                       grad_clip_norm=clip)
    lr_lambda = sched_cfg.lr_lambda(cfg.steps) if sched_cfg is not None else None
    engine = make_engine(policy, hyper, device=device, lr_lambda=lr_lambda, loss_weights=cfg.loss_weighting,
                         strategy=getattr(dcfg, "strategy", "zero2"), comm=getattr(dcfg, "comm", "auto"),
                         grad_accum_steps=ga)
    n_params = sum(p.numel() for p in policy.parameters())
    n_train = sum(p.numel() for p in policy.parameters() if p.requires_grad)

    # ---- resume
    step = 0
    ckpt_root = out_dir / CHECKPOINTS_DIR
    if cfg.resume:
        last = ckpt_root / LAST_LINK
        if not last.exists():
            raise FileNotFoundError(f"resume requested but {last} does not exist")
        last = last.resolve()
        if not checkpoint_is_complete(last):      # against the world size recorded by the save
            raise RuntimeError(f"checkpoint {last} is incomplete (interrupted save)")
        from safetensors.torch import load_file
        sd = load_file(str(last / "model.safetensors"))
        import contextlib
        # a parameter-sharded engine holds slices: load into a temporary full copy and write the slices back
        with (engine.full_params(writeback=True) if hasattr(engine, "full_params") else contextlib.nullcontext()):
            missing, unexpected = policy.load_state_dict(type(policy)._fix_state_dict_keys(sd, cfg.policy),
                                                         strict=False)
        bad = [k for k in missing if "normalize" not in k]
        if bad:
            raise RuntimeError(f"checkpoint misses {len(bad)} tensors, e.g. {bad[:3]}")
        step = load_training_state(last, engine, rank, world, cfg.seed)
        engine.step_count = step
        logging.info("resumed from %s at step %d", last, step)

    # success rates are kept highest-first, losses lowest-first (reference scripts/train.py: higher_is_better is
    # true only for the eval-success metric); "auto" means success when an environment is evaluated in training
    resolved = getattr(cfg, "running_best_metric_resolved", None)
    best_on_success = resolved == "eval_success" if resolved is not None else (
        cfg.running_best_metric in ("success", "eval_success") or (
            cfg.running_best_metric == "auto" and cfg.env is not None and cfg.eval_freq > 0))
    best = RunningBestTracker(out_dir, cfg.running_best_count, cfg.running_best_metric,
                              higher_is_better=best_on_success) if cfg.running_best_count else None
    names = list(train_mix.meta.dataset_names)
    tot_w = float(sum(train_mix.weights)) or 1.0
    head_w: dict[str, float] = {}
    for n, w in zip(train_mix.names, train_mix.weights):
        key = names[train_mix.meta.dataset_to_norm_index[n]]
        head_w[key] = head_w.get(key, 0.0) + w / tot_w

    if is_main:
        logging.info("output dir: %s", out_dir)
        logging.info("steps=%s  global batch=%d (micro %d x accumulation %d x ranks %d)", format_big_number(cfg.steps),
                     micro_bs * ga * world, micro_bs, ga, world)
        logging.info("dataset frames=%s  params=%s (trainable %s)  strategy=%s comm=%s",
                     format_big_number(train_mix.num_frames), format_big_number(n_params), format_big_number(n_train),
                     engine.strategy, engine.comm)

    meters = {"loss": AverageMeter("loss", ":.3f"), "mse_loss": AverageMeter("mse", ":.3f"),
              "ce_loss": AverageMeter("ce", ":.3f"), "grad_norm": AverageMeter("grdn", ":.3f"),
              "lr": AverageMeter("lr", ":0.1e"), "update_s": AverageMeter("updt_s", ":.3f"),
              "dataloading_s": AverageMeter("data_s", ":.3f")}
    tracker = MetricsTracker(micro_bs * ga * world, train_mix.num_frames, None, meters, initial_step=step)
    final: dict[str, float] = {}

    # ---- hot loop
    while step < cfg.steps:
        t0 = time.perf_counter()
        batches = [to_device(next(dl_iter), device) for _ in range(ga)]
        tracker.dataloading_s = time.perf_counter() - t0
        t1 = time.perf_counter()
        out = update_policy(engine, batches)
        gathered = control.gather_scalars({"loss": out["loss"], "MSE": out.get("MSE", torch.zeros(())),
                                           "CE": out.get("CE", torch.zeros(())), "grad_norm": out["grad_norm"]},
                                          device=device)
        engine.check()      # the gather above synchronised: a peer-memory wait that gave up is fatal here, not later
        tracker.update_s = time.perf_counter() - t1
        step += 1
        tracker.step()
        tracker.loss = float(gathered["loss"].mean())
        tracker.mse_loss = float(gathered["MSE"].mean())
        tracker.ce_loss = float(gathered["CE"].mean())
        tracker.grad_norm = float(gathered["grad_norm"].mean())
        tracker.lr = engine.current_lr()
        if cfg.trace_nans and not all(map(lambda v: v == v, (tracker.loss.val, tracker.grad_norm.val))):
            raise FloatingPointError(f"NaN at step {step}: loss={tracker.loss.val} grad_norm={tracker.grad_norm.val}")
        final = {"loss": tracker.loss.val, "mse": tracker.mse_loss.val, "ce": tracker.ce_loss.val,
                 "grad_norm": tracker.grad_norm.val}

        is_log = cfg.log_freq > 0 and step % cfg.log_freq == 0
        is_save = cfg.save_checkpoint and (step % cfg.save_freq == 0 or step == cfg.steps)
        is_val = val_mix is not None and cfg.val_freq > 0 and step % cfg.val_freq == 0
        is_eval = cfg.env is not None and cfg.eval_freq > 0 and step % cfg.eval_freq == 0
        metrics: dict[str, float] = {}

        if is_log:
            if is_main:
                logging.info(str(tracker))
            d = tracker.to_dict()
            metrics.update({"Training/Loss": d["loss"], "Training/MSE Loss": d["mse_loss"], "Training/CE Loss": d["ce_loss"],
                            "Training/Learning Rate": d["lr"], "Training/Grad Norm": d["grad_norm"],
                            "Training/Num Samples": float(tracker.samples)})
            tracker.reset_averages()

        if is_val:
            # deterministic and complete: every validation sample once, strided over the ranks
            vloader = val_mix.get_combined_val_dataloader(micro_bs, cfg.num_workers, rank, world, cfg.prefetch_factor)
            vm = run_validation(policy, vloader, cfg.val_max_batches, device, names, head_w, cfg.loss_weighting,
                                dataset_names=list(val_mix.names)) if vloader is not None else {}
            metrics.update(vm)
            if is_main and vm:
                logging.info("validation @%d: loss %.4f (MSE %.4f, CE %.4f)", step, vm["Validation/Loss"],
                             vm["Validation/MSE Loss"], vm["Validation/CE Loss"])

        if is_eval:
            from .eval import collect_grid_summary_videos, eval_policy_on_config
            # fresh environments per evaluation, closed before training resumes (a simulator's render contexts hold
            # device memory that the caching allocator cannot give back); grid videos and the consolidated
            # eval_info.json land under <output_dir>/eval/videos_step_<id>
            step_id = get_step_checkpoint_dir(out_dir, cfg.steps, step).name
            videos_dir = out_dir / "eval" / f"videos_step_{step_id}"
            t_eval = time.perf_counter()
            try:
                info = eval_policy_on_config(policy, cfg, device, rank=rank, world=world, videos_dir=videos_dir)
            finally:
                policy.reset()                  # per-evaluation observation / action queues must not reach training
            metrics["Success Rate"] = info["aggregated"]["pc_success"]
            metrics["Evaluation Time"] = time.perf_counter() - t_eval
            for g, v in info.get("per_group", {}).items():
                metrics[f"Success/{g}"] = v["pc_success"]
            if is_main:
                videos_dir.mkdir(parents=True, exist_ok=True)
                (videos_dir / "eval_info.json").write_text(json.dumps(info, indent=2, default=str))
                tracker_wb.log_videos({f"Eval Videos/{task}": path for task, path in collect_grid_summary_videos(videos_dir)},
                                  step, enabled=not cfg.wandb.disable_video and cfg.eval.max_episodes_rendered > 0)
            control.wait_for_everyone()

        if is_save:
            control.wait_for_everyone()
            ckpt = get_step_checkpoint_dir(out_dir, cfg.steps, step)
            save_checkpoint(ckpt, step, cfg, policy, engine, rank=rank, is_main=is_main)
            control.wait_for_everyone()
            if is_main:
                if not checkpoint_is_complete(ckpt, world):
                    raise RuntimeError(f"checkpoint {ckpt} is incomplete after the save barrier")
                update_last_checkpoint(ckpt)
                keep = {ckpt.name}
                if best is not None:
                    keep |= best.kept
                if cfg.last_checkpoint_only:
                    prune_checkpoints(out_dir, keep)
                logging.info("checkpoint saved: %s", ckpt)

        if best is not None and (is_val or is_eval) and metrics:
            key = "Success Rate" if best_on_success else "Validation/Loss"
            if key in metrics:
                # rank 0 decides BEFORE anything is written and every rank follows the broadcast decision: a rank
                # that looked at the directory instead would skip its own shard once rank 0 had created it
                decision = None
                if is_main:
                    ckpt0 = get_step_checkpoint_dir(out_dir, cfg.steps, step)
                    decision = (bool(best.would_keep(metrics[key])), not (is_save and ckpt0.exists()))
                keep_it, need_save = control.broadcast_object(decision)
                if keep_it:
                    sid = get_step_identifier(step, cfg.steps)
                    ckpt = get_step_checkpoint_dir(out_dir, cfg.steps, step)
                    if need_save:
                        save_checkpoint(ckpt, step, cfg, policy, engine, rank=rank, is_main=is_main)
                    control.wait_for_everyone()
                    if is_main:
                        if not checkpoint_is_complete(ckpt, world):
                            raise RuntimeError(f"running-best checkpoint {ckpt} is incomplete after the save barrier")
                        best.update(sid, metrics[key])
                        if cfg.last_checkpoint_only:
                            last_name = (ckpt_root / LAST_LINK).resolve().name if (ckpt_root / LAST_LINK).exists() else ""
                            prune_checkpoints(out_dir, best.kept | {last_name})

        if metrics and is_main:
            tracker_wb.log(metrics, step)

    control.wait_for_everyone()
    tracker_wb.finish()
    if is_main:
        logging.info("End of training")
    return final


@parser.wrap()
def train_main(cfg: TrainPipelineConfig):
    return train(cfg)


def main() -> None:
    train_main()
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
