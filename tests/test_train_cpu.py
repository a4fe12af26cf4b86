"""The training script end to end on CPU with a tiny pi0.5 and the synthetic dataset: loss goes down, metrics are
logged, checkpoints are written / pruned, validation runs, and a resumed run continues from the saved step."""

import json

import torch

from helpers import TINY
from opentau_b200.configs.train import TrainPipelineConfig
from opentau_b200.scripts.train import bucket_per_sample, mixture_weighted_aggregate, train


def _cfg(out, steps, resume=False, **kw):
    raw = {
        "dataset_mixture": {"datasets": [{"synthetic": {"length": 64, "state_dim": 6, "action_dim": 6, "name": "a"}}],
                            "action_freq": 10.0, "val_split_ratio": 0.25},
        "policy": {"type": "pi05", "chunk_size": 10, "n_action_steps": 10, "prompt_max_length": 24,
                   "discrete_action_max_length": 8, "discrete_action_vocab_size": 256, "dropout": 0.0, "device": "cpu",
                   "optimizer_lr": 2e-3, "scheduler_warmup_steps": 2, "scheduler_decay_steps": 50, **TINY},
        "output_dir": str(out), "resume": resume, "seed": 3, "resolution": [224, 224], "num_cams": 1, "action_chunk": 10,
        "batch_size": 4, "steps": steps, "log_freq": 2, "save_freq": 4, "val_freq": 4, "num_workers": 0,
        "use_policy_training_preset": True, **kw}
    return TrainPipelineConfig.from_dict(raw)


def test_train_checkpoint_resume(tmp_path):
    out = tmp_path / "run"
    torch.manual_seed(0)
    first = train(_cfg(out, 8))
    assert first["loss"] == first["loss"] and first["grad_norm"] > 0
    rows = [json.loads(line) for line in (out / "metrics.jsonl").read_text().splitlines()]
    assert [r["step"] for r in rows] == [2, 4, 6, 8]
    assert "Training/Loss" in rows[0] and "Validation/Loss" in rows[1] and "Validation/synthetic:a/MSE Loss" in rows[1]
    assert rows[-1]["Training/Loss"] < rows[0]["Training/Loss"]
    ck = out / "checkpoints"
    assert (ck / "last").resolve().name == "000008" and not (ck / "000004").exists()     # pruned to the last one
    for f in ("model.safetensors", "config.json", "train_config.json", "training_step.json", "optimizer_rank0.safetensors"):
        assert (ck / "000008" / f).exists(), f
    # the per-rank shards + layout consolidate into named fp32 masters that round to the saved bf16 / fp32 weights
    from safetensors.torch import load_file
    from opentau_b200.scripts.zero_to_fp32 import consolidate
    full = consolidate(ck / "000008", moments=True)
    saved = load_file(str(ck / "000008" / "model.safetensors"))
    name = next(k for k in saved if k.endswith("action_in_proj.weight"))
    assert full[name].dtype == torch.float32 and full[name].shape == saved[name].shape
    torch.testing.assert_close(full[name].to(saved[name].dtype), saved[name])
    assert full[name + ".exp_avg_sq"].min() >= 0 and (ck / "000008" / "flat_layout.json").exists()
    resumed = train(_cfg(out, 10, resume=True))
    rows = [json.loads(line) for line in (out / "metrics.jsonl").read_text().splitlines()]
    assert rows[-1]["step"] == 10 and (ck / "last").resolve().name == "000010"
    assert resumed["loss"] < rows[0]["Training/Loss"]


def test_validation_buckets_are_exact_masked_means():
    ps = {"MSE_sum": torch.tensor([2.0, 4.0, 9.0]), "MSE_count": torch.tensor([1.0, 3.0, 3.0]),
          "CE_sum": torch.tensor([0.0, 6.0, 3.0]), "CE_count": torch.tensor([0.0, 2.0, 1.0])}
    b = bucket_per_sample(ps, torch.tensor([0, 0, 1]), ["a", "b"])
    assert b["a"]["MSE"] == 6.0 / 4.0 and b["a"]["CE"] == 3.0 and b["b"]["MSE"] == 3.0 and b["b"]["n"] == 1.0
    agg = mixture_weighted_aggregate(b, {"a": 0.75, "b": 0.25})
    assert abs(agg["MSE"] - (0.75 * 1.5 + 0.25 * 3.0)) < 1e-9


def test_train_on_a_recorded_lerobot_dataset(tmp_path):
    """Raw LeRobot feature names / widths flow into the normalisation heads through the mixture metadata."""
    from test_datasets_cpu import _record
    _record(tmp_path / "toy", episodes=(12, 12))
    raw = {
        "dataset_mixture": {"datasets": [{"repo_id": "local/toy", "root": str(tmp_path / "toy")}], "action_freq": 10.0},
        "policy": {"type": "pi05", "chunk_size": 10, "n_action_steps": 10, "prompt_max_length": 32,
                   "discrete_action_max_length": 8, "discrete_action_vocab_size": 256, "dropout": 0.0, "device": "cpu", **TINY},
        "output_dir": str(tmp_path / "run"), "seed": 1, "resolution": [224, 224], "num_cams": 1, "action_chunk": 10,
        "batch_size": 2, "steps": 2, "log_freq": 1, "save_checkpoint": False, "num_workers": 0,
        "use_policy_training_preset": True}
    out = train(TrainPipelineConfig.from_dict(raw))
    assert out["loss"] == out["loss"] and out["grad_norm"] > 0


def test_running_best_checkpoints_are_kept_and_complete(tmp_path):
    """Periodic saves with a running-best tracker: the best validation steps survive pruning next to the last one,
    every kept checkpoint carries its rank marker and optimizer shard, and the tracker orders losses lowest-first."""
    from opentau_b200.utils.train_utils import RunningBestTracker, checkpoint_is_complete
    out = tmp_path / "run"
    torch.manual_seed(0)
    train(_cfg(out, 8, running_best_count=1))
    ck = out / "checkpoints"
    best = json.loads((ck / "running_best.json").read_text())
    assert best["higher_is_better"] is False and len(best["entries"]) == 1
    kept = ck / best["entries"][0]["step"]
    assert kept.is_dir() and checkpoint_is_complete(kept, 1) and (kept / "optimizer_rank0.safetensors").exists()
    assert (kept / "rng_state_rank0.safetensors").exists()
    assert (ck / "last").resolve().name == "000008"
    # a success-rate tracker keeps the HIGHEST values
    t = RunningBestTracker(tmp_path / "t", 2, "eval_success", higher_is_better=True)
    for sid, v in (("a", 0.2), ("b", 0.9), ("c", 0.5)):
        if t.would_keep(v):
            t.update(sid, v)
    assert t.kept == {"b", "c"}


def test_train_and_resume_with_sharded_parameters(tmp_path):
    """``distributed.strategy = fsdp`` through the trainer: the checkpoint holds full weights (gathered for the
    export), and a resumed run loads them back into the shards and continues."""
    from safetensors.torch import load_file
    out = tmp_path / "run"
    torch.manual_seed(0)
    first = train(_cfg(out, 4, distributed={"strategy": "fsdp"}, val_freq=0))
    assert first["loss"] == first["loss"]
    saved = load_file(str(out / "checkpoints" / "000004" / "model.safetensors"))
    name = next(k for k in saved if k.endswith("layers.1.mlp.down_proj.weight"))
    assert saved[name].abs().sum() > 0
    resumed = train(_cfg(out, 6, resume=True, distributed={"strategy": "fsdp"}, val_freq=0))
    rows = [json.loads(line) for line in (out / "metrics.jsonl").read_text().splitlines()]
    assert rows[-1]["step"] == 6 and resumed["loss"] < rows[0]["Training/Loss"] * 1.5


def test_validation_pass_is_complete_and_split_by_head_and_dataset(tmp_path):
    """Two synthetic members under different heads: every validation sample is scored once, per head and per
    dataset, and the headline is weighted like the training mixture."""
    from opentau_b200.datasets.factory import make_dataset_mixture
    from opentau_b200.policies.factory import make_policy
    from opentau_b200.scripts.train import run_validation
    cfg = _cfg(tmp_path / "o", 1)
    cfg.dataset_mixture.datasets.append(type(cfg.dataset_mixture.datasets[0])(
        synthetic={"length": 40, "state_dim": 6, "action_dim": 6, "name": "b"}))
    cfg.dataset_mixture.weights = [3.0, 1.0]
    train_mix, val_mix = make_dataset_mixture(cfg)
    assert len(val_mix) == 16 + 10
    shards = [val_mix.get_combined_val_dataloader(4, rank=r, world=3).dataset for r in range(3)]
    seen = sorted((s[i]["source"], int(s[i]["frame_index"]) + 100 * int(s[i]["episode_index"]))
                  for s in shards for i in range(len(s)))
    assert len(seen) == 26 and len(set(seen)) == 26                       # a partition: nothing twice, nothing lost
    assert sorted(val_mix.get_per_dataset_dataloaders(4)) == sorted(val_mix.names)
    policy = make_policy(cfg.policy, ds_meta=train_mix.meta)
    names = list(train_mix.meta.dataset_names)
    weights = {names[train_mix.meta.dataset_to_norm_index[n]]: w / 4.0 for n, w in zip(train_mix.names, train_mix.weights)}
    loader = val_mix.get_combined_val_dataloader(4)
    m = run_validation(policy, loader, None, torch.device("cpu"), names, weights, {"MSE": 1.0, "CE": 1.0},
                       dataset_names=list(val_mix.names))
    assert m["Validation/Num Samples"] == 26.0
    for n in names:
        assert f"Validation/{n}/Loss" in m
    for n in val_mix.names:
        assert f"Validation/by_dataset/{n}/MSE Loss" in m
    expect = sum(weights[n] * m[f"Validation/{n}/MSE Loss"] for n in names)
    assert abs(m["Validation/MSE Loss"] - expect) < 1e-6
    capped = run_validation(policy, loader, 2, torch.device("cpu"), names, weights, {"MSE": 1.0, "CE": 1.0})
    assert capped["Validation/Num Samples"] == 8.0 and not any("by_dataset" in k for k in capped)
    assert policy.training                                                  # the mode it came in with is restored
    agg = train_mix.meta.aggregated_action_stats([3.0, 1.0])
    assert agg["mean"].shape == (32,)


def _ragged_rank(rank, world, port, ret):
    import os

    import torch.distributed as dist

    from opentau_b200.parallel import control
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n = 3 if rank == 0 else 1
    out = control.gather_ragged({"a": torch.arange(n, dtype=torch.float32) + 10 * rank,
                                 "b": torch.full((n, 2), rank, dtype=torch.long)})
    ret[rank] = (out["a"].tolist(), out["b"][:, 0].tolist())
    dist.destroy_process_group()


def test_ragged_gather_keeps_rows_aligned_across_ranks():
    import torch.multiprocessing as mp

    from helpers import free_port
    ret = mp.Manager().dict()
    mp.spawn(_ragged_rank, args=(2, free_port(), ret), nprocs=2, join=True)
    assert ret[0] == ret[1] == ([0.0, 1.0, 2.0, 10.0], [0, 0, 0, 1])


def test_in_training_evaluation_writes_videos_and_info(tmp_path):
    """``eval_freq`` with an environment: fresh environments per evaluation, success metrics in the log, the grid video
    and the consolidated eval_info.json under <output_dir>/eval/videos_step_<id>."""
    out = tmp_path / "run"
    cfg = _cfg(out, 2, val_freq=0, eval_freq=2, save_freq=100,
               env={"type": "fake", "state_dim": 12, "action_dim": 6, "resolution": [224, 224], "episode_length": 6},
               eval={"n_episodes": 2, "batch_size": 2, "max_episodes_rendered": 2, "use_async_envs": False})
    train(cfg)
    rows = [json.loads(line) for line in (out / "metrics.jsonl").read_text().splitlines()]
    last = next(r for r in reversed(rows) if "Success Rate" in r)
    assert last["step"] == 2 and "Evaluation Time" in last and any(k.startswith("Success/") for k in last)
    vdir = out / "eval" / "videos_step_000002"
    info = json.loads((vdir / "eval_info.json").read_text())
    assert info["aggregated"]["n"] == 2
    grids = list(vdir.rglob("grid_summary.mp4"))
    assert len(grids) == 1
    noted = [r for r in rows if "videos" in r]
    assert noted and list(noted[-1]["videos"].values())[0].endswith("grid_summary.mp4")
