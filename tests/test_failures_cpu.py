"""Failure handling, injected on the host only: interrupted or damaged checkpoints, a changed world size on resume, a
rank that leaves before a collective, and ranks that disagree on a branch decision.  Nothing here touches a GPU."""

import datetime
import json
import os

import pytest
from helpers import free_port
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from test_train_cpu import _cfg
from opentau_b200.scripts.train import train
from opentau_b200.utils.train_utils import checkpoint_is_complete, load_training_state


def _trained(tmp_path):
    out = tmp_path / "run"
    train(_cfg(out, 4))
    return out, (out / "checkpoints" / "last").resolve()


def test_interrupted_save_is_detected_and_resume_refuses(tmp_path):
    out, ck = _trained(tmp_path)
    assert checkpoint_is_complete(ck, 1) and not checkpoint_is_complete(ck, 2)      # one marker per rank is required
    (ck / "random_states_0.marker").unlink()                                        # the save died before its marker
    assert not checkpoint_is_complete(ck, 1)
    with pytest.raises(RuntimeError, match="incomplete"):
        train(_cfg(out, 6, resume=True))


def test_damaged_optimizer_shard_raises_instead_of_training_on(tmp_path):
    out, ck = _trained(tmp_path)
    shard = ck / "optimizer_rank0.safetensors"
    shard.write_bytes(shard.read_bytes()[: shard.stat().st_size // 3])              # truncated file
    with pytest.raises(Exception) as e:
        train(_cfg(out, 6, resume=True))
    assert "safetensor" in str(e.value).lower() or "header" in str(e.value).lower() or "deserializ" in str(e.value).lower()


def test_resume_on_another_world_size_rebuilds_masters(tmp_path):
    out, ck = _trained(tmp_path)
    # pretend the checkpoint came from two ranks: this rank's shard layout no longer matches
    (ck / "optimizer_rank1.safetensors").write_bytes((ck / "optimizer_rank0.safetensors").read_bytes())
    (ck / "random_states_1.marker").write_text("4")

    class Engine:
        step_count, rebuilt = 0, 0

        def rebuild_masters_from_live(self):
            self.rebuilt += 1

        def load_state_dict(self, sd):
            raise AssertionError("shards of another world size must not be loaded")

    eng = Engine()
    step = load_training_state(ck, eng, rank=0, world_size=1, seed=3)
    assert step == 4 and eng.step_count == 4 and eng.rebuilt == 1


def _leaver(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    t = torch.ones(4)
    dist.all_reduce(t)                           # a healthy step first
    if rank == 1:
        os._exit(0)                              # leaves between steps, nothing of its own in flight
    try:
        dist.all_reduce(t)
        ret["outcome"] = "completed"
    except Exception as e:  # noqa: BLE001
        ret["outcome"] = type(e).__name__
    os._exit(0)                                  # the group cannot be torn down cleanly any more


def test_surviving_rank_gets_an_error_not_a_hang():
    mgr = mp.Manager()
    ret = mgr.dict()
    ctx = mp.spawn(_leaver, args=(2, free_port(), ret), nprocs=2, join=False)
    for p in ctx.processes:
        p.join(timeout=60)
        assert not p.is_alive(), "a rank is still waiting for the one that left"
    assert ret.get("outcome") not in (None, "completed")


def _disagree(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        from opentau_b200.parallel import control
        # rank 1 alone has the optional input; the decision that guards a collective is OR-reduced first, so both
        # ranks take the same branch and the collective inside it is entered by everyone
        mine = [rank == 1, False]
        agreed = control.any_rank(mine)
        entered = 0
        if agreed[0]:
            dist.all_reduce(torch.ones(1))
            entered = 1
        ret[rank] = (agreed, entered, control.all_ranks_agree(("layout", 3)), control.all_ranks_agree(rank))
    finally:
        dist.destroy_process_group()


def test_branch_decisions_are_made_uniform_before_collectives():
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_disagree, args=(2, free_port(), ret), nprocs=2, join=True)
    assert ret[0] == ret[1] == ([True, False], 1, True, False)


def test_metrics_file_survives_a_crash_between_steps(tmp_path):
    """Every logged step is a complete JSON line: a run killed later leaves a readable history."""
    out, _ = _trained(tmp_path)
    lines = (out / "metrics.jsonl").read_text().splitlines()
    assert lines and all(json.loads(x)["step"] for x in lines)


def _rng_rank(rank, world, port, ckdir, q):
    import os
    import torch
    import torch.distributed as dist
    from pathlib import Path
    from opentau_b200.utils.random_utils import load_rng_state, save_rng_state, set_seed
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    set_seed(11, rank)
    torch.rand(3)                                   # advance the stream a little
    save_rng_state(Path(ckdir), rank)
    expected = torch.rand(4)                        # what the uninterrupted run would draw next
    dist.barrier()
    set_seed(999, 0)                                # a restarted process: every rank starts from the same state
    load_rng_state(Path(ckdir), rank)
    q.put((rank, expected.tolist(), torch.rand(4).tolist()))
    dist.destroy_process_group()


def test_every_rank_resumes_its_own_rng_stream(tmp_path):
    """After a resume the ranks must not share one stream (identical noise / time draws on every rank) and each
    must continue exactly where it stopped."""
    import torch.multiprocessing as mp
    from helpers import free_port
    ctx = mp.get_context("spawn")
    q, port = ctx.Queue(), free_port()
    procs = [ctx.Process(target=_rng_rank, args=(r, 2, port, str(tmp_path), q)) for r in range(2)]
    [p.start() for p in procs]
    got = sorted(q.get(timeout=120) for _ in procs)
    [p.join(30) for p in procs]
    assert got[0][1] == got[0][2] and got[1][1] == got[1][2]      # each rank continues its own stream
    assert got[0][2] != got[1][2]                                  # and the two streams differ
    assert (tmp_path / "rng_state_rank0.safetensors").exists() and (tmp_path / "rng_state_rank1.safetensors").exists()
