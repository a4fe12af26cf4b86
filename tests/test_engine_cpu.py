"""Training engine: flat store, fused-AdamW numerics vs torch.optim, and 2-rank gloo sharded steps."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import tiny_batch, tiny_pi05, free_port
from opentau_b200.parallel.engine import OptimHyper, TrainEngine, assemble_weighted_loss


def test_assemble_weighted_loss_order_and_zero_weight_drop():
    l = {"MSE": torch.tensor(2.0, requires_grad=True), "CE": torch.tensor(3.0, requires_grad=True)}
    assert assemble_weighted_loss(l, {"MSE": 1.0, "CE": 0.5}).item() == pytest.approx(3.5)
    t = assemble_weighted_loss(l, {"MSE": 1.0, "CE": 0.0})
    t.backward()
    assert l["CE"].grad is None
    with pytest.raises(ValueError):
        assemble_weighted_loss(l, {"MSE": 0.0, "CE": 0.0})


def test_flat_store_views_and_main_grad():
    pol = tiny_pi05()
    before = {n: p.detach().clone() for n, p in pol.named_parameters()}
    eng = TrainEngine(pol, OptimHyper(), device="cpu")
    for n, p in pol.named_parameters():
        assert torch.equal(p.detach(), before[n])
        if p.requires_grad:
            assert p.main_grad.shape == p.shape
    g = eng.store.groups[0]
    p0 = g.params[0]
    p0.data.fill_(1.5)
    assert g.data[g.offsets[0]].item() == 1.5


def test_engine_step_matches_torch_adamw():
    torch.manual_seed(0)
    pol_a, pol_b = tiny_pi05(seed=3), tiny_pi05(seed=3)
    hyper = OptimHyper(lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01, grad_clip_norm=1.0)
    eng = TrainEngine(pol_a, hyper, device="cpu")
    params_b = [p for p in pol_b.parameters() if p.requires_grad]
    opt = torch.optim.AdamW(params_b, lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01)
    b = tiny_batch()
    noise, time = torch.randn(4, 10, 32), torch.full((4,), 0.6)
    for _ in range(2):
        out = pol_a(b, noise=noise, time=time)
        (out["MSE"] + out["CE"]).backward()
        norm_a = eng.optimizer_step()
        out_b = pol_b(b, noise=noise, time=time)
        (out_b["MSE"] + out_b["CE"]).backward()
        norm_b = torch.nn.utils.clip_grad_norm_(params_b, 1.0)
        opt.step()
        opt.zero_grad()
        torch.testing.assert_close(norm_a, norm_b, rtol=1e-4, atol=1e-6)
    for (n, pa), (_, pb) in zip(pol_a.named_parameters(), pol_b.named_parameters()):
        torch.testing.assert_close(pa, pb, rtol=1e-4, atol=1e-6, msg=lambda m, n=n: f"{n}: {m}")


def test_lr_schedule_is_applied():
    pol = tiny_pi05()
    from opentau_b200.optim.schedulers import CosineDecayWithWarmupSchedulerConfig
    sch = CosineDecayWithWarmupSchedulerConfig(num_warmup_steps=10, num_decay_steps=100, peak_lr=1e-3, decay_lr=1e-4)
    eng = TrainEngine(pol, OptimHyper(lr=1e-3), device="cpu", lr_lambda=sch.lr_lambda(100))
    assert eng.current_lr() == pytest.approx(1e-3 / 11)
    eng.train_step(tiny_batch())
    assert eng.current_lr() == pytest.approx(1e-3 * ((1 / 11 - 1) * (1 - 1 / 10) + 1))


def _rank_main(rank, world, port, strategy, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        pol = tiny_pi05(seed=10 + rank)      # different inits: rank 0 must win
        # small buckets: the tiny model then has several, each sliced over the two ranks
        eng = TrainEngine(pol, OptimHyper(lr=1e-3, grad_clip_norm=1.0), device="cpu", strategy=strategy,
                          bucket_elems=200_000)
        assert len(eng.store.buckets) > 3
        full = tiny_batch(batch_size=4, seed=5)
        half = {k: v[rank * 2:(rank + 1) * 2] for k, v in full.items()}
        noise, time = torch.randn(4, 10, 32, generator=torch.Generator().manual_seed(1)), torch.full((4,), 0.5)
        for _ in range(2):
            out = pol(half, noise=noise[rank * 2:(rank + 1) * 2], time=time[rank * 2:(rank + 1) * 2])
            (out["MSE"] + out["CE"]).backward()
            norm = eng.optimizer_step()
        flat = eng.store.groups[0].data.clone()
        gathered = [torch.empty_like(flat) for _ in range(world)]
        dist.all_gather(gathered, flat)
        if rank == 0:
            ret["same"] = bool(all(torch.equal(gathered[0], g) for g in gathered))
            ret["norm"] = float(norm)
            ret["named"] = {n: p.detach().clone() for n, p in pol.named_parameters() if p.requires_grad}
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("strategy", ["zero2", "ddp"])
def test_two_rank_gloo_step_keeps_replicas_identical_and_matches_single_rank(strategy):
    port = free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main, args=(2, port, strategy, ret), nprocs=2, join=True)
    assert ret["same"]
    # single-rank run on the full batch with mean-of-halves loss == DP run
    pol = tiny_pi05(seed=10)
    eng = TrainEngine(pol, OptimHyper(lr=1e-3, grad_clip_norm=1.0), device="cpu")
    full = tiny_batch(batch_size=4, seed=5)
    noise, time = torch.randn(4, 10, 32, generator=torch.Generator().manual_seed(1)), torch.full((4,), 0.5)
    for _ in range(2):
        tot = 0
        for r in range(2):
            half = {k: v[r * 2:(r + 1) * 2] for k, v in full.items()}
            out = pol(half, noise=noise[r * 2:(r + 1) * 2], time=time[r * 2:(r + 1) * 2])
            ((out["MSE"] + out["CE"]) / 2).backward()
        norm = eng.optimizer_step()
    assert float(norm) == pytest.approx(ret["norm"], rel=1e-4)
    # compared by name: bucket boundaries (and so the offsets inside the flat buffer) depend on the world size
    for n, p in pol.named_parameters():
        if p.requires_grad:
            torch.testing.assert_close(p.detach(), ret["named"][n], rtol=1e-4, atol=1e-6, msg=n)


def _fsdp_rank(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from helpers import TINY
        from opentau_b200.parallel.fsdp import ShardedParamEngine, make_engine
        deep = dict(vlm=dict(TINY["vlm"], num_hidden_layers=3), expert=dict(TINY["expert"], num_hidden_layers=3))
        res = {}
        for strat in ("zero2", "fsdp"):
            pol = tiny_pi05(seed=10 + rank, **deep).train()
            eng = make_engine(pol, OptimHyper(lr=1e-3, grad_clip_norm=1.0), device="cpu", strategy=strat)
            batch = tiny_batch(batch_size=2, seed=5 + rank)
            g = torch.Generator().manual_seed(1 + rank)
            noise, time = torch.randn(2, 10, 32, generator=g), torch.full((2,), 0.5)
            norms = []
            for _ in range(3):
                out = pol(batch, noise=noise, time=time)
                (out["MSE"] + out["CE"]).backward()
                norms.append(float(eng.optimizer_step()))
            if strat == "fsdp":
                assert isinstance(eng, ShardedParamEngine) and eng.store.groups[0].data is None
                # three layers share two slots per tower.  Per step: the root unit once, every layer for its forward
                # (3 + 3), and for the backward only layer 0 of each tower (its slot was taken by layer 2; layers 2
                # and 1 are still resident when the backward pass reaches them)
                per_step = (eng._gathers - 1) / 3
                assert per_step == 1 + 6 + 2, per_step
                rest = sum(p.numel() for p in eng.pshard)
                assert rest * world == sum(g_.numel for g_ in eng.store.groups)
                with eng.full_params():
                    named = {k: p.detach().clone() for k, p in pol.named_parameters() if p.requires_grad}
                sd = eng.state_dict()
                eng.load_state_dict(sd)
                # a state dict loaded into a fresh sharded engine lands in the shards
                pol2 = tiny_pi05(seed=99, **deep).train()
                eng2 = make_engine(pol2, OptimHyper(lr=1e-3, grad_clip_norm=1.0), device="cpu", strategy="fsdp")
                with eng.full_params():
                    full_sd = {k: v.clone() for k, v in pol.state_dict().items()}
                with eng2.full_params(writeback=True):
                    pol2.load_state_dict(full_sd)
                eng2.rebuild_masters_from_live()
                assert abs(float(eng2.param_checksum()) - float(eng.param_checksum())) < 1e-6
                o1, o2 = pol(batch, noise=noise, time=time), pol2(batch, noise=noise, time=time)
                assert abs(float(o1["MSE"]) - float(o2["MSE"])) < 1e-6
            else:
                named = {k: p.detach().clone() for k, p in pol.named_parameters() if p.requires_grad}
            res[strat] = (norms, named)
        (na, pa), (nb, pb) = res["zero2"], res["fsdp"]
        worst = max(float((pa[k] - pb[k]).abs().max()) for k in pa)
        gathered = [None] * world
        dist.all_gather_object(gathered, (max(abs(x - y) for x, y in zip(na, nb)), worst))
        if rank == 0:
            ret["fsdp"] = gathered
    finally:
        dist.destroy_process_group()


def test_parameter_sharded_engine_matches_zero2_on_two_ranks():
    """``strategy=fsdp``: parameters live as 1 / W slices, layers are gathered into rotating slots before their
    forward and backward; three steps give the same gradient norms and parameters as ZeRO-2, and a full state dict
    can be exported from and loaded into the shards."""
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_fsdp_rank, args=(2, free_port(), ret), nprocs=2, join=True)
    for dn, dp in ret["fsdp"]:
        assert dn < 1e-4 and dp < 1e-5


def test_parameter_sharding_strategies_are_not_silently_replicated():
    import pytest as _pt
    with _pt.raises(ValueError, match="shards the PARAMETERS"):
        TrainEngine(tiny_pi05(), OptimHyper(), device="cpu", strategy="fsdp")
