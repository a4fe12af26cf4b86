"""Context-parallel attention on two gloo ranks (library data path): forward and gradients equal the unsharded op."""

import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import free_port

from opentau_b200 import ops


def _inputs():
    torch.manual_seed(0)
    B, S, H, Hkv, D = 2, 12, 4, 2, 16
    q, k, v = torch.randn(B, S, H, D), torch.randn(B, S, Hkv, D), torch.randn(B, S, Hkv, D)
    blk = torch.tensor([0, 0, 0, 0, 1, 1, 2, 3, 3, 4, 5, 6], dtype=torch.int32)[None].expand(B, S).contiguous()
    valid = torch.ones(B, S, dtype=torch.bool)
    valid[1, 5] = False
    do = torch.randn(B, S, H * D)
    return q, k, v, blk, valid, do


def _rank_main(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from opentau_b200.parallel.cp import ContextParallel
        q, k, v, blk, valid, do = _inputs()
        qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
        want = ops.block_attention(qr, kr, vr, blk, blk, valid, valid, 0.25)
        want.backward(do)
        cp = ContextParallel("cpu")
        ql, kl, vl = (cp.shard(t).clone().requires_grad_(True) for t in (q, k, v))
        got = cp.attention(ql, kl, vl, cp.shard(blk).contiguous(), blk, cp.shard(valid).contiguous(), valid, 0.25)
        got.backward(cp.shard(do).contiguous())
        errs = [float((got - cp.shard(want)).abs().max()), float((ql.grad - cp.shard(qr.grad)).abs().max()),
                float((kl.grad - cp.shard(kr.grad)).abs().max()), float((vl.grad - cp.shard(vr.grad)).abs().max())]
        gathered = [None] * world
        dist.all_gather_object(gathered, errs)
        if rank == 0:
            ret["err"] = max(max(e) for e in gathered)
    finally:
        dist.destroy_process_group()


def test_context_parallel_attention_matches_unsharded_on_two_ranks():
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main, args=(2, free_port(), ret), nprocs=2, join=True)
    assert ret["err"] < 1e-5


def _policy_rank(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from helpers import tiny_batch, tiny_pi05
        from opentau_b200.parallel.cp import ContextParallel
        batch = tiny_batch(batch_size=2, seed=50 + rank)          # every rank has its own samples
        g = torch.Generator().manual_seed(3 + rank)
        noise, time = torch.randn(2, 10, 32, generator=g), torch.full((2,), 0.4)
        results = []
        for use_cp in (False, True):
            pol = tiny_pi05(seed=7).train()
            if use_cp:
                pol.model.context_parallel = ContextParallel("cpu")
            out = pol(batch, noise=noise, time=time)
            (out["MSE"] + out["CE"]).backward()
            grads = {}
            for n, p in pol.named_parameters():
                if p.requires_grad and p.grad is not None:
                    gsum = p.grad.clone()
                    dist.all_reduce(gsum)                          # what the data-parallel step would apply
                    grads[n] = gsum
            results.append((float(out["MSE"]), float(out["CE"]), grads))
        (m0, c0, g0), (m1, c1, g1) = results
        worst = max(float((g0[n] - g1[n]).abs().max()) / (float(g0[n].abs().max()) + 1e-6) for n in g0)
        gathered = [None] * world
        dist.all_gather_object(gathered, (abs(m0 - m1), abs(c0 - c1), worst, set(g0) == set(g1)))
        if rank == 0:
            ret["policy"] = gathered
    finally:
        dist.destroy_process_group()


def test_policy_loss_and_gradients_are_unchanged_by_context_parallelism():
    """pi0.5 (knowledge insulation + FAST tokens) with the prefix split over two ranks: each rank's losses equal
    those of the unsharded pass on its samples, and the rank-summed gradients of every parameter agree."""
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_policy_rank, args=(2, free_port(), ret), nprocs=2, join=True)
    for dm, dc, worst, same_keys in ret["policy"]:
        assert dm < 1e-5 and dc < 1e-5 and worst < 1e-3 and same_keys
