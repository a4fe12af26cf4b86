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
