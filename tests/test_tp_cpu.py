"""Tensor-parallel decoder layer on two gloo ranks (library data path): same result as the unsharded layer."""

import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from opentau_b200 import ops
from opentau_b200.models.layers import DecoderLayer, TowerConfig
from helpers import free_port

CFG = dict(hidden_size=128, num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
           intermediate_size=256, vocab_size=64, hidden_act="silu", qk_norm=True, norm_unit_offset=False)


def _full_layer(layer, x, pos, blk, valid):
    """Unsharded forward of one decoder layer on ``x [B,S,d]``."""
    cfg = layer.cfg
    h = layer.input_layernorm(x)[0]
    q, k, v = layer.self_attn.qkv(h)
    cs = ops.rope_angles(pos, cfg.head_dim, cfg.rope_theta)
    q, k = ops.rope(q, *cs), ops.rope(k, *cs)
    att = ops.block_attention(q, k, v, blk, blk, valid, valid, cfg.attn_scale)
    y = layer.self_attn.o_proj(att, residual=x)
    return layer.mlp(layer.post_attention_layernorm(y)[0], residual=y)


def _rank_main(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from opentau_b200.parallel.tp import TensorParallel, TPDecoderLayer
        torch.manual_seed(0)
        layer = DecoderLayer(TowerConfig(**CFG), 0)
        B, S, d = 4, 6, 128
        x = torch.randn(B, S, d)
        pos = torch.arange(S)[None].expand(B, S)
        blk = torch.tensor([0, 0, 0, 1, 2, 3], dtype=torch.int32)[None].expand(B, S).contiguous()
        valid = torch.ones(B, S, dtype=torch.bool)
        valid[1, 2] = False
        want = _full_layer(layer, x, pos, blk, valid)
        tp = TensorParallel("cpu")
        tpl = TPDecoderLayer(layer, tp)
        Ml = B * S // world
        x_local = x.view(B * S, d)[rank * Ml:(rank + 1) * Ml]
        cs = ops.rope_angles(pos, CFG["head_dim"], 10000.0)
        got, k, v = tpl(x_local, B, S, cs, blk, valid)
        assert k.shape == (B, S, 1, 32) and v.shape == (B, S, 1, 32)
        err = (got - want.view(B * S, d)[rank * Ml:(rank + 1) * Ml]).abs().max().item()
        # parameter-sharded linear: each rank owns half of the weight rows and has its own activations
        w_full = torch.randn(24, d)
        xa = torch.randn(5, d, generator=torch.Generator().manual_seed(100 + rank))
        bias = torch.randn(24)
        y = tp.fsdp_linear(xa, w_full[rank * 12:(rank + 1) * 12].contiguous(), bias)
        err = max(err, (y - (xa @ w_full.t() + bias)).abs().max().item())
        gathered = [None] * world
        dist.all_gather_object(gathered, err)
        if rank == 0:
            ret["err"] = max(gathered)
    finally:
        dist.destroy_process_group()


def test_tp_layer_matches_unsharded_layer_on_two_ranks():
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main, args=(2, free_port(), ret), nprocs=2, join=True)
    assert ret["err"] < 1e-4


def test_kv_heads_are_replicated_when_fewer_than_ranks():
    from opentau_b200.parallel.tp import TensorParallel, TPDecoderLayer
    layer = DecoderLayer(TowerConfig(**{**CFG, "num_key_value_heads": 1}), 0)
    tp = TensorParallel("cpu")
    tp.world, tp.rank = 4, 3                      # shard arithmetic only; no collective is issued
    tpl = TPDecoderLayer(layer, tp)
    assert tpl.h_local == 1 and tpl.hk_local == 1 and tpl.w_qkv.shape == (3 * 32, 128)
    wq, wk, wv = layer.self_attn.qkv_proj.weight.split([128, 32, 32], 0)
    assert torch.equal(tpl.w_qkv[:32], wq[96:128]) and torch.equal(tpl.w_qkv[32:64], wk)
    assert tpl.w_o.shape == (128, 32) and tpl.w_gu.shape == (128, 128) and tpl.w_down.shape == (128, 64)


def _cosmos_rank(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import sys
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from helpers import tiny_batch
        from test_policies_cpu import _cosmos3
        from opentau_b200.datasets.synthetic import identity_stats
        from opentau_b200.parallel.tp import TensorParallel
        from opentau_b200.policies.cosmos3.tensor_parallel import TPBackbone
        from opentau_b200.policies.factory import make_policy
        errs = []
        for col in (None, 1):
            torch.manual_seed(0)
            pol = make_policy(_cosmos3(col=col), per_dataset_stats=[identity_stats()]).eval()
            b = tiny_batch(batch_size=4)
            images, masks = pol.prepare_images(b)
            lt, lm = pol.prepare_language(b)
            w = pol.model.qwen3vl_with_expert
            with torch.no_grad():
                full, pos_full = w.run_prefix(images, masks, lt, lm)
            sl = slice(rank * 2, rank * 2 + 2)
            tpb = TPBackbone(w, TensorParallel("cpu"))
            cache, pos = tpb.run_prefix([im[sl] for im in images], [m[sl] for m in masks], lt[sl], lm[sl])
            layers = [col] if col is not None else range(full.k.shape[0])
            for li in layers:
                n = full.length                         # the replicated cache carries spare slots behind the prefix
                errs.append(float((cache.k[li][:, :n] - full.k[li, sl, :n]).abs().max()))
                errs.append(float((cache.v[li][:, :n] - full.v[li, sl, :n]).abs().max()))
            assert torch.equal(pos, pos_full[:, sl]) and torch.equal(cache.valid, full.valid[sl])
        gathered = [None] * world
        dist.all_gather_object(gathered, max(errs))
        if rank == 0:
            ret["err"] = max(gathered)
    finally:
        dist.destroy_process_group()


def test_cosmos3_tensor_parallel_prefix_equals_replicated_backbone():
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_cosmos_rank, args=(2, free_port(), ret), nprocs=2, join=True)
    assert ret["err"] < 1e-4
