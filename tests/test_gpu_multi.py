"""Two-GPU checks of the peer-memory data-parallel step against the library (NCCL) step.

Skipped unless two CUDA devices are visible.  Ranks are child processes; NVLS is switched off; every rank
leaves only between steps with nothing in flight.
"""

import os

import pytest
from helpers import free_port
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, comm, ret, variant="plain"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import sys
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from helpers import tiny_batch, tiny_pi05
        from opentau_b200.ops import cuda_ops
        from opentau_b200.parallel.engine import OptimHyper, TrainEngine
        train_vision = variant == "mixed"            # the SigLIP patch / position tables stay fp32: a second flat group
        pol = tiny_pi05(device="cuda", seed=20 + rank, freeze_vision_encoder=not train_vision).to(torch.bfloat16)
        pol.train()
        from opentau_b200.parallel.fsdp import make_engine
        strategy = {"ddp": "ddp", "fsdp": "fsdp" if comm == "p2p" else "zero2"}.get(variant, "zero2")
        eng = make_engine(pol, OptimHyper(lr=1e-3, grad_clip_norm=1.0), device=dev, strategy=strategy, comm=comm,
                          overlap=variant != "no_overlap", bucket_elems=150_000)
        key = f"{comm}:{variant}"
        batch = tiny_batch(device=dev, seed=100 + rank)
        g = torch.Generator().manual_seed(7 + rank)
        noise = torch.randn(4, 10, 32, generator=g).to(dev)
        time = torch.full((4,), 0.5, device=dev)
        norms = []
        for _ in range(4):                   # step 1 learns the delivery counts, steps 2+ reduce under the backward
            out = pol(batch, noise=noise, time=time)
            loss = out["MSE"] + out["CE"]
            if eng.p2p is not None:
                eng._arm()
            loss.backward()
            norms.append(float(eng.optimizer_step()))
        torch.cuda.synchronize()
        cuda_ops.check_status()
        eng.check()
        import contextlib
        with (eng.full_params() if hasattr(eng, "full_params") else contextlib.nullcontext()):
            named = {n: p.detach().float().cpu() for n, p in pol.named_parameters() if p.requires_grad}
        if rank == 0:
            ret[key] = (named, norms, len(eng.store.groups), len(eng.store.buckets),
                        bool(eng.p2p is not None and eng._expected is not None))
        gathered = [None] * world
        dist.all_gather_object(gathered, float(sum(v.double().sum() for v in named.values())))
        if rank == 0:
            ret[key + "_same"] = all(abs(x - gathered[0]) < 1e-6 for x in gathered)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("variant", ["plain", "no_overlap", "ddp", "mixed", "fsdp"])
def test_peer_memory_step_matches_nccl_step(variant):
    """The bucketed, overlapped peer-memory step gives the parameters and gradient norms of the library step:
    with the reduction under the backward pass and without, under the ``ddp`` label (the norm must not be counted
    once per rank), for a model with an fp32 parameter group beside the bf16 one, and with the parameters
    themselves sharded (``fsdp``: per-layer gathers by peer loads into rotating slots)."""
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    ret = mgr.dict()
    for comm in ("nccl", "p2p"):
        mp.spawn(_worker, args=(2, free_port(), comm, ret, variant), nprocs=2, join=True)
    assert ret[f"nccl:{variant}_same"] and ret[f"p2p:{variant}_same"]
    (fa, na, _, _, _), (fb, nb, ngroups, nbuckets, learned) = ret[f"nccl:{variant}"], ret[f"p2p:{variant}"]
    assert nbuckets > 3 and learned
    if variant == "mixed":
        assert ngroups == 2
    for x, y in zip(na, nb):
        assert abs(x - y) / max(1e-6, abs(x)) < 2e-2
    for n in fa:
        torch.testing.assert_close(fa[n], fb[n], rtol=2e-2, atol=2e-3, msg=n)


def _timeout_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import sys
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from helpers import tiny_batch, tiny_pi05
        from opentau_b200.parallel.engine import OptimHyper, TrainEngine
        pol = tiny_pi05(device="cuda", seed=3).to(torch.bfloat16).train()
        eng = TrainEngine(pol, OptimHyper(lr=1e-2, grad_clip_norm=1.0), device=dev, comm="p2p", overlap=False)
        batch = tiny_batch(device=dev, seed=100 + rank)
        eng.train_step(batch)                                # a good step first
        torch.cuda.synchronize()
        eng.check()
        before = [g.data.clone() for g in eng.store.groups]
        dist.barrier()
        # Both ranks now wait on a flag value that nobody will ever write (the epoch jumps ahead on the waiting
        # side only, by a different amount per rank), with a budget of a few milliseconds: every wait gives up,
        # records it, and the data kernels behind it must leave the parameters alone.
        eng.p2p.wait_budget = 5_000_000
        eng.p2p.epoch += 1000 * (rank + 1)
        out = pol(batch)
        (out["MSE"] + out["CE"]).backward()
        eng.optimizer_step()
        torch.cuda.synchronize()
        raised = False
        try:
            eng.check()
        except RuntimeError:
            raised = True
        unchanged = all(torch.equal(a, g.data) for a, g in zip(before, eng.store.groups))
        flags = [None] * world
        dist.all_gather_object(flags, (raised, unchanged))
        if rank == 0:
            ret["timeout"] = flags
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_a_wait_that_gives_up_is_fatal_and_leaves_the_parameters_alone():
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_timeout_worker, args=(2, free_port(), ret), nprocs=2, join=True)
    assert all(r and u for r, u in ret["timeout"]), ret["timeout"]


def _tp_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from opentau_b200 import ops
        from opentau_b200.models.layers import DecoderLayer, TowerConfig
        from opentau_b200.ops import cuda_ops
        from opentau_b200.parallel.tp import TensorParallel, TPDecoderLayer
        torch.manual_seed(0)
        cfg = TowerConfig(hidden_size=512, num_hidden_layers=1, num_attention_heads=8, num_key_value_heads=2,
                          head_dim=64, intermediate_size=1024, vocab_size=64, hidden_act="silu", qk_norm=True,
                          norm_unit_offset=False)
        layer = DecoderLayer(cfg, 0).to(dev).to(torch.bfloat16)
        B, S, d = 4, 160, 512
        x = torch.randn(B, S, d, device=dev).to(torch.bfloat16)
        dist.broadcast(x, 0)
        for p in layer.parameters():
            dist.broadcast(p.data, 0)
        pos = torch.arange(S, device=dev)[None].expand(B, S)
        blk = (torch.arange(S, device=dev, dtype=torch.int32) // 40)[None].expand(B, S).contiguous()
        valid = torch.ones(B, S, dtype=torch.bool, device=dev)
        cs = ops.rope_angles(pos, cfg.head_dim, cfg.rope_theta)
        with torch.no_grad():
            h = layer.input_layernorm(x)[0]
            q, k, v = layer.self_attn.qkv(h)
            q, k = ops.rope(q, *cs), ops.rope(k, *cs)
            att = ops.block_attention(q, k, v, blk, blk, valid, valid, cfg.attn_scale)
            y = layer.self_attn.o_proj(att, residual=x)
            want = layer.mlp(layer.post_attention_layernorm(y)[0], residual=y).view(B * S, d)
            tp = TensorParallel(dev, backend="p2p", wait_budget=4_000_000_000)
            tpl = TPDecoderLayer(layer, tp)
            Ml = B * S // world
            x_local = x.view(B * S, d)[rank * Ml:(rank + 1) * Ml].contiguous()
            errs = []
            for _ in range(4):                       # several steps: both parities of every workspace are reused
                got, _, _ = tpl(x_local, B, S, cs, blk, valid)
                errs.append(float((got.float() - want[rank * Ml:(rank + 1) * Ml].float()).abs().max()))
            # parameter-sharded linear: weight rows split over the ranks, every rank with its own activations
            w_full = (torch.randn(1024, d, device=dev) * 0.05).to(torch.bfloat16)
            dist.broadcast(w_full, 0)
            xa = torch.randn(192, d, device=dev).to(torch.bfloat16)          # differs per rank (seeded per device)
            shard = w_full[rank * 512:(rank + 1) * 512].contiguous()
            for _ in range(3):
                got = tp.fsdp_linear(xa, shard)
                errs.append(float((got.float() - xa.float() @ w_full.float().t()).abs().max()) / 4.0)
            torch.cuda.synchronize()
            cuda_ops.check_status()
        allerr = [None] * world
        dist.all_gather_object(allerr, max(errs))
        if rank == 0:
            ret["tp_err"] = max(allerr)
            ret["tp_scale"] = float(want.float().abs().max())
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_tensor_parallel_layer_matches_unsharded_layer():
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_tp_worker, args=(2, free_port(), ret), nprocs=2, join=True)
    assert ret["tp_err"] < 0.03 * max(1.0, ret["tp_scale"])


def _cp_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from opentau_b200 import ops
        from opentau_b200.ops import cuda_ops
        from opentau_b200.parallel.cp import ContextParallel
        torch.manual_seed(0)
        B, S, H, Hkv, D = 2, 640, 8, 4, 256
        q = torch.randn(B, S, H, D, device=dev).to(torch.bfloat16)
        k = torch.randn(B, S, Hkv, D, device=dev).to(torch.bfloat16)
        v = torch.randn(B, S, Hkv, D, device=dev).to(torch.bfloat16)
        do = torch.randn(B, S, H * D, device=dev).to(torch.bfloat16)
        for t in (q, k, v, do):
            dist.broadcast(t, 0)
        blk = (torch.arange(S, device=dev, dtype=torch.int32) // 100)[None].expand(B, S).contiguous()
        valid = torch.ones(B, S, dtype=torch.bool, device=dev)
        valid[1, 37] = False
        qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
        want = ops.block_attention(qr, kr, vr, blk, blk, valid, valid, D ** -0.5)
        want.backward(do)
        cp = ContextParallel(dev, backend="p2p", wait_budget=4_000_000_000)
        errs = []
        for _ in range(3):                           # both parities of the K/V shards are reused
            ql, kl, vl = (cp.shard(t).clone().requires_grad_(True) for t in (q, k, v))
            got = cp.attention(ql, kl, vl, cp.shard(blk).contiguous(), blk, cp.shard(valid).contiguous(), valid, D ** -0.5)
            got.backward(cp.shard(do).contiguous())
            errs += [float((got.float() - cp.shard(want).float()).abs().max()),
                     float((ql.grad.float() - cp.shard(qr.grad).float()).abs().max()),
                     float((kl.grad.float() - cp.shard(kr.grad).float()).abs().max()),
                     float((vl.grad.float() - cp.shard(vr.grad).float()).abs().max())]
        torch.cuda.synchronize()
        cuda_ops.check_status()
        allerr = [None] * world
        dist.all_gather_object(allerr, max(errs))
        if rank == 0:
            ret["cp_err"] = max(allerr)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_context_parallel_attention_matches_single_gpu():
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_cp_worker, args=(2, free_port(), ret), nprocs=2, join=True)
    assert ret["cp_err"] < 0.06


def _cp_policy_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import sys
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from helpers import tiny_batch, tiny_pi05
        from opentau_b200.ops import cuda_ops
        from opentau_b200.parallel.cp import ContextParallel
        batch = tiny_batch(device=dev, batch_size=2, seed=50 + rank)
        g = torch.Generator().manual_seed(3 + rank)
        noise, time = torch.randn(2, 10, 32, generator=g).to(dev), torch.full((2,), 0.4, device=dev)
        results = []
        for use_cp in (False, True):
            pol = tiny_pi05(device="cuda", seed=7).to(dev).to(torch.bfloat16).train()
            if use_cp:
                pol.model.context_parallel = ContextParallel(dev, backend="p2p", wait_budget=4_000_000_000)
            for _ in range(2):                      # twice: both parities of the staging buffers
                pol.zero_grad(set_to_none=True)
                out = pol(batch, noise=noise, time=time)
                (out["MSE"] + out["CE"]).backward()
            grads = {}
            for n, p in pol.named_parameters():
                if p.requires_grad and p.grad is not None:
                    gsum = p.grad.float().clone()
                    dist.all_reduce(gsum)
                    grads[n] = gsum
            results.append((float(out["MSE"]), float(out["CE"]), grads))
        torch.cuda.synchronize()
        cuda_ops.check_status()
        (m0, c0, g0), (m1, c1, g1) = results
        worst = max(float((g0[n] - g1[n]).abs().max()) / (float(g0[n].abs().max()) + 1e-3) for n in g0)
        gathered = [None] * world
        dist.all_gather_object(gathered, (abs(m0 - m1) / max(1.0, abs(m0)), abs(c0 - c1) / max(1.0, abs(c0)), worst))
        if rank == 0:
            ret["cp_policy"] = gathered
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_policy_under_context_parallelism_matches_the_unsharded_policy():
    """Tiny pi0.5 in bf16 with the prefix split over two GPUs (fused forward kernel, sharded backward, peer-memory
    K/V gather and dK/dV reduce-scatter): losses and rank-summed gradients equal the unsharded pass."""
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_cp_policy_worker, args=(2, free_port(), ret), nprocs=2, join=True)
    for dm, dc, worst in ret["cp_policy"]:
        assert dm < 3e-2 and dc < 3e-2 and worst < 0.15, ret["cp_policy"]


def _tp_backbone_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import sys
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from helpers import tiny_batch
        from opentau_b200.configs.types import FeatureType, PolicyFeature
        from opentau_b200.datasets.synthetic import identity_stats
        from opentau_b200.ops import cuda_ops
        from opentau_b200.parallel.tp import TensorParallel
        from opentau_b200.policies.cosmos3.tensor_parallel import TPBackbone
        from opentau_b200.policies.factory import make_policy, make_policy_config
        feats = {"camera0": PolicyFeature(FeatureType.VISUAL, (3, 224, 224)),
                 "state": PolicyFeature(FeatureType.STATE, (32,))}
        errs, scale = [], 1.0
        for col in (None, 1):
            torch.manual_seed(0)
            cfg = make_policy_config(
                "cosmos3", chunk_size=10, n_action_steps=10, prompt_max_length=32, dropout=0.0, device=str(dev),
                image_resize=128, input_features=dict(feats), num_steps=3, load_pretrained_backbone=False,
                output_features={"actions": PolicyFeature(FeatureType.ACTION, (32,))},
                backbone=dict(hidden_size=512, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2,
                              head_dim=64, intermediate_size=1024, vocab_size=1024, mrope_sections=(12, 10, 10)),
                vision=dict(hidden_size=64, depth=2, num_heads=4, intermediate_size=128, out_hidden_size=512,
                            num_position_embeddings=64, deepstack_visual_indexes=(0,)),
                expert_hidden_size=128, expert_intermediate_size=256, expert_num_hidden_layers=2,
                expert_num_attention_heads=4, expert_num_key_value_heads=2, expert_head_dim=64,
                expert_adarms_cond_dim=32, proj_width=128, condition_on_layer=col)
            pol = make_policy(cfg, per_dataset_stats=[identity_stats()]).to(dev).to(torch.bfloat16).eval()
            for p in pol.parameters():
                dist.broadcast(p.data, 0)
            b = tiny_batch(device=dev, batch_size=4, prompt_len=32)
            images, masks = pol.prepare_images(b)
            lt, lm = pol.prepare_language(b)
            w = pol.model.qwen3vl_with_expert
            with torch.no_grad():
                full, pos_full = w.run_prefix(images, masks, lt, lm)
            sl = slice(rank * 2, rank * 2 + 2)
            tpb = TPBackbone(w, TensorParallel(dev, backend="p2p", wait_budget=4_000_000_000))
            for _ in range(2):                      # twice: both parities of the kernels' workspaces
                cache, pos = tpb.run_prefix([im[sl] for im in images], [m[sl] for m in masks], lt[sl], lm[sl])
            layers = [col] if col is not None else range(full.k.shape[0])
            n = full.length
            for li in layers:
                errs.append(float((cache.k[li][:, :n].float() - full.k[li, sl, :n].float()).abs().max()))
                errs.append(float((cache.v[li][:, :n].float() - full.v[li, sl, :n].float()).abs().max()))
                scale = max(scale, float(full.k[li].float().abs().max()), float(full.v[li].float().abs().max()))
            assert torch.equal(pos, pos_full[:, sl])
        # sampling through the sharded backbone: eager, then with the expert loop replayed from a graph (captured on
        # the first call, replayed on the second); same noise, so the three chunks agree
        w.tp_backbone = tpb
        mine = {k: (v[sl] if isinstance(v, (torch.Tensor, list)) else v) for k, v in b.items()}
        noise = torch.randn(2, 10, 32, device=dev, generator=torch.Generator(device=dev).manual_seed(5))
        eager = pol.sample_actions(mine, noise=noise).float()
        pol.enable_cuda_graphs(True)
        first = pol.sample_actions(mine, noise=noise).float()
        again = pol.sample_actions(mine, noise=noise).float()
        graph_err = max(float((first - eager).abs().max()), float((again - eager).abs().max()))
        torch.cuda.synchronize()
        cuda_ops.check_status()
        gathered = [None] * world
        dist.all_gather_object(gathered, (max(errs), scale, graph_err))
        if rank == 0:
            ret["tpb"] = gathered
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_cosmos3_tensor_parallel_backbone_matches_the_replicated_backbone_on_gpus():
    """``TPBackbone.run_prefix`` with the fused GEMM + collective kernels on two GPUs leaves each rank the same
    per-layer keys / values for its own samples as the replicated backbone (all layers, and one conditioning layer)."""
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_tp_backbone_worker, args=(2, free_port(), ret), nprocs=2, join=True)
    for err, scale, graph_err in ret["tpb"]:
        assert err < 0.04 * scale, ret["tpb"]
        assert graph_err < 0.05, ret["tpb"]
