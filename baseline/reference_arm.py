"""Reference arm of ``bench.py``: the UNMODIFIED reference package installed under ``baseline/_ref``, driven
through its own public classes on the benchmark's config.

Training step (what ``opentau/scripts/train.py: update_policy`` does for the DDP / single-process backend):
``PI05Policy.forward(batch)`` -> weighted ``MSE + CE`` -> ``backward`` -> ``MasterWeightOptimizer.clip_grad_norm_``
-> ``MasterWeightOptimizer.step`` -> ``zero_grad`` -> scheduler step -> read the loss on the host.  For N > 1 the
policy is wrapped in ``torch.nn.parallel.DistributedDataParallel`` (what accelerate's MULTI_GPU backend does) and
the loss is all-gathered like ``gather_for_metrics``.

None of this repository's models, kernels or engine is imported here.  What is NOT the reference's own, and is
disclosed in the printed line:

* ``reference_shims``: stand-in modules for pure-Python dependencies missing from the offline image
  (``ref_shims.py``); none of them runs inside the step.
* ``tokenizer_assets``: the PaliGemma tokenizer and the FAST action tokenizer are hub downloads.  Synthetic
  objects with the same call surface emit uniform-random ids of the configured lengths (which is what the
  benchmark's synthetic data is anyway); they are cheaper than the real CPU tokenizers, which favours the reference.
"""

from __future__ import annotations

import contextlib
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.path.join(HERE, "_ref")


class SyntheticTokenizer:
    """Call surface of the PaliGemma tokenizer used by the reference policy; ids are uniform random."""

    vocab_size = 257152
    bos_token_id, eos_token_id, pad_token_id = 2, 1, 0
    eos_token, bos_token, pad_token = "<eos>", "<bos>", "<pad>"

    def __init__(self, seed: int = 0, id_high: int = 256000):
        import torch
        self._g = torch.Generator().manual_seed(seed)
        self._high = id_high

    def __len__(self):
        return self.vocab_size

    def add_tokens(self, tokens, special_tokens=False):
        return 0

    def convert_tokens_to_ids(self, tok):
        return {"<eos>": 1, "<bos>": 2, "<pad>": 0}.get(tok, 3)

    def encode(self, text, add_special_tokens=False):
        # short indicator strings ("State: ", ":\n", "Response: ", "Action: "): a few fixed ids
        return [100 + (ord(c) % 50) for c in text.strip()[:3]] or [100]

    def __call__(self, texts, padding=None, padding_side="right", max_length=None, return_tensors="pt",
                 truncation=True, **_):
        import torch
        n = len(texts)
        ids = torch.randint(3, self._high, (n, max_length), generator=self._g, dtype=torch.long)
        return {"input_ids": ids, "attention_mask": torch.ones(n, max_length, dtype=torch.long)}

    def decode(self, ids, **_):
        return ""

    def batch_decode(self, ids, **_):
        return ["" for _ in ids]


class SyntheticFastProcessor:
    """Call surface of the FAST action tokenizer: one list of ``n_tokens`` uniform ids per sample."""

    def __init__(self, vocab_size: int, n_tokens: int, seed: int = 1):
        import numpy as np
        self.vocab_size, self.n_tokens = vocab_size, n_tokens
        self._rng = np.random.default_rng(seed)

    def __call__(self, actions):
        return [self._rng.integers(0, self.vocab_size, self.n_tokens).tolist() for _ in range(len(actions))]

    def decode(self, tokens, **_):
        raise NotImplementedError("synthetic FAST processor: decoding is not part of the training step")


def _unavailable(why: str) -> int:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why[:400]}))
    return 0


def _prepare_imports():
    sys.path.insert(0, HERE)
    sys.path.insert(0, REF_ROOT)
    import ref_shims
    return ref_shims.install()


def _tiny_geometry(module):
    """CPU plumbing check only: shrink the wrapper's default geometry after the reference built it (the wrapper
    config cannot take geometry dictionaries); the benchmark never uses this."""
    full = module.PaliGemmaWithExpertConfig

    def make(**kw):
        c = full(**kw)
        t, v, e = c.paligemma_config.text_config, c.paligemma_config.vision_config, c.gemma_expert_config
        for obj, vals in ((t, dict(hidden_size=256, intermediate_size=512, num_attention_heads=4, num_hidden_layers=2,
                                   num_key_value_heads=1, head_dim=64, vocab_size=1024)),
                          (v, dict(hidden_size=128, intermediate_size=256, num_attention_heads=4, num_hidden_layers=2,
                                   projection_dim=256)),
                          (e, dict(hidden_size=128, intermediate_size=256, num_attention_heads=4, num_hidden_layers=2,
                                   num_key_value_heads=1, head_dim=64, vocab_size=1024, adarms_cond_dim=128)),
                          (c.paligemma_config, dict(hidden_size=256, projection_dim=256, image_token_index=1024,
                                                    _vocab_size=1024))):
            for k, val in vals.items():
                setattr(obj, k, val)
        return c

    module.PaliGemmaWithExpertConfig = make


def run_train(args) -> int:
    """Prints the benchmark line for the reference's pi0.5 training step (or its ``unavailable`` line)."""
    if not os.path.isdir(os.path.join(REF_ROOT, "opentau")):
        return _unavailable("baseline/_ref holds no installed reference (pip install --target baseline/_ref "
                            "<reference checkout> was not run on this machine)")
    try:
        shims = _prepare_imports()
        import torch
        import torch.distributed as dist
        import opentau  # noqa: F401  (applies the reference's own transformers patches)
        from opentau.configs.types import FeatureType, PolicyFeature
        from opentau.optim.master_weights import MasterWeightOptimizer
        from opentau.policies.pi05 import modeling_pi05 as ref_modeling
        from opentau.policies.pi05.configuration_pi05 import PI05Config
    except Exception as exc:  # the import chain itself does not work on this image
        import traceback
        return _unavailable(f"reference import failed: {type(exc).__name__}: {exc} | "
                            f"{traceback.format_exc().strip().splitlines()[-3:]}")

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available()
    device = torch.device(f"cuda:{local_rank}" if use_cuda else "cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl" if use_cuda else "gloo", device_id=device if use_cuda else None)

    cams, fast_len, fast_vocab = 3, 256, 2048
    prompt_len = 200
    if args.tiny:
        fast_len, fast_vocab, prompt_len = 16, 256, 16
        _tiny_geometry(ref_modeling)
        SyntheticTokenizer.vocab_size = 1024
    tok = SyntheticTokenizer(seed=rank, id_high=1000 if args.tiny else 256000)
    fast = SyntheticFastProcessor(fast_vocab, fast_len, seed=100 + rank)

    class _Tok:
        @staticmethod
        def from_pretrained(*_a, **_k):
            return tok

    class _Proc:
        @staticmethod
        def from_pretrained(*_a, **_k):
            return fast

    # the two hub assets, swapped in the reference module's namespace (the files stay untouched)
    ref_modeling.AutoTokenizer, ref_modeling.AutoProcessor = _Tok, _Proc

    feats = {f"camera{i}": PolicyFeature(type=FeatureType.VISUAL, shape=(3, 224, 224)) for i in range(cams)}
    feats["state"] = PolicyFeature(type=FeatureType.STATE, shape=(32,))
    attn = args.ref_attn
    compile_on = args.ref_compile == "on"
    try:
        cfg = PI05Config(chunk_size=50, n_action_steps=50, prompt_max_length=prompt_len,
                         discrete_action_max_length=fast_len, knowledge_insulation=True, dropout=args.dropout,
                         freeze_vision_encoder=not args.train_vision, train_expert_only=False,
                         attention_implementation=attn, use_torch_compile=compile_on,
                         **({"proj_width": 128} if args.tiny else {}),
                         input_features=feats,
                         output_features={"actions": PolicyFeature(type=FeatureType.ACTION, shape=(32,))})
        torch.manual_seed(1234)
        stats = _identity_stats(torch, cams)
        with torch.device(device):
            policy = ref_modeling.PI05Policy(cfg, per_dataset_stats=[stats])
        policy.to(device)
        policy.to(torch.bfloat16)  # train.py does this for every backend but FSDP
        policy.train()
        policy.maybe_compile_for_training()
        inner = cfg.get_optimizer_preset().build(p for p in policy.get_optim_params() if p.requires_grad)
        scheduler = cfg.get_scheduler_preset().build(inner, 30_000)
        optimizer = MasterWeightOptimizer.from_existing(inner)
        scheduler.optimizer = optimizer
    except Exception as exc:
        import traceback
        traceback.print_exc(file=sys.stderr)
        return _unavailable(f"reference policy construction failed on this image (transformers "
                            f"{_tf_version()}): {type(exc).__name__}: {exc}")

    model = policy
    if world > 1:
        find_unused = os.environ.get("FIND_UNUSED_PARAMS", "true").lower() == "true"  # train.py's default
        model = torch.nn.parallel.DistributedDataParallel(
            policy, device_ids=[local_rank] if use_cuda else None, find_unused_parameters=find_unused)

    B = args.batch
    n_host = 4

    def host_batch(seed):
        g = torch.Generator().manual_seed(seed)
        b = {f"camera{i}": torch.rand(B, 3, 224, 224, generator=g) for i in range(cams)}
        b["state"] = torch.randn(B, 32, generator=g).clamp_(-1, 1)
        b["actions"] = torch.randn(B, 50, 32, generator=g)
        b["action_is_pad"] = torch.zeros(B, 50, dtype=torch.bool)
        b["dataset_index"] = torch.zeros(B, dtype=torch.long)
        b["real_action_dim"] = torch.full((B,), 32, dtype=torch.long)
        if use_cuda:
            b = {k: v.pin_memory() for k, v in b.items()}
        return b

    host = [host_batch(1000 * rank + i) for i in range(n_host)]
    prompts = ["pick up the object and place it in the bin"] * B
    h2d_bytes = sum(v.numel() * v.element_size() for v in host[0].values())
    weights = {"MSE": 1.0, "CE": 1.0}

    accum = max(1, int(getattr(args, "ref_accum", 1)))   # the reference's gradient_accumulation_steps
    micro = B // accum

    def step(batch):
        """One optimizer step over ``accum`` micro-batches (accelerate's ``accumulate``: gradients are synchronised
        on the last micro-batch only, the loss is divided by the number of micro-batches)."""
        total = None
        for a in range(accum):
            mb = batch if accum == 1 else {k: v[a * micro:(a + 1) * micro] for k, v in batch.items()}
            last = a == accum - 1
            ctx = model.no_sync() if (world > 1 and not last) else contextlib.nullcontext()
            with ctx:
                losses = model(mb) if world > 1 else policy.forward(mb)
                losses.pop("outlier_records", None)
                # scripts/train.py: _assemble_weighted_loss with the default loss_weighting {"MSE": 1, "CE": 1},
                # summed in the fixed (MSE, CE) order (importing that script would pull the whole launcher stack)
                loss = weights["MSE"] * losses["MSE"] + weights["CE"] * losses["CE"]
                (loss / accum if accum > 1 else loss).backward()
            total = loss.detach() if total is None else total + loss.detach()
        optimizer.clip_grad_norm_(10.0)
        optimizer.step()
        optimizer.zero_grad()
        scheduler.step()
        return total / accum

    def to_device(hb, non_blocking):
        b = {k: v.to(device, non_blocking=non_blocking) for k, v in hb.items()}
        b["prompt"] = list(prompts)
        return b

    dev_batches = [to_device(h, False) for h in host[:2]]

    def sync():
        if world > 1:
            dist.barrier()
        if use_cuda:
            torch.cuda.synchronize()

    def run_device_only(n):
        for i in range(n):
            step(dict(dev_batches[i % 2]))

    def run_e2e(n):
        last = None
        for i in range(n):
            loss = step(to_device(host[i % n_host], True))
            if world > 1:  # gather_for_metrics(loss).mean().item()
                out = [torch.empty_like(loss) for _ in range(world)]
                dist.all_gather(out, loss.detach())
                last = float(torch.stack(out).float().mean().item())
            else:
                last = float(loss.item())
        return last

    def timed(fn, n):
        sync()
        if use_cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            res = fn(n)
            e1.record()
            sync()
            ms = e0.elapsed_time(e1)
        else:
            t0 = time.perf_counter()
            res = fn(n)
            ms = (time.perf_counter() - t0) * 1e3
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), res

    failure = None
    try:
        t_first = time.perf_counter()
        run_device_only(1)
        if use_cuda:
            torch.cuda.synchronize()
        first_step_s = time.perf_counter() - t_first
        run_device_only(max(args.warmup - 1, 0))
    except Exception as exc:
        import traceback
        traceback.print_exc(file=sys.stderr)
        failure = (type(exc).__name__, str(exc)[:160])
    if failure is not None:
        # outside the except block, so the failed step's frames (and their activations) are gone before the retry
        oom = "OutOfMemory" in failure[0]
        retry = None
        if compile_on and not oom:
            # the reference's default (use_torch_compile) does not build on this image: its eager path
            retry = dict(ref_compile="off", compile_error=f"{failure[0]}: {failure[1]}")
        elif oom and accum < 4 and B % (accum * 2) == 0:
            # batch 32 does not fit in one pass of the reference: its own lever, gradient_accumulation_steps
            retry = dict(ref_accum=accum * 2, oom_at=getattr(args, "oom_at", []) + [f"micro-batch {micro}"])
        if retry is None:
            return _unavailable(f"reference training step failed on this image (attention={attn}, "
                                f"compile={compile_on}, micro-batch {micro}): {failure[0]}: {failure[1]}")
        for k, v in retry.items():
            setattr(args, k, v)
        policy = model = optimizer = inner = scheduler = dev_batches = None  # noqa: F841  (drops the closures' cells)
        import gc
        torch._dynamo.reset()
        gc.collect()
        if use_cuda:
            torch.cuda.empty_cache()
        return run_train(args)

    sampler = args.clock_sampler(local_rank) if (rank == 0 and use_cuda) else None
    if sampler:
        sampler.start()
    ms_dev, _ = timed(run_device_only, args.steps)
    run_e2e(1)
    ms_e2e, last_loss = timed(run_e2e, args.steps)
    clocks = sampler.stop() if sampler else {}
    gb = B * world
    if rank == 0:
        peak_gb = torch.cuda.max_memory_allocated() / 2**30 if use_cuda else 0.0
        print(json.dumps({
            "metric": "pi0.5 train samples/s/box", "value": round(gb * args.steps / (ms_dev / 1e3), 3),
            "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_dev / args.steps, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
            "config": {"model": "pi0.5 full (reference PI05Policy, default geometry)" if not args.tiny
                       else "pi0.5 tiny (plumbing)", "global_batch": gb, "seq_len": 3 * 256 + prompt_len + 3 + fast_len,
                       "parallelism": f"dp{world}-ddp-{'nccl' if use_cuda else 'gloo'}" if world > 1 else "single",
                       "optimizer": "MasterWeightOptimizer(AdamW fused) + clip 10", "attention_implementation": attn,
                       "use_torch_compile": compile_on, "dropout": args.dropout,
                       **({"torch_compile_failed": args.compile_error} if getattr(args, "compile_error", None) else {}),
                       "gradient_accumulation_steps": accum, "micro_batch": micro,
                       **({"out_of_memory_at": args.oom_at} if getattr(args, "oom_at", None) else {}),
                       "knowledge_insulation": True, "fast_tokens": fast_len,
                       "frozen_weights": "none" if args.train_vision else "SigLIP tower (policy default)",
                       "first_step_s": round(first_step_s, 1), "peak_mem_gib": round(peak_gb, 2),
                       "l2": "per-step working set far exceeds the 126 MB L2; no explicit flush"},
            "reference_shims": shims,
            "env": {k: os.environ.get(k) for k in ("PYTORCH_CUDA_ALLOC_CONF", "CXX", "CC", "FIND_UNUSED_PARAMS")},
            "tokenizer_assets": "synthetic (hub tokenizers unavailable offline): uniform-random ids, 200 prompt + "
                                "256 FAST tokens",
            "clocks": clocks,
            "e2e": {"value": round(gb * args.steps / (ms_e2e / 1e3), 3), "unit": "samples/s",
                    "ms_per_step": round(ms_e2e / args.steps, 3), "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": 4, "last_loss": last_loss},
            "gpu_launches": 0,
        }))
    if world > 1:
        dist.destroy_process_group()
    return 0


def run_infer(args) -> int:
    """Prints the benchmark line for the reference's pi0.5 action-chunk latency (scripts/benchmark_inference.py:
    policy in bf16 with the SigLIP embeddings kept fp32, ``policy.model.sample_actions`` compiled unless
    ``--ref-compile off``, batch 1, ``policy.sample_actions`` in a timed loop), or its ``unavailable`` line."""
    if args.model != "pi05":
        return _unavailable(f"the reference arm builds pi0.5 only; the {args.model} policy of the reference needs its "
                            "backbone's hub processor files, which this machine cannot fetch (cosmos3 has a "
                            "published 1 x B200 figure instead, carried in vs_baseline)")
    if not os.path.isdir(os.path.join(REF_ROOT, "opentau")):
        return _unavailable("baseline/_ref holds no installed reference (pip install --target baseline/_ref "
                            "<reference checkout> was not run on this machine)")
    try:
        shims = _prepare_imports()
        import torch
        import torch.distributed as dist
        import opentau  # noqa: F401
        from opentau.configs.types import FeatureType, PolicyFeature
        from opentau.policies.pi05 import modeling_pi05 as ref_modeling
        from opentau.policies.pi05.configuration_pi05 import PI05Config
        from opentau.policies.utils import to_dtype_preserving_siglip_float32
    except Exception as exc:
        import traceback
        return _unavailable(f"reference import failed: {type(exc).__name__}: {exc} | "
                            f"{traceback.format_exc().strip().splitlines()[-3:]}")

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available()
    device = torch.device(f"cuda:{local_rank}" if use_cuda else "cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl" if use_cuda else "gloo", device_id=device if use_cuda else None)

    cams, prompt_len, num_steps = 3, 200, 10
    if args.tiny:
        prompt_len = 16
        _tiny_geometry(ref_modeling)
        SyntheticTokenizer.vocab_size = 1024
    tok = SyntheticTokenizer(seed=rank, id_high=1000 if args.tiny else 256000)
    fast = SyntheticFastProcessor(256 if args.tiny else 2048, 16 if args.tiny else 256, seed=100 + rank)
    ref_modeling.AutoTokenizer = type("_Tok", (), {"from_pretrained": staticmethod(lambda *a, **k: tok)})
    ref_modeling.AutoProcessor = type("_Proc", (), {"from_pretrained": staticmethod(lambda *a, **k: fast)})

    feats = {f"camera{i}": PolicyFeature(type=FeatureType.VISUAL, shape=(3, 224, 224)) for i in range(cams)}
    feats["state"] = PolicyFeature(type=FeatureType.STATE, shape=(32,))
    compile_on = args.ref_compile == "on"
    try:
        cfg = PI05Config(chunk_size=50, n_action_steps=50, prompt_max_length=prompt_len, num_steps=num_steps,
                         discrete_action_max_length=16 if args.tiny else 256,
                         attention_implementation=args.ref_attn,
                         **({"proj_width": 128} if args.tiny else {}),
                         input_features=feats,
                         output_features={"actions": PolicyFeature(type=FeatureType.ACTION, shape=(32,))})
        torch.manual_seed(1234)
        with torch.device(device):
            policy = ref_modeling.PI05Policy(cfg, per_dataset_stats=[_identity_stats(torch, cams)])
        to_dtype_preserving_siglip_float32(policy, device=device, dtype=torch.bfloat16)
        policy.eval()
        policy.reset()
    except Exception as exc:
        import traceback
        traceback.print_exc(file=sys.stderr)
        return _unavailable(f"reference policy construction failed on this image (transformers "
                            f"{_tf_version()}): {type(exc).__name__}: {exc}")

    g = torch.Generator().manual_seed(7 + rank)
    host = {f"camera{i}": torch.rand(1, 3, 224, 224, generator=g).to(torch.bfloat16) for i in range(cams)}
    host["state"] = torch.randn(1, 32, generator=g).clamp_(-1, 1).to(torch.bfloat16)
    if use_cuda:
        host = {k: v.pin_memory() for k, v in host.items()}
    h2d_bytes = sum(v.numel() * v.element_size() for v in host.values())
    prompt = ["pick up the object and place it in the bin"]

    def observation(non_blocking):
        b = {k: v.to(device, non_blocking=non_blocking) for k, v in host.items()}
        b["prompt"] = list(prompt)
        return b

    resident = observation(False)
    eager = policy.model.sample_actions
    compile_error = None

    def one(e2e: bool):
        if use_cuda:
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        t0 = time.perf_counter()
        with torch.inference_mode():
            out = policy.sample_actions(observation(True) if e2e else dict(resident))
            if e2e:
                out = out.float().cpu()
        if use_cuda:
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1), out
        return (time.perf_counter() - t0) * 1e3, out

    n_warm = max(args.warmup, 3)
    if compile_on:
        torch._dynamo.reset()
        policy.model.sample_actions = torch.compile(eager, mode="reduce-overhead", fullgraph=False)
    try:
        first_ms = one(False)[0]
        for _ in range(n_warm - 1):
            one(False)
    except Exception as exc:
        if not compile_on:
            import traceback
            traceback.print_exc(file=sys.stderr)
            return _unavailable(f"reference sample_actions failed on this image: {type(exc).__name__}: "
                                f"{str(exc)[:160]}")
        compile_error = f"{type(exc).__name__}: {str(exc)[:160]}"
    if compile_error is not None:
        # the compiled sampler does not build here: the reference's own --no-compile path
        torch._dynamo.reset()
        policy.model.sample_actions = eager
        compile_on = False
        first_ms = one(False)[0]
        for _ in range(n_warm - 1):
            one(False)

    def sync():
        if world > 1:
            dist.barrier()
        if use_cuda:
            torch.cuda.synchronize()

    sampler = args.clock_sampler(local_rank) if (rank == 0 and use_cuda) else None
    if sampler:
        sampler.start()
    sync()
    dev_ms = sorted(one(False)[0] for _ in range(args.steps))
    sync()
    one(True)
    res = [one(True) for _ in range(args.steps)]
    sync()
    clocks = sampler.stop() if sampler else {}
    e2e_ms, out = sorted(r[0] for r in res), res[-1][1]
    stats = torch.tensor([dev_ms[len(dev_ms) // 2], e2e_ms[len(e2e_ms) // 2], sum(dev_ms) / len(dev_ms)],
                         dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({
            "metric": f"pi05 p50 {num_steps}-step action-chunk latency", "value": round(float(stats[0]), 3),
            "unit": "ms", "n_gpus": world, "steps": args.steps, "warmup": n_warm,
            "ms_per_step": round(float(stats[2]), 3), "higher_is_better": False, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
            "config": {"model": "pi0.5 full (reference PI05Policy, default geometry)" if not args.tiny
                       else "pi0.5 tiny (plumbing)", "global_batch": world, "parallelism": f"replica x{world}",
                       "denoise_steps": num_steps, "action_chunk": "50x32", "prompt_tokens": prompt_len,
                       "attention_implementation": args.ref_attn,
                       "torch_compile": "reduce-overhead" if compile_on else "off",
                       **({"torch_compile_failed": compile_error} if compile_error else {}),
                       "first_call_ms": round(first_ms, 1),
                       "l2": "each call streams every bf16 weight once (GBs, far more than the 126 MB L2); no "
                             "explicit flush"},
            "reference_shims": shims,
            "env": {k: os.environ.get(k) for k in ("PYTORCH_CUDA_ALLOC_CONF", "CXX", "CC")},
            "tokenizer_assets": "synthetic (hub tokenizers unavailable offline): uniform-random ids",
            "clocks": clocks,
            "e2e": {"value": round(float(stats[1]), 3), "unit": "ms", "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": out.numel() * out.element_size()},
            "gpu_launches": 0,
        }))
    if world > 1:
        dist.destroy_process_group()
    return 0


def _tf_version() -> str:
    try:
        import transformers
        return transformers.__version__
    except Exception:
        return "?"


def _identity_stats(torch, cams: int) -> dict:
    """Per-dataset statistics under which every normalisation mode is the identity map."""
    def one(shape, img=False):
        z, o = torch.zeros(shape), torch.ones(shape)
        return {"mean": z.clone(), "std": o.clone(), "min": -o.clone() if not img else z.clone(), "max": o.clone(),
                "q01": -o.clone(), "q99": o.clone()}
    s = {f"camera{i}": one((3, 1, 1), img=True) for i in range(cams)}
    s["state"] = one((32,))
    s["actions"] = one((32,))
    return s
