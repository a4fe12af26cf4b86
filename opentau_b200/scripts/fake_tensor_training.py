"""Shape / wiring smoke test on fake tensors (reference ``src/opentau/scripts/fake_tensor_training.py:34-93``): build
the policy and run one forward + backward under ``FakeTensorMode``, which allocates nothing, so even the largest
configuration can be checked on a laptop.  Native kernels are bypassed (fake tensors have no storage): the oracle
operator set is selected for the duration."""

from __future__ import annotations

import logging
import os

import torch

from ..configs import parser
from ..configs.train import TrainPipelineConfig
from ..utils.fake_tensor import FakeTensorContext


@parser.wrap()
def main(cfg: TrainPipelineConfig):
    from ..datasets.synthetic import SyntheticSpec, identity_stats, make_synthetic_batch
    from ..policies.factory import make_policy
    os.environ["OPENTAU_B200_ORACLE"] = "1"
    pc = cfg.policy
    spec = SyntheticSpec(batch_size=2, num_cams=cfg.num_cams, resolution=tuple(cfg.resolution),
                         prompt_len=getattr(pc, "prompt_max_length", 16), chunk_size=cfg.action_chunk,
                         discrete_action_len=getattr(pc, "discrete_action_max_length", 8),
                         discrete_action_vocab=getattr(pc, "discrete_action_vocab_size", 256))
    batch = make_synthetic_batch(spec)
    with FakeTensorContext():
        policy = make_policy(pc, per_dataset_stats=[identity_stats(cfg.max_state_dim, cfg.max_action_dim)])
        out = policy(batch)
        (out["MSE"] + out["CE"]).backward()
    n = sum(p.numel() for p in policy.parameters())
    logging.info("fake-tensor step ok: %.2f B parameters, losses %s", n / 1e9, {k: tuple(v.shape) for k, v in out.items()
                                                                            if isinstance(v, torch.Tensor)})
    return n


if __name__ == "__main__":
    main()
