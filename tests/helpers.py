"""Shared builders for tiny models used across the test-suite."""

import torch

from opentau_b200.configs.types import FeatureType, PolicyFeature
from opentau_b200.datasets.synthetic import SyntheticSpec, identity_stats, make_synthetic_batch
from opentau_b200.policies.pi05.configuration_pi05 import PI05Config
from opentau_b200.policies.pi05.modeling_pi05 import PI05Policy

TINY = dict(
    vlm=dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1, head_dim=64,
             intermediate_size=1024, vocab_size=1024),
    expert=dict(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1, head_dim=64,
                intermediate_size=512, vocab_size=1024),
    vision=dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4, patch_size=14,
                image_size=224),
)


def tiny_pi05_config(device="cpu", **over) -> PI05Config:
    feats = {"camera0": PolicyFeature(FeatureType.VISUAL, (3, 224, 224)),
             "state": PolicyFeature(FeatureType.STATE, (32,))}
    kw = dict(chunk_size=10, n_action_steps=10, prompt_max_length=16, discrete_action_max_length=8,
              discrete_action_vocab_size=256, dropout=0.0, device=device, input_features=feats,
              output_features={"actions": PolicyFeature(FeatureType.ACTION, (32,))}, **TINY)
    kw.update(over)
    return PI05Config(**kw)


def tiny_pi05(device="cpu", seed=0, **over) -> PI05Policy:
    torch.manual_seed(seed)
    return PI05Policy(tiny_pi05_config(device, **over), per_dataset_stats=[identity_stats()])


def tiny_batch(device="cpu", seed=1, **over):
    return make_synthetic_batch(SyntheticSpec(**over), device=device, seed=seed)


def free_port() -> int:
    """A TCP port that is free right now on the loopback interface (the kernel picks it), for rendezvous in
    multi-process tests: a port derived from the pid can collide with another process or an earlier test."""
    import socket
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as sk:
        sk.bind(("127.0.0.1", 0))
        return sk.getsockname()[1]
