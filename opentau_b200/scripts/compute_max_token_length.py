"""Scan a dataset mixture for the longest prompt / response / discrete-action token sequences, to size
``prompt_max_length`` & co. without truncation (reference ``src/opentau/scripts/compute_max_token_length.py``)."""

from __future__ import annotations

import json
import logging

import numpy as np

from ..configs import parser
from ..configs.train import TrainPipelineConfig


def scan(mixture, tokenizer, action_tokenizer=None, max_samples: int = 2000, seed: int = 0) -> dict:
    rng = np.random.default_rng(seed)
    idx = rng.choice(len(mixture), size=min(max_samples, len(mixture)), replace=False)
    lens: dict[str, list[int]] = {"prompt": [], "response": [], "discrete_actions": []}
    for i in idx:
        it = mixture.get_global(int(i))
        for key in ("prompt", "response"):
            if it.get(key):
                lens[key].append(len(tokenizer.encode(it[key])))
        if action_tokenizer is not None and not bool(it["action_is_pad"].all()):
            lens["discrete_actions"].append(len(action_tokenizer(it["actions"].float()[None])[0]))
    return {k: {"max": int(max(v)), "p99": float(np.percentile(v, 99)), "mean": float(np.mean(v)), "n": len(v)}
            for k, v in lens.items() if v}


@parser.wrap()
def main(cfg: TrainPipelineConfig):
    from ..datasets.factory import make_dataset_mixture
    from ..utils.logging_utils import init_logging
    from ..utils.tokenizer import load_action_tokenizer, load_text_tokenizer
    init_logging()
    res = make_dataset_mixture(cfg)
    mix = res[0] if isinstance(res, tuple) else res
    tok = load_text_tokenizer(getattr(cfg.policy, "tokenizer_path", ""), 257152)
    atok = load_action_tokenizer(getattr(cfg.policy, "discrete_action_tokenizer_path", ""),
                                 getattr(cfg.policy, "discrete_action_vocab_size", 2048))
    out = scan(mix, tok, atok)
    logging.info("token lengths: %s", out)
    print(json.dumps(out, indent=2))
    return out


if __name__ == "__main__":
    main()
