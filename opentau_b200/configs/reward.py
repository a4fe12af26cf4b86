"""Reward settings of the value model and advantage pipeline (reference ``src/opentau/configs/reward.py:24-45``)."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class RewardConfig:
    number_of_bins: int = 201        # value head classes over the normalised return range [-1, 0]
    C_neg: float = -1000.0           # added to the return of failed episodes
    reward_normalizer: int = 400     # episode-length scale that maps returns into [-1, 0]
    N_steps_look_ahead: int = 50     # horizon of the n-step return used for advantages
