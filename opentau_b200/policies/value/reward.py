"""Sparse-reward returns for the value model (reference ``src/opentau/policies/value/reward.py:24-91``).

Every step costs -1; the return at step ``t`` of an episode whose exclusive end index is ``e`` is ``t - e + 1`` (0 at the last
step), and a failed episode additionally pays ``c_neg``.
"""

from __future__ import annotations


def calculate_return_bins_with_equal_width(success: bool, b: int, episode_end_idx: int, reward_normalizer: int,
                                           current_idx: int, c_neg: float = -100.0) -> tuple[int, float]:
    """``(bin_idx, normalised_return)``: the return scaled to [-1, 0] and its index among ``b`` equal bins."""
    ret = current_idx - episode_end_idx + 1
    if not success:
        ret = ret + c_neg
    ret_norm = ret / reward_normalizer
    bin_idx = int((ret_norm + 1) * (b - 1))
    return bin_idx, ret_norm


def calculate_n_step_return(success: bool, n_steps_look_ahead: int, episode_end_idx: int, reward_normalizer: int,
                            current_idx: int, c_neg: float = -100.0) -> float:
    """Normalised reward accumulated over the next ``n_steps_look_ahead`` steps (clipped at the episode end);
    the failure penalty is included only when the episode ends inside the look-ahead window."""
    ret = max(current_idx - episode_end_idx + 1, -n_steps_look_ahead)
    if not success and current_idx + n_steps_look_ahead >= episode_end_idx:
        ret = ret + c_neg
    return ret / reward_normalizer
