"""pi0.7 low-level controller on PaliGemma (reference
``src/opentau/policies/pi07_paligemma/low_level/modeling_pi07_low_level.py``): same prefix layout, branch
synchronisation, losses and sampler as the Gemma-3 controller; the backbone pair is
``model.paligemma_with_expert.*`` and the attention is the shared block-causal kernel (the reference's legacy
consumer of its WMMA flash kernel)."""

from __future__ import annotations

from ...pi05.modeling_pi05 import PaliGemmaWithExpertModel, gemma_2b_config
from ...pi07.low_level.modeling_pi07_low_level import PI07LowLevelFlowMatching, PI07LowLevelPolicy
from .configuration_pi07_low_level import PI07PaligemmaLowLevelConfig


class PI07PaligemmaLowLevelFlowMatching(PI07LowLevelFlowMatching):
    wrapper_attr = "paligemma_with_expert"

    def build_wrapper(self, config):
        return PaliGemmaWithExpertModel(config)

    def _tower(self):
        return self.wrapper.paligemma.vision_tower

    def _projector(self):
        return self.wrapper.paligemma.model.multi_modal_projector


class PI07PaligemmaLowLevelPolicy(PI07LowLevelPolicy):
    config_class = PI07PaligemmaLowLevelConfig
    name = "pi07_paligemma_low_level"
    model_class = PI07PaligemmaLowLevelFlowMatching

    @staticmethod
    def _vocab_size(config) -> int:
        return gemma_2b_config(**(config.vlm or {})).vocab_size

    @classmethod
    def _fix_state_dict_keys(cls, state, config):
        """Checkpoints written by the Gemma-3 code path under the legacy name are mapped back."""
        state = super()._fix_state_dict_keys(state, config)
        return {k.replace("model.gemma3_with_expert.", "model.paligemma_with_expert."): v for k, v in state.items()}
