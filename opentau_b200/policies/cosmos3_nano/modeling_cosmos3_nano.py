"""cosmos3_nano policy class (8B backbone defaults)."""

from ..cosmos3.modeling_cosmos3 import Cosmos3Policy
from .configuration_cosmos3_nano import Cosmos3NanoConfig


class Cosmos3NanoPolicy(Cosmos3Policy):
    config_class = Cosmos3NanoConfig
    name = "cosmos3_nano"
