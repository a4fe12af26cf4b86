from .configuration_value import ValueConfig
from .modeling_value import ValueFunction, ValueModel

__all__ = ["ValueConfig", "ValueFunction", "ValueModel"]
