from .configuration_pi05_mem import PI05MemConfig
from .modeling_pi05_mem import PI05MemFlowMatching, PI05MemPolicy

__all__ = ["PI05MemConfig", "PI05MemFlowMatching", "PI05MemPolicy"]
