from .configs import EnvConfig, FakeEnvConfig, LiberoEnvConfig, RoboCasaEnvConfig
from .factory import make_envs
from .fake import FakeRobotEnv, SyncVectorEnv
from .utils import add_envs_task, preprocess_observation

__all__ = ["EnvConfig", "FakeEnvConfig", "LiberoEnvConfig", "RoboCasaEnvConfig", "make_envs", "FakeRobotEnv",
           "SyncVectorEnv", "preprocess_observation", "add_envs_task"]
