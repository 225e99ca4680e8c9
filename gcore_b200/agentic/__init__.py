from .envs import ENV_REGISTRY, FrozenLakeEnv, SimpleAgenticEnv, SokobanEnv, make_env  # noqa: F401
from .parsers import ToolCall, ToolReasonEnvWrapper, ToolRegistry, parse_tool_calls, split_reasoning  # noqa: F401
from .traj_env_manager import TrajEnvManager, conversation_to_tokens_and_mask  # noqa: F401
