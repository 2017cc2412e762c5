"""Small shared helpers: environment flags, timers, clock sampling."""
from .env import env_flag, env_flag_enabled, env_int, env_str
from .timing import CudaTimer, PhaseTimer, nvtx_range

__all__ = [
    "env_flag", "env_flag_enabled", "env_int", "env_str",
    "CudaTimer", "PhaseTimer", "nvtx_range",
]
