from .logging import IronCoreLogger, MLFlowLogger, TensorboardLogger
from .timers import DeviceTimer, Timer, get_memory_usage, profile_context, profile_function

__all__ = ["DeviceTimer", "IronCoreLogger", "MLFlowLogger", "TensorboardLogger", "Timer", "get_memory_usage",
           "profile_context", "profile_function"]
