from .config import NPUToolConfig, NsightToolConfig, ProfilerConfig, TorchMemoryToolConfig, TorchProfilerToolConfig

__all__ = ["ProfilerConfig", "NsightToolConfig", "TorchProfilerToolConfig", "TorchMemoryToolConfig", "NPUToolConfig"]
