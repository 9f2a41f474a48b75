"""Profiler configuration dataclasses (verl/utils/profiler/config.py:24-160)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from ...base_config import BaseConfig


@dataclass
class NsightToolConfig(BaseConfig):
    discrete: bool = False
    controller_nsight_options: Optional[dict] = None
    worker_nsight_options: Optional[dict] = None


@dataclass
class TorchProfilerToolConfig(BaseConfig):
    step_start: int = -1
    step_end: int = -1
    contents: list = field(default_factory=list)
    discrete: bool = False


@dataclass
class TorchMemoryToolConfig(BaseConfig):
    trace_alloc_max_entries: int = 100_000
    stack_depth: int = 32
    context: str = "all"
    stacks: str = "all"
    kw_args: dict = field(default_factory=dict)


@dataclass
class NPUToolConfig(NsightToolConfig):
    contents: list = field(default_factory=list)
    level: str = "level1"
    analysis: bool = False


@dataclass
class ProfilerConfig(BaseConfig):
    """Per-role profiler switch. ``union`` / ``intersect`` combine the configs of colocated roles."""

    tool: Optional[str] = None
    enable: bool = False
    all_ranks: bool = False
    ranks: list = field(default_factory=list)
    save_path: Optional[str] = "outputs/profile"
    tool_config: Any = None
    global_tool_config: Optional[Any] = None
    steps: Optional[list] = None
    profile_continuous_steps: bool = False

    def union(self, other: "ProfilerConfig") -> "ProfilerConfig":
        assert self.tool == other.tool, f"Cannot union ProfilerConfig with different tools: {self.tool} vs {other.tool}"
        return ProfilerConfig(tool=self.tool, enable=self.enable or other.enable,
                              all_ranks=self.all_ranks or other.all_ranks,
                              ranks=sorted(set(self.ranks or []) | set(other.ranks or [])), save_path=self.save_path,
                              tool_config=self.tool_config, global_tool_config=self.global_tool_config)

    def intersect(self, other: "ProfilerConfig") -> "ProfilerConfig":
        assert self.tool == other.tool, f"Cannot intersect ProfilerConfig with different tools: {self.tool} vs {other.tool}"
        return ProfilerConfig(tool=self.tool, enable=self.enable and other.enable,
                              all_ranks=self.all_ranks and other.all_ranks,
                              ranks=sorted(set(self.ranks or []) & set(other.ranks or [])), save_path=self.save_path,
                              tool_config=self.tool_config, global_tool_config=self.global_tool_config)
