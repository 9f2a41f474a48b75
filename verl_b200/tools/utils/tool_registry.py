"""Build tool instances from a YAML list (verl/tools/utils/tool_registry.py):

    tools:
      - class_name: verl_b200.tools.gsm8k_tool.Gsm8kTool
        config: {type: native}
        tool_schema: {type: function, function: {name: calc_gsm8k_reward, ...}}
"""

from __future__ import annotations

import importlib
from enum import Enum

import yaml

from ..schemas import OpenAIFunctionToolSchema


class ToolType(Enum):
    NATIVE = "native"
    MCP = "mcp"


def get_tool_class(cls_name: str):
    mod, name = cls_name.rsplit(".", 1)
    if mod.startswith("verl."):
        mod = "verl_b200." + mod[len("verl."):]
    return getattr(importlib.import_module(mod), name)


def initialize_tools_from_config(tools_config_file: str) -> list:
    with open(tools_config_file) as f:
        conf = yaml.safe_load(f) or {}
    tools = []
    for tc in conf.get("tools", []):
        cls = get_tool_class(tc["class_name"])
        ttype = ToolType((tc.get("config") or {}).get("type", "native"))
        if ttype == ToolType.NATIVE:
            schema = OpenAIFunctionToolSchema.model_validate(tc["tool_schema"]) if tc.get("tool_schema") else None
            tools.append(cls(config=tc.get("config") or {}, tool_schema=schema))
        else:
            raise NotImplementedError("MCP tool servers need network access; register native tools instead")
    return tools
