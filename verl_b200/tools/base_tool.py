"""Tool interface (verl/tools/base_tool.py:24): ``create -> execute* -> calc_reward -> release`` per trajectory."""

from __future__ import annotations

import json
from typing import Any, Optional
from uuid import uuid4

from .schemas import OpenAIFunctionToolSchema, ToolResponse


class BaseTool:
    def __init__(self, config: dict, tool_schema: OpenAIFunctionToolSchema):
        self.config = config
        self.tool_schema = tool_schema or self.get_openai_tool_schema()
        assert self.tool_schema is not None, "Tool schema is not set!"
        self.name = self.tool_schema.function.name

    def get_openai_tool_schema(self) -> OpenAIFunctionToolSchema:
        return self.tool_schema

    async def create(self, instance_id: Optional[str] = None, **kwargs) -> tuple[str, ToolResponse]:
        return (instance_id or str(uuid4())), ToolResponse()

    async def execute(self, instance_id: str, parameters: dict[str, Any], **kwargs) -> tuple[ToolResponse, float, dict]:
        """Returns (tool response, step reward, metrics)."""
        return ToolResponse(text="Updated the tool state."), 0.0, {}

    async def calc_reward(self, instance_id: str, **kwargs) -> float:
        return 0.0

    async def release(self, instance_id: str, **kwargs) -> None:
        pass
