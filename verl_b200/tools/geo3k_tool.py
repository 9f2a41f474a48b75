"""Geometry3K answer-checking tool (verl/tools/geo3k_tool.py): like the GSM8K tool with the geo3k scorer."""

from __future__ import annotations

from typing import Any, Optional
from uuid import uuid4

from ..utils.reward_score import geo3k
from .base_tool import BaseTool
from .schemas import OpenAIFunctionToolSchema, ToolResponse


class Geo3kTool(BaseTool):
    def __init__(self, config: dict, tool_schema: OpenAIFunctionToolSchema):
        super().__init__(config, tool_schema)
        self._instances: dict[str, dict] = {}

    async def create(self, instance_id: Optional[str] = None, ground_truth: Optional[str] = None, **kwargs):
        instance_id = instance_id or str(uuid4())
        if ground_truth is None:
            ground_truth = (kwargs.get("create_kwargs") or {}).get("ground_truth")
        self._instances[instance_id] = {"response": "", "ground_truth": ground_truth, "reward": 0.0}
        return instance_id, ToolResponse()

    async def execute(self, instance_id: str, parameters: dict[str, Any], **kwargs):
        answer = str(parameters.get("answer", ""))
        inst = self._instances[instance_id]
        inst["response"] = answer
        reward = await self.calc_reward(instance_id)
        step = 0.0 if reward > inst["reward"] else -0.05
        inst["reward"] = reward
        return ToolResponse(text=f"Current parsed {answer=} {reward=}"), step, {}

    async def calc_reward(self, instance_id: str, **kwargs) -> float:
        inst = self._instances[instance_id]
        return float(geo3k.compute_score(inst["response"], inst["ground_truth"], use_boxed=False, format_score=0.0))

    async def release(self, instance_id: str, **kwargs) -> None:
        self._instances.pop(instance_id, None)
