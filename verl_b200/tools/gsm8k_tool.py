"""GSM8K answer-checking tool (verl/tools/gsm8k_tool.py): the model submits an answer, the tool scores it."""

from __future__ import annotations

from typing import Any, Optional
from uuid import uuid4

from ..utils.reward_score import gsm8k
from .base_tool import BaseTool
from .schemas import OpenAIFunctionToolSchema, ToolResponse


class Gsm8kTool(BaseTool):
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
        inst["response"] = answer if answer.startswith("#### ") else "#### " + answer
        reward = await self.calc_reward(instance_id)
        step = 0.0 if reward > inst["reward"] else -0.05  # penalise non-improving submissions
        inst["reward"] = reward
        return ToolResponse(text=f"Current parsed {answer=} {reward=}"), step, {}

    async def calc_reward(self, instance_id: str, **kwargs) -> float:
        inst = self._instances[instance_id]
        return float(gsm8k.compute_score(inst["response"], inst["ground_truth"], "flexible", 0.0, 1.0))

    async def release(self, instance_id: str, **kwargs) -> None:
        self._instances.pop(instance_id, None)
