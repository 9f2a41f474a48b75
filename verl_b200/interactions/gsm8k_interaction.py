"""GSM8K feedback interaction (verl/interactions/gsm8k_interaction.py): tells the model whether its last answer
is right and ends the conversation when it is."""

from __future__ import annotations

from typing import Any, Optional
from uuid import uuid4

from ..utils.reward_score import gsm8k
from .base import BaseInteraction


class Gsm8kInteraction(BaseInteraction):
    def __init__(self, config: dict):
        super().__init__(config)
        self._inst: dict = {}

    async def start_interaction(self, instance_id: Optional[str] = None, ground_truth: Optional[str] = None, **kwargs) -> str:
        instance_id = instance_id or str(uuid4())
        self._inst[instance_id] = {"response": "", "ground_truth": ground_truth, "reward": 0.0}
        return instance_id

    async def generate_response(self, instance_id: str, messages: list[dict[str, Any]], **kwargs):
        content = ""
        for m in reversed(messages):
            if m.get("role") == "assistant":
                content = m.get("content", "")
                break
        self._inst[instance_id]["response"] = content
        reward = await self.calculate_score(instance_id)
        if reward == 1.0:
            return True, "Your response is correct!", 1.0, {}
        return False, "Your response is incorrect! You need to reflect on your answer and try again.", 0.0, {}

    async def calculate_score(self, instance_id: str, **kwargs) -> float:
        i = self._inst[instance_id]
        return float(gsm8k.compute_score(i["response"], i["ground_truth"], "strict", 0.0, 1.0))

    async def finalize_interaction(self, instance_id: str, **kwargs) -> None:
        self._inst.pop(instance_id, None)
