"""Weather-assistant interaction (verl/interactions/weather_interaction.py): a scripted user who checks that the
assistant's last reply mentions weather information and otherwise asks again."""

from __future__ import annotations

from typing import Any, Optional
from uuid import uuid4

from .base import BaseInteraction


class WeatherInteraction(BaseInteraction):
    KEYWORDS = ("weather", "temperature", "forecast", "rain", "sunny", "cloud", "°")

    def __init__(self, config: dict):
        super().__init__(config)
        self._inst: dict = {}

    async def start_interaction(self, instance_id: Optional[str] = None, **kwargs) -> str:
        instance_id = instance_id or str(uuid4())
        self._inst[instance_id] = {"response": "", "reward": 0.0}
        return instance_id

    async def generate_response(self, instance_id: str, messages: list[dict[str, Any]], **kwargs):
        content = next((m.get("content", "") for m in reversed(messages) if m.get("role") == "assistant"), "")
        self._inst[instance_id]["response"] = content
        reward = await self.calculate_score(instance_id)
        if reward > 0.5:
            return True, "Thank you for providing the weather information!", 1.0, {}
        return False, "Please use the weather tool to get current weather information first.", 0.0, {}

    async def calculate_score(self, instance_id: str, **kwargs) -> float:
        text = str(self._inst[instance_id]["response"]).lower()
        return 1.0 if any(k in text for k in self.KEYWORDS) else 0.0

    async def finalize_interaction(self, instance_id: str, **kwargs) -> None:
        self._inst.pop(instance_id, None)
