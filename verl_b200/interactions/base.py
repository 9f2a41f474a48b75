"""Interaction interface for multi-turn user simulation (verl/interactions/base.py)."""

from __future__ import annotations

from typing import Any, Optional
from uuid import uuid4


class BaseInteraction:
    def __init__(self, config: dict[str, Any]):
        self.config = config
        self.name: str = config.get("name", "interaction_agent")

    async def start_interaction(self, instance_id: Optional[str] = None, **kwargs) -> str:
        return instance_id or str(uuid4())

    async def generate_response(self, instance_id: str, messages: list[dict[str, Any]], **kwargs) -> tuple[bool, str, float, dict]:
        """Returns (should_terminate_sequence, response text, turn score, extra data)."""
        return False, "Your current result seems acceptable.", 0.0, {}

    async def calculate_score(self) -> float:
        return 0.0

    async def finalize_interaction(self) -> None:
        pass
