"""Retrieval tool calling an HTTP search service (verl/tools/search_tool.py, utils/search_r1_like_utils.py)."""

from __future__ import annotations

import asyncio
import json
from typing import Any, Optional
from uuid import uuid4

from .base_tool import BaseTool
from .schemas import OpenAIFunctionToolSchema, ToolResponse


from .utils.search_r1_like_utils import perform_single_search_batch  # noqa: E402


class SearchTool(BaseTool):
    def __init__(self, config: dict, tool_schema: OpenAIFunctionToolSchema):
        super().__init__(config, tool_schema)
        self.url = config.get("retrieval_service_url")
        assert self.url, "Configuration must include 'retrieval_service_url'"
        self.topk = config.get("topk", 3)
        self.timeout = config.get("timeout", 30)
        self._sem = asyncio.Semaphore(int(config.get("rate_limit", 120)))
        self._instances: dict = {}

    async def create(self, instance_id: Optional[str] = None, **kwargs):
        instance_id = instance_id or str(uuid4())
        self._instances[instance_id] = {"reward": []}
        return instance_id, ToolResponse()

    async def execute(self, instance_id: str, parameters: dict[str, Any], **kwargs):
        queries = parameters.get("query_list")
        if not isinstance(queries, list) or not queries:
            return ToolResponse(text=json.dumps({"result": "Error: 'query_list' is missing, empty, or not a list in parameters."})), 0.0, {}
        async with self._sem:
            text, meta = await asyncio.get_event_loop().run_in_executor(
                None, lambda: perform_single_search_batch(self.url, queries, self.topk, None, self.timeout,
                                                          max_retries=int(self.config.get("max_retries", 3))))
        return ToolResponse(text=text), 0.0, meta

    async def release(self, instance_id: str, **kwargs):
        self._instances.pop(instance_id, None)
