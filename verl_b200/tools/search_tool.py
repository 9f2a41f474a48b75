"""Retrieval tool calling an HTTP search service (verl/tools/search_tool.py, utils/search_r1_like_utils.py)."""

from __future__ import annotations

import asyncio
import json
from typing import Any, Optional
from uuid import uuid4

from .base_tool import BaseTool
from .schemas import OpenAIFunctionToolSchema, ToolResponse


def _passages_to_string(result: list[dict]) -> str:
    out = []
    for i, doc in enumerate(result):
        content = doc.get("document", {}).get("contents", "") if isinstance(doc.get("document"), dict) else str(doc)
        title, _, text = content.partition("\n")
        out.append(f"Doc {i + 1} (Title: {title})\n{text}\n")
    return "\n".join(out)


def perform_single_search_batch(retrieval_service_url: str, query_list: list[str], topk: int = 3, timeout: int = 30):
    import requests

    payload = {"queries": query_list, "topk": topk, "return_scores": True}
    last = None
    for attempt in range(3):
        try:
            r = requests.post(retrieval_service_url, json=payload, timeout=timeout)
            r.raise_for_status()
            results = r.json().get("result", [])
            text = "\n---\n".join(_passages_to_string(x) for x in results)
            return json.dumps({"result": text}, ensure_ascii=False), {"status": "success", "total_results": sum(len(x) for x in results)}
        except Exception as e:
            last = e
    return json.dumps({"result": f"Search error: {last}"}), {"status": "error"}


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
                None, perform_single_search_batch, self.url, queries, self.topk, self.timeout)
        return ToolResponse(text=text), 0.0, meta

    async def release(self, instance_id: str, **kwargs):
        self._instances.pop(instance_id, None)
