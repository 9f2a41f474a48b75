"""Model-Context-Protocol tools (verl/tools/mcp_base_tool.py, mcp_search_tool.py, utils/mcp_clients/): a tool whose
``execute`` forwards the call to an MCP server through ``McpClientManager``. The ``mcp`` / ``fastmcp`` client
packages are not part of this image; the manager raises a clear error at first use, and accepts an injected
``call_tool`` coroutine (which is also how the tests drive it)."""

from __future__ import annotations

import asyncio
import json
from typing import Any, Awaitable, Callable, Optional
from uuid import uuid4

from .base_tool import BaseTool
from .schemas import OpenAIFunctionToolSchema, ToolResponse


class McpClientManager:
    """Round-robin over configured MCP servers with a token-bucket rate limit (``rate_limit`` calls / second)."""

    def __init__(self):
        self.initialized = False
        self._call: Optional[Callable[[str, dict, float], Awaitable[Any]]] = None
        self._lock = asyncio.Lock()
        self._rate, self._tokens, self._last = 10.0, 10.0, None

    async def initialize(self, config_path: Optional[str] = None, rate_limit: float = 10.0,
                         call_tool: Optional[Callable] = None):
        self._rate = self._tokens = float(rate_limit)
        if call_tool is not None:
            self._call = call_tool
        else:
            try:
                import fastmcp  # noqa: F401
            except ImportError as e:
                raise RuntimeError("MCP tools need the 'fastmcp' client package, which is not installed") from e
            raise RuntimeError("no MCP server reachable from this process")
        self.initialized = True

    async def _acquire(self):
        loop = asyncio.get_running_loop()
        while True:
            async with self._lock:
                now = loop.time()
                self._last = now if self._last is None else self._last
                self._tokens = min(self._rate, self._tokens + (now - self._last) * self._rate)
                self._last = now
                if self._tokens >= 1:
                    self._tokens -= 1
                    return
                wait = (1 - self._tokens) / self._rate
            await asyncio.sleep(wait)

    async def call_tool(self, tool_name: str, parameters: dict, timeout: float = 30.0):
        if not self.initialized:
            raise RuntimeError("McpClientManager.initialize() has not been called")
        await self._acquire()
        return await asyncio.wait_for(self._call(tool_name, parameters, timeout), timeout)


ClientManager = McpClientManager()


class MCPBaseTool(BaseTool):
    def __init__(self, config: dict, tool_schema: OpenAIFunctionToolSchema):
        super().__init__(config, tool_schema)
        self._instances: dict[str, dict] = {}
        self.timeout = float(config.get("timeout", 30))

    async def create(self, instance_id: Optional[str] = None, **kwargs):
        instance_id = instance_id or str(uuid4())
        self._instances[instance_id] = {"response": "", "reward": []}
        return instance_id, ToolResponse()

    def _parse_tool_result(self, content) -> tuple[str, dict]:
        if isinstance(content, (dict, list)):
            return json.dumps(content, ensure_ascii=False), {}
        return str(content), {}

    async def execute(self, instance_id: str, parameters: dict[str, Any], **kwargs):
        if self.name == "" or self.name is None or parameters is None:
            return ToolResponse(text="Error: 'parameters' is missing or empty."), 0.0, {}
        try:
            raw = await ClientManager.call_tool(self.name, parameters, self.timeout)
            text, meta = self._parse_tool_result(raw)
            meta.update(api_request_error="", status="success")
        except Exception as e:
            text, meta = f"Tool call failed: {e}", {"api_request_error": str(e), "status": "error"}
        self._instances[instance_id]["reward"].append(text.strip())
        return ToolResponse(text=text), 0.0, meta

    async def calc_reward(self, instance_id: str, **kwargs):
        return self._instances[instance_id]["reward"]

    async def release(self, instance_id: str, **kwargs) -> None:
        self._instances.pop(instance_id, None)


class MCPSearchTool(MCPBaseTool):
    """MCP search servers answer with a list of content parts; the text parts' JSON payloads carry the hits under
    ``results`` (verl/tools/mcp_search_tool.py:25-69)."""

    def _parse_tool_result(self, content) -> tuple[str, dict]:
        parts = content if isinstance(content, list) else [content]
        hits, queries = [], []
        for part in parts:
            text = part.get("text") if isinstance(part, dict) else getattr(part, "text", None)
            if not text:
                continue
            try:
                body = json.loads(text)
            except (TypeError, ValueError):
                hits.append(str(text))
                continue
            queries.append(body.get("query", ""))
            res = body.get("results", body.get("result", []))
            hits.extend(str(r) for r in (res if isinstance(res, list) else [res]))
        meta = {"queries": queries, "query_count": len(queries), "total_results": len(hits)}
        return ("\n".join(hits) if hits else "no search result."), meta
