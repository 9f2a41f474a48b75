"""Code-execution tool backed by a Sandbox-Fusion service, with a token-bucket limit on concurrent calls
(verl/tools/sandbox_fusion_tools.py)."""

from __future__ import annotations

import asyncio
import threading
from typing import Any, Optional
from uuid import uuid4

from ..utils.reward_score.sandbox_fusion import call_sandbox_api
from .base_tool import BaseTool
from .schemas import OpenAIFunctionToolSchema, ToolResponse


class TokenBucket:
    """Bounded number of in-flight executions shared by all tool instances."""

    def __init__(self, rate_limit: int):
        self._sem = threading.Semaphore(rate_limit)

    def acquire(self):
        self._sem.acquire()

    def release(self):
        self._sem.release()


class SandboxFusionTool(BaseTool):
    def __init__(self, config: dict, tool_schema: OpenAIFunctionToolSchema):
        super().__init__(config, tool_schema)
        self.url = config.get("sandbox_fusion_url", "")
        if not self.url:
            raise ValueError("sandbox_fusion_url is not set")
        self.default_timeout = config.get("default_timeout", 30)
        self.default_language = config.get("default_language", "python")
        self.memory_limit_mb = config.get("memory_limit_mb", 1024)
        self.bucket = TokenBucket(int(config.get("rate_limit", 10)))
        self._instances: dict = {}

    async def create(self, instance_id: Optional[str] = None, ground_truth: Optional[str] = None, **kwargs):
        instance_id = instance_id or str(uuid4())
        self._instances[instance_id] = {"ground_truth": ground_truth, "reward": []}
        return instance_id, ToolResponse()

    def _run(self, code: str, timeout: int, language: str) -> str:
        self.bucket.acquire()
        try:
            resp, err = call_sandbox_api(self.url, code, None, timeout, self.memory_limit_mb, language)
        finally:
            self.bucket.release()
        if err or resp is None:
            return f"no stdout here (sandbox error: {err})"
        run = resp.get("run_result") or {}
        if resp.get("status") == "Success":
            return (run.get("stdout") or "") + (run.get("stderr") or "")
        return "no stdout here"

    async def execute(self, instance_id: str, parameters: dict[str, Any], **kwargs):
        code = parameters.get("code", "")
        if not isinstance(code, str):
            code = str(code)
        out = await asyncio.get_event_loop().run_in_executor(
            None, self._run, code, parameters.get("timeout", self.default_timeout),
            parameters.get("language", self.default_language))
        return ToolResponse(text=out), 0.0, {}

    async def release(self, instance_id: str, **kwargs):
        self._instances.pop(instance_id, None)
