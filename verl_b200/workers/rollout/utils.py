"""Rollout server helpers (verl/workers/rollout/utils.py:26-70)."""

from __future__ import annotations

import asyncio
import logging

from ...utils.net_utils import get_free_port

logger = logging.getLogger(__name__)


def get_max_position_embeddings(hf_config) -> int:
    max_len = getattr(hf_config, "max_position_embeddings", None)
    if max_len is None and getattr(hf_config, "text_config", None) is not None:
        max_len = getattr(hf_config.text_config, "max_position_embeddings", None)
    if max_len is None:
        raise ValueError("max_position_embeddings not found in the model config")
    return int(max_len)


async def run_unvicorn(app, server_args, server_address: str, max_retries: int = 5):
    """Start ``app`` under uvicorn on a free port of ``server_address``, retrying when the port was taken between
    the probe and the bind. Returns (port, serving task). (The misspelt name is the reference's public one.)"""
    import uvicorn

    last = None
    for attempt in range(max_retries):
        port = get_free_port(server_address)
        try:
            app.server_args = server_args
            server = uvicorn.Server(uvicorn.Config(app, host=server_address, port=int(port), log_level="warning"))
            task = asyncio.create_task(server.serve())
            for _ in range(200):
                if server.started or task.done():
                    break
                await asyncio.sleep(0.01)
            if task.done():
                task.result()
                raise OSError("server exited during start-up")
            task.server = server
            return int(port), task
        except (OSError, SystemExit) as e:
            last = e
            logger.error("failed to start HTTP server on port %s at try %d: %s", port, attempt, e)
    raise RuntimeError(f"could not start the HTTP server after {max_retries} tries: {last}")


async def ensure_async_iterator(iterable):
    if hasattr(iterable, "__aiter__"):
        async for item in iterable:
            yield item
    else:
        for item in iterable:
            yield item
