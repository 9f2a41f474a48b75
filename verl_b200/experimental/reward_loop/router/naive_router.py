"""Round-robin HTTP proxy in front of several reward-model servers
(role of verl/experimental/reward_loop/router/naive_router.py:1-183)."""

from __future__ import annotations

import itertools
import threading
from typing import Optional


class NaiveRouter:
    def __init__(self, worker_urls: list[str], host: str = "127.0.0.1", port: int = 0, timeout_s: float = 600.0):
        if not worker_urls:
            raise ValueError("NaiveRouter needs at least one worker url")
        self.worker_urls = [u.rstrip("/") for u in worker_urls]
        self._rr = itertools.cycle(range(len(self.worker_urls)))
        self._lock = threading.Lock()
        self.host, self.port, self.timeout_s = host, port, timeout_s
        self._server = None
        self._thread: Optional[threading.Thread] = None

    def next_worker(self) -> str:
        with self._lock:
            return self.worker_urls[next(self._rr)]

    def build_app(self):
        import aiohttp
        from fastapi import FastAPI, Request, Response

        app = FastAPI()

        @app.get("/health")
        async def health():
            return {"status": "ok", "workers": len(self.worker_urls)}

        @app.api_route("/{path:path}", methods=["GET", "POST"])
        async def proxy(path: str, request: Request):
            url = f"{self.next_worker()}/{path}"
            body = await request.body()
            async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=self.timeout_s)) as sess:
                async with sess.request(request.method, url, data=body or None,
                                        headers={"content-type": request.headers.get("content-type", "application/json")}) as r:
                    return Response(content=await r.read(), status_code=r.status, media_type=r.headers.get("content-type"))

        return app

    def start(self) -> str:
        import socket

        import uvicorn

        if self.port == 0:
            with socket.socket() as s:
                s.bind((self.host, 0))
                self.port = s.getsockname()[1]
        self._server = uvicorn.Server(uvicorn.Config(self.build_app(), host=self.host, port=self.port, log_level="warning"))
        self._thread = threading.Thread(target=self._server.run, daemon=True)
        self._thread.start()
        return f"http://{self.host}:{self.port}"

    def stop(self):
        if self._server is not None:
            self._server.should_exit = True
        if self._thread is not None:
            self._thread.join(timeout=5)
