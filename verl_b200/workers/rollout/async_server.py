"""Asynchronous token-in / token-out server around the native rollout engine.

Contract of the reference's ``vLLMHttpServer`` (verl/workers/rollout/vllm_rollout/vllm_async_server.py:445-682):
``generate(prompt_ids, sampling_params, request_id) -> TokenOutput`` as a coroutine, ``wake_up / sleep``,
``clear_kv_cache``, ``wait_for_requests_to_drain``, ``abort_all_requests`` (aborted requests still deliver their
partial output with ``stop_reason="aborted"``), ``abort_request``, ``start_profile / stop_profile``.

The engine steps in a dedicated thread; coroutines wait on futures that the step loop resolves. An optional
FastAPI app exposes ``/generate``, ``/health`` and an OpenAI-style ``/v1/completions`` for token ids.
"""

from __future__ import annotations

import asyncio
import threading
import time
import uuid
from concurrent.futures import Future
from typing import Any, Optional

from ...rollout import NativeRolloutEngine, SamplingParams, TokenOutput


class NativeAsyncServer:
    def __init__(self, engine: NativeRolloutEngine, response_length: int = 512, prompt_length: int = 512,
                 coalesce_ms: float = 20.0, tp_group=None):
        """``tp_group``: control group (gloo) of the ranks of a tensor-parallel replica. The first rank of the group is
        the leader: it takes the requests; every iteration of its engine thread broadcasts what it is about to do (new
        requests, aborts, wake-up / sleep / cache operations, whether to step) and the other ranks' engine threads do
        the same to their slice of the model, so that all schedulers stay identical and every ``step()`` is one
        collective forward of the replica (role of the rank-0 driver with tensor-parallel workers behind
        verl/workers/rollout/vllm_rollout/vllm_async_server.py)."""
        self.engine = engine
        self.tp_group = tp_group
        self.tp_leader = True
        self._tp_src = 0
        if tp_group is not None:
            import torch.distributed as dist

            ranks = dist.get_process_group_ranks(tp_group)
            self._tp_src = ranks[0]
            self.tp_leader = dist.get_rank() == ranks[0]
        self._ctrl: list = []  # engine operations queued for the engine thread (replica-wide under tensor parallelism)
        self.coalesce_s = float(coalesce_ms) / 1e3  # longest wait for the rest of a burst of new requests
        self.response_length, self.prompt_length = response_length, prompt_length
        self._lock = threading.Lock()
        self._pending: dict[str, Future] = {}
        self._inbox: list = []
        self._aborts: list[str] = []
        self._wake = threading.Event()
        self._stop = False
        self._paused = False
        self._idle = threading.Event()
        self._idle.set()
        self._thread = threading.Thread(target=self._loop, daemon=True, name="rollout-engine")
        self._thread.start()

    # ------------------------------------------------------------ engine thread
    def _loop(self):
        eng = self.engine
        if getattr(eng, "on_gpu", False):
            import torch

            torch.cuda.set_device(eng.device)  # the engine thread launches on the engine's GPU
        while True:
            if not self.tp_leader:
                # follower of a tensor-parallel replica: do what the leader announces
                cmd = self._bcast(None)
                if self._apply(cmd) == "stop":
                    return
                continue
            if self._stop:
                self._bcast({"stop": True})
                return
            with self._lock:
                inbox, self._inbox = self._inbox, []
                aborts, self._aborts = self._aborts, []
                ctrl, self._ctrl = self._ctrl, []
            if inbox:
                # Requests of one batch arrive within a few milliseconds of each other. Taking them in one go lets the
                # prefill see them together and the decode batch start at its full size, instead of growing through
                # every padded size (each of which would need its own CUDA graph after a wake-up).
                deadline = time.monotonic() + self.coalesce_s
                quiet = 0
                while time.monotonic() < deadline and quiet < 3:  # three quiet milliseconds end the burst
                    time.sleep(0.001)
                    with self._lock:
                        more, self._inbox = self._inbox, []
                    quiet = 0 if more else quiet + 1
                    inbox.extend(more)
            for name, args, done in ctrl:
                try:
                    if self.tp_group is not None:
                        self._bcast({"ctrl": [(name, args)]})
                    getattr(eng, name)(*args)
                    done.set_result(None)
                except Exception as e:
                    done.set_exception(e)
            if self.tp_group is not None and (inbox or aborts):
                self._bcast({"add": inbox, "abort": aborts})
            for rid, prompt, sp, mm in inbox:
                try:
                    eng.add_request(rid, prompt, sp, multi_modal_inputs=mm)
                except Exception as e:
                    fut = self._pending.pop(rid, None)
                    if fut is not None:
                        fut.set_exception(e)
            for rid in aborts:
                out = eng.abort_request(rid)
                fut = self._pending.pop(rid, None)
                if fut is not None and out is not None:
                    fut.set_result(out)
            if self._paused or not eng.has_unfinished():
                self._idle.set()
                self._wake.wait(timeout=0.05)
                self._wake.clear()
                continue
            self._idle.clear()
            try:
                if self.tp_group is not None:
                    self._bcast({"step": True})
                outs = eng.step()
            except Exception as e:  # fail every waiter rather than hang them
                with self._lock:
                    pend, self._pending = self._pending, {}
                for fut in pend.values():
                    if not fut.done():
                        fut.set_exception(e)
                eng.abort_all_requests()
                continue
            for o in outs:
                fut = self._pending.pop(o.request_id, None)
                if fut is not None and not fut.done():
                    fut.set_result(o)

    # ------------------------------------------------- tensor-parallel lockstep
    def _bcast(self, cmd):
        import torch.distributed as dist

        box = [cmd]
        dist.broadcast_object_list(box, src=self._tp_src, group=self.tp_group)
        return box[0]

    def _apply(self, cmd: dict):
        """A follower's side of one announcement."""
        eng = self.engine
        if cmd.get("stop"):
            return "stop"
        for name, args in cmd.get("ctrl", ()):
            getattr(eng, name)(*args)
        for rid, prompt, sp, mm in cmd.get("add", ()):
            try:
                eng.add_request(rid, prompt, sp, multi_modal_inputs=mm)
            except Exception:
                pass  # the leader saw the same error and failed the request
        for rid in cmd.get("abort", ()):
            eng.abort_request(rid)
        if cmd.get("step"):
            try:
                eng.step()
            except Exception:
                eng.abort_all_requests()  # as the leader does
        return None

    def _engine_op(self, name: str, *args):
        """Run an engine operation: directly without tensor parallelism, through the engine thread (and with it on
        every rank of the replica) otherwise."""
        if self.tp_group is None:
            getattr(self.engine, name)(*args)
            return None
        done: Future = Future()
        with self._lock:
            self._ctrl.append((name, args, done))
        self._wake.set()
        return done

    # ------------------------------------------------------------------ public
    def _multi_modal_inputs(self, image_data, video_data) -> Optional[dict]:
        """What a request brings for its vision placeholders (already expanded in ``prompt_ids``, one token per merged
        patch): a ``multi_modal_inputs`` dict of patches and grids as the datasets make them, or raw images / videos,
        which are cut into patches here with the model's geometry (role of the ``multi_modal_data`` that
        verl/workers/rollout/vllm_rollout/vllm_async_server.py:445-547 hands to the inference engine)."""
        if isinstance(image_data, dict) and ("pixel_values" in image_data or "pixel_values_videos" in image_data):
            return image_data
        if not image_data and not video_data:
            return None
        from ...utils.dataset.vision_utils import images_to_patches, videos_to_patches

        v = self.engine.full_cfg.extra.get("vision_config") or {}
        geo = (int(v.get("patch_size", 14)), int(v.get("spatial_merge_size", 2)), int(v.get("temporal_patch_size", 2)))
        mm = {}
        if image_data:
            mm["pixel_values"], mm["image_grid_thw"] = images_to_patches(list(image_data), *geo)
        if video_data:
            mm["pixel_values_videos"], mm["video_grid_thw"] = videos_to_patches(list(video_data), *geo)
        return mm

    def submit(self, prompt_ids: list[int], sampling_params: Optional[dict] = None, request_id: Optional[str] = None,
               multi_modal_inputs: Optional[dict] = None) -> Future:
        sp = dict(sampling_params or {})
        if "max_tokens" not in sp and "max_new_tokens" not in sp:
            sp["max_tokens"] = self.response_length + self.prompt_length - len(prompt_ids)
        max_new = sp.get("max_tokens", sp.get("max_new_tokens"))
        sp["max_tokens"] = max(0, min(int(max_new), self.engine.max_model_len - len(prompt_ids)))
        sp.pop("max_new_tokens", None)
        rid = request_id or uuid.uuid4().hex
        fut: Future = Future()
        with self._lock:
            self._pending[rid] = fut
            self._inbox.append((rid, list(prompt_ids), SamplingParams.from_dict(sp), multi_modal_inputs))
        self._wake.set()
        return fut

    async def generate(self, prompt_ids: list[int], sampling_params: Optional[dict] = None, request_id: Optional[str] = None,
                       image_data=None, video_data=None, priority: int = 0) -> TokenOutput:
        fut = self.submit(prompt_ids, sampling_params, request_id, self._multi_modal_inputs(image_data, video_data))
        return await asyncio.wrap_future(fut)

    async def abort_request(self, request_id: str, reset_prefix_cache: bool = False) -> dict[str, Any]:
        known = request_id in self._pending
        with self._lock:
            self._aborts.append(request_id)
        self._wake.set()
        return {"aborted": known, "request_id": request_id}

    async def abort_all_requests(self, reset_prefix_cache: bool = True) -> dict[str, Any]:
        with self._lock:
            ids = list(self._pending.keys())
            self._aborts.extend(ids)
        self._wake.set()
        await self.wait_for_requests_to_drain()
        if reset_prefix_cache:
            self.engine.clear_kv_cache()
        return {"aborted_count": len(ids), "request_ids": ids}

    async def wait_for_requests_to_drain(self, timeout: float = 600.0):
        t0 = time.monotonic()
        while (self._pending or self._inbox) and time.monotonic() - t0 < timeout:
            await asyncio.sleep(0.005)

    async def resume_all_requests(self):
        self._paused = False
        self._wake.set()

    async def pause(self):
        self._paused = True

    async def wake_up(self, tags: Optional[list[str]] = None):
        fut = self._engine_op("wake_up", tags)
        if fut is not None:
            await asyncio.wrap_future(fut)

    async def sleep(self):
        await self.wait_for_requests_to_drain()
        self._idle.wait(5.0)
        fut = self._engine_op("sleep")
        if fut is not None:
            await asyncio.wrap_future(fut)

    async def clear_kv_cache(self):
        fut = self._engine_op("clear_kv_cache")
        if fut is not None:
            await asyncio.wrap_future(fut)

    async def start_profile(self, **kwargs):
        import torch

        if torch.cuda.is_available():
            torch.cuda.profiler.start()

    async def stop_profile(self):
        import torch

        if torch.cuda.is_available():
            torch.cuda.profiler.stop()

    def shutdown(self):
        self._stop = True
        self._wake.set()
        self._thread.join(2.0)

    # ------------------------------------------------------------------- HTTP
    def build_app(self):
        """FastAPI app with token-level endpoints (served with uvicorn by :func:`run_unvicorn`)."""
        from fastapi import FastAPI

        app = FastAPI()
        server = self

        @app.get("/health")
        async def health():
            return {"status": "ok", **server.engine.sched.stats()} if server.engine.sched else {"status": "sleeping"}

        @app.post("/generate")
        async def generate(body: dict):
            out = await server.generate(body["prompt_ids"], body.get("sampling_params"), body.get("request_id"),
                                        image_data=_decode_tensors(body.get("multi_modal_inputs")))
            res = {"token_ids": out.token_ids, "log_probs": out.log_probs, "stop_reason": out.stop_reason,
                   "num_preempted": out.num_preempted}
            if out.routed_experts is not None:  # int16 [tokens, layers, top-k], as bytes
                import base64

                import numpy as np

                rec = np.ascontiguousarray(out.routed_experts, dtype=np.int16)
                res["routed_experts"] = {"shape": list(rec.shape), "data": base64.b64encode(rec.tobytes()).decode("ascii")}
            return res

        @app.post("/v1/completions")
        async def completions(body: dict):
            prompt = body["prompt"]
            assert isinstance(prompt, list), "prompt must be a list of token ids"
            sp = {"temperature": body.get("temperature", 1.0), "top_p": body.get("top_p", 1.0),
                  "max_tokens": body.get("max_tokens", 16), "logprobs": bool(body.get("logprobs"))}
            out = await server.generate(prompt, sp)
            return {"id": f"cmpl-{uuid.uuid4().hex}", "object": "text_completion",
                    "choices": [{"index": 0, "token_ids": out.token_ids, "logprobs": out.log_probs,
                                 "finish_reason": "stop" if out.stop_reason == "completed" else "length"}]}

        @app.post("/abort_request")
        async def abort(body: dict):
            return await server.abort_request(body["request_id"])

        @app.post("/wake_up")
        async def wake_up():
            await server.wake_up()
            return {"ok": True}

        @app.post("/sleep")
        async def sleep():
            await server.sleep()
            return {"ok": True}

        @app.post("/abort_all_requests")
        async def abort_all(body: dict):
            return await server.abort_all_requests(bool(body.get("reset_prefix_cache", True)))

        @app.post("/resume_all_requests")
        async def resume_all():
            await server.resume_all_requests()
            return {"ok": True}

        @app.post("/clear_kv_cache")
        async def clear_cache():
            await server.clear_kv_cache()
            return {"ok": True}

        @app.get("/metrics")
        async def metrics():
            """Prometheus text exposition of the scheduler gauges (scraped by the job that
            ``update_prometheus_config`` writes)."""
            from fastapi.responses import PlainTextResponse

            stats = server.engine.sched.stats() if server.engine.sched else {}
            stats["pending_requests"] = len(server._pending)
            lines = []
            for k, v in stats.items():
                if isinstance(v, (int, float)):
                    lines += [f"# TYPE verl_rollout_{k} gauge", f"verl_rollout_{k} {v}"]
            return PlainTextResponse("\n".join(lines) + "\n", media_type="text/plain; version=0.0.4")

        return app


from .utils import run_unvicorn  # noqa: E402,F401  (historical import location)


def _encode_tensors(d: Optional[dict]) -> Optional[dict]:
    """Tensors of a ``multi_modal_inputs`` dict as JSON fields (dtype, shape, base64 bytes)."""
    if d is None:
        return None
    import base64

    import torch

    out = {}
    for k, t in d.items():
        t = torch.as_tensor(t).contiguous().cpu()
        out[k] = {"dtype": str(t.dtype).replace("torch.", ""), "shape": list(t.shape),
                  "data": base64.b64encode(t.numpy().tobytes()).decode("ascii")}
    return out


def _decode_tensors(d: Optional[dict]) -> Optional[dict]:
    if d is None:
        return None
    import base64

    import numpy as np
    import torch

    return {k: torch.from_numpy(np.frombuffer(base64.b64decode(v["data"]), dtype=np.dtype(v["dtype"])).reshape(v["shape"]).copy())
            for k, v in d.items()}


def serve_in_thread(server: NativeAsyncServer, address: str = "127.0.0.1") -> str:
    """Serve ``server.build_app()`` from a background thread of this process (its own event loop); returns
    ``host:port``. Used by worker processes, whose main thread belongs to the worker group's command loop."""
    box: dict = {}
    ready = threading.Event()

    def run():
        async def main():
            port, task = await run_unvicorn(server.build_app(), None, address)
            box["port"], box["task"] = port, task
            ready.set()
            await task

        try:
            asyncio.run(main())
        except BaseException as e:  # surface start-up failures to the caller
            box["error"] = e
            ready.set()

    t = threading.Thread(target=run, daemon=True, name="rollout-http")
    t.start()
    ready.wait(60)
    if "error" in box or "port" not in box:
        raise RuntimeError(f"rollout HTTP server did not start: {box.get('error')}")
    server._http_thread, server._http_task = t, box["task"]
    return f"{address}:{box['port']}"


class HttpServerHandle:
    """Client-side handle of a :class:`NativeAsyncServer` in another process: the coroutine interface the agent
    loops use, carried over the server's HTTP endpoints."""

    def __init__(self, address: str, timeout: float = 3600.0):
        self.address, self.timeout = address, timeout
        self._session = None

    async def _post(self, path: str, body: Optional[dict] = None) -> dict:
        import aiohttp

        # one session per event loop (the agent-loop manager runs a fresh loop per batch)
        loop = asyncio.get_running_loop()
        if self._session is None or self._session[0] is not loop or self._session[1].closed:
            self._session = (loop, aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=self.timeout)))
        async with self._session[1].post(f"http://{self.address}{path}", json=body or {}) as resp:
            resp.raise_for_status()
            return await resp.json()

    async def generate(self, prompt_ids: list[int], sampling_params: Optional[dict] = None, request_id: Optional[str] = None,
                       image_data=None, video_data=None, priority: int = 0) -> TokenOutput:
        sp = {k: v for k, v in (sampling_params or {}).items() if isinstance(v, (int, float, bool, str, list, type(None)))}
        req = {"prompt_ids": [int(t) for t in prompt_ids], "sampling_params": sp, "request_id": request_id}
        if image_data is not None or video_data is not None:
            if not (isinstance(image_data, dict) and video_data is None):
                raise NotImplementedError("over HTTP the vision inputs travel as a multi_modal_inputs dict of patches and "
                                          "grids (VLProcessor / the datasets make it); raw images stay in-process")
            req["multi_modal_inputs"] = _encode_tensors(image_data)
        body = await self._post("/generate", req)
        routed = body.get("routed_experts")
        if routed is not None:
            import base64

            import numpy as np

            routed = np.frombuffer(base64.b64decode(routed["data"]), dtype=np.int16).reshape(routed["shape"]).copy()
        return TokenOutput(token_ids=body["token_ids"], log_probs=body.get("log_probs"), routed_experts=routed,
                           stop_reason=body.get("stop_reason"), num_preempted=int(body.get("num_preempted", 0) or 0),
                           request_id=request_id)

    async def abort_request(self, request_id: str, reset_prefix_cache: bool = False):
        return await self._post("/abort_request", {"request_id": request_id})

    async def abort_all_requests(self, reset_prefix_cache: bool = True):
        return await self._post("/abort_all_requests", {"reset_prefix_cache": reset_prefix_cache})

    async def resume_all_requests(self):
        return await self._post("/resume_all_requests")

    async def wake_up(self, tags=None):
        return await self._post("/wake_up")

    async def sleep(self):
        return await self._post("/sleep")

    async def clear_kv_cache(self):
        return await self._post("/clear_kv_cache")

    async def close(self):
        if self._session is not None and not self._session[1].closed:
            await self._session[1].close()
