"""Rollout tracing (role of verl/utils/rollout_trace.py:29-257): ``rollout_trace_op`` decorates async agent-loop
steps and reports their inputs / outputs to a tracing backend; ``rollout_trace_attr`` sets the attributes of the
enclosing trajectory (step, sample index, rollout number, validate flag). The backends of the reference (weave,
mlflow) need network services; ``file`` writes one JSON line per op, ``None`` disables tracing."""

from __future__ import annotations

import contextlib
import contextvars
import functools
import inspect
import json
import os
import threading
import time
from typing import Optional

_ATTRS: contextvars.ContextVar = contextvars.ContextVar("rollout_trace_attrs", default=None)


class RolloutTraceConfig:
    _instance: Optional["RolloutTraceConfig"] = None
    _lock = threading.Lock()

    def __init__(self):
        self.backend: Optional[str] = None
        self.token2text = False
        self.project_name = self.experiment_name = None
        self.path: Optional[str] = None
        self.max_samples_per_step_per_worker: Optional[int] = None

    @classmethod
    def get_instance(cls) -> "RolloutTraceConfig":
        with cls._lock:
            if cls._instance is None:
                cls._instance = cls()
            return cls._instance

    @classmethod
    def init(cls, project_name: str, experiment_name: str, backend: Optional[str], token2text: bool = False,
             max_samples_per_step_per_worker: Optional[int] = None, path: Optional[str] = None):
        c = cls.get_instance()
        if backend in ("weave", "mlflow"):
            print(f"[rollout_trace] backend {backend!r} needs a tracking service that this process cannot reach; using 'file'")
            backend = "file"
        if backend not in (None, "file"):
            raise ValueError(f"Unknown rollout trace backend: {backend}")
        c.backend, c.token2text, c.project_name, c.experiment_name = backend, token2text, project_name, experiment_name
        c.max_samples_per_step_per_worker = max_samples_per_step_per_worker
        c.path = path or os.path.join(os.environ.get("VERL_ROLLOUT_TRACE_DIR", "rollout_trace"), f"{project_name}_{experiment_name}.jsonl")
        return c

    @classmethod
    def get_backend(cls):
        return cls.get_instance().backend

    @classmethod
    def enable_token2text(cls) -> bool:
        return cls.get_instance().token2text

    @classmethod
    def reset(cls):
        cls._instance = None


@contextlib.contextmanager
def rollout_trace_attr(sample_index=None, step=None, rollout_n=None, name="rollout_trace", validate=False, trace: bool = True):
    tok = _ATTRS.set({"sample_index": sample_index, "step": step, "rollout_n": rollout_n, "name": name, "validate": validate,
                      "trace": trace} if RolloutTraceConfig.get_backend() else None)
    try:
        yield
    finally:
        _ATTRS.reset(tok)


def _jsonable(v, depth=0):
    if depth > 3:
        return str(type(v).__name__)
    if isinstance(v, (str, int, float, bool)) or v is None:
        return v
    if isinstance(v, (list, tuple)):
        return [_jsonable(x, depth + 1) for x in v[:64]]
    if isinstance(v, dict):
        return {str(k): _jsonable(x, depth + 1) for k, x in list(v.items())[:64]}
    if hasattr(v, "tolist"):
        try:
            return _jsonable(v.tolist(), depth + 1)
        except Exception:
            pass
    return repr(v)[:200]


_WRITE_LOCK = threading.Lock()


def rollout_trace_op(func):
    """Decorator for (async) methods: records name, inputs, output and duration under the current trace attributes."""

    def record(self, args, kwargs, result, dt, err):
        cfg = RolloutTraceConfig.get_instance()
        attrs = _ATTRS.get()
        if cfg.backend != "file" or not attrs or not attrs.get("trace", True):
            return
        sig = inspect.signature(func)
        try:
            bound = sig.bind(self, *args, **kwargs)
            inputs = {k: _jsonable(v) for k, v in bound.arguments.items() if k != "self"}
        except TypeError:
            inputs = {}
        row = {"op": func.__qualname__, "attrs": attrs, "inputs": inputs, "output": _jsonable(result), "seconds": dt,
               "error": repr(err) if err else None, "time": time.time()}
        os.makedirs(os.path.dirname(cfg.path) or ".", exist_ok=True)
        with _WRITE_LOCK, open(cfg.path, "a") as f:
            f.write(json.dumps(row) + "\n")

    if inspect.iscoroutinefunction(func):
        @functools.wraps(func)
        async def awrapper(self, *args, **kwargs):
            if RolloutTraceConfig.get_backend() is None:
                return await func(self, *args, **kwargs)
            t0, err, res = time.perf_counter(), None, None
            try:
                res = await func(self, *args, **kwargs)
                return res
            except Exception as e:
                err = e
                raise
            finally:
                record(self, args, kwargs, res, time.perf_counter() - t0, err)

        return awrapper

    @functools.wraps(func)
    def wrapper(self, *args, **kwargs):
        if RolloutTraceConfig.get_backend() is None:
            return func(self, *args, **kwargs)
        t0, err, res = time.perf_counter(), None, None
        try:
            res = func(self, *args, **kwargs)
            return res
        except Exception as e:
            err = e
            raise
        finally:
            record(self, args, kwargs, res, time.perf_counter() - t0, err)

    return wrapper
