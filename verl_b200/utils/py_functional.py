"""Small Python helpers (verl/utils/py_functional.py): timeouts, dict utilities, dynamic enums."""

from __future__ import annotations

import importlib
import multiprocessing
import os
import queue
import signal
import threading
from contextlib import contextmanager
from functools import wraps
from types import SimpleNamespace
from typing import Any, Callable, Iterator, Optional


def _mp_target(q, fn, args, kwargs):
    try:
        q.put((True, fn(*args, **kwargs)))
    except Exception as e:  # carried to the parent
        q.put((False, e))


def timeout_limit(seconds: float, use_signals: bool = False):
    """Decorator: raise ``TimeoutError`` if the call runs longer than ``seconds``. ``use_signals`` uses
    SIGALRM (main thread only, no pickling); otherwise the call runs in a child process."""

    def deco(fn):
        if use_signals:
            if threading.current_thread() is not threading.main_thread():
                raise RuntimeError("timeout_limit with signals must be used from the main thread")

            @wraps(fn)
            def sig_wrapper(*args, **kwargs):
                def handler(signum, frame):
                    raise TimeoutError(f"Function {fn.__name__} timed out after {seconds} seconds (signal)!")

                old = signal.signal(signal.SIGALRM, handler)
                signal.setitimer(signal.ITIMER_REAL, seconds)
                try:
                    return fn(*args, **kwargs)
                finally:
                    signal.setitimer(signal.ITIMER_REAL, 0)
                    signal.signal(signal.SIGALRM, old)

            return sig_wrapper

        @wraps(fn)
        def mp_wrapper(*args, **kwargs):
            q = multiprocessing.Queue(maxsize=1)
            p = multiprocessing.Process(target=_mp_target, args=(q, fn, args, kwargs))
            p.start()
            p.join(timeout=seconds)
            if p.is_alive():
                p.terminate()
                p.join(0.5)
                if p.is_alive():
                    p.kill()
                raise TimeoutError(f"Function {fn.__name__} timed out after {seconds} seconds (multiprocessing)!")
            try:
                ok, val = q.get(timeout=0.1)
            except queue.Empty as e:
                raise RuntimeError(f"Child process exited without a result (exit code {p.exitcode})") from e
            if ok:
                return val
            raise val

        return mp_wrapper

    return deco


def union_two_dict(dict1: dict, dict2: dict) -> dict:
    for k, v in dict2.items():
        if k in dict1:
            assert dict2[k] == dict1[k], f"{k} in meta_dict1 and meta_dict2 are not the same object"
        dict1[k] = v
    return dict1


def append_to_dict(data: dict, new_data: dict, prefix: str = "") -> None:
    """Append each value of ``new_data`` to the list under the same (prefixed) key of ``data``."""
    for k, v in new_data.items():
        data.setdefault(f"{prefix}{k}", []).append(v)


def rename_dict(data: dict, prefix: str = "") -> dict:
    return {f"{prefix}{k}": v for k, v in data.items()}


class NestedNamespace(SimpleNamespace):
    def __init__(self, dictionary, **kwargs):
        super().__init__(**kwargs)
        for k, v in dictionary.items():
            setattr(self, k, NestedNamespace(v) if isinstance(v, dict) else v)


def convert_to_regular_types(obj):
    from .config import to_container

    return to_container(obj)


def load_extern_object(module_path: Optional[str], object_name: str):
    """Load ``object_name`` from a python file path or an importable module name."""
    if module_path is None:
        return None
    if os.path.exists(module_path):
        spec = importlib.util.spec_from_file_location("custom_module", module_path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    else:
        mod = importlib.import_module(module_path)
    if not hasattr(mod, object_name):
        raise AttributeError(f"'{object_name}' not found in '{module_path}'")
    return getattr(mod, object_name)


@contextmanager
def temp_env_var(key: str, value: str) -> Iterator[None]:
    old = os.environ.get(key)
    os.environ[key] = value
    try:
        yield
    finally:
        if old is None:
            os.environ.pop(key, None)
        else:
            os.environ[key] = old
