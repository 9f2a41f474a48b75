"""``exists`` / ``makedirs`` / ``copy`` that accept local paths and ``hdfs://`` URLs (verl/utils/hdfs_io.py:28-150).
HDFS operations shell out to the ``hdfs dfs`` command line, which must be on PATH for such paths."""

from __future__ import annotations

import logging
import os
import shutil
import subprocess

logger = logging.getLogger(__name__)
_HDFS_PREFIX = "hdfs://"
_HDFS_BIN = shutil.which("hdfs") or "hdfs"


def is_non_local(path: str) -> bool:
    return str(path).startswith(_HDFS_PREFIX)


def _run(args: list[str]) -> int:
    try:
        return subprocess.run([_HDFS_BIN, "dfs", *args], capture_output=True, timeout=600).returncode
    except (FileNotFoundError, subprocess.TimeoutExpired) as e:
        logger.warning("hdfs command failed: %s", e)
        return 127


def exists(path: str, **kwargs) -> bool:
    return _run(["-test", "-e", path]) == 0 if is_non_local(path) else os.path.exists(path)


def makedirs(name: str, mode: int = 0o777, exist_ok: bool = False, **kwargs) -> None:
    if is_non_local(name):
        rc = _run(["-mkdir", "-p", name])
        if rc != 0:
            raise OSError(f"hdfs dfs -mkdir -p {name} returned {rc}")
    else:
        os.makedirs(name, mode=mode, exist_ok=exist_ok)


def copy(src: str, dst: str, **kwargs) -> bool:
    if is_non_local(src) or is_non_local(dst):
        if is_non_local(src) and not is_non_local(dst):
            args = ["-get", src, dst]
        elif is_non_local(dst) and not is_non_local(src):
            args = ["-put", "-f", src, dst]
        else:
            args = ["-cp", "-f", src, dst]
        return _run(args) == 0
    if os.path.isdir(src):
        shutil.copytree(src, dst, dirs_exist_ok=True)
    else:
        shutil.copy(src, dst)
    return True
