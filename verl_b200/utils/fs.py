"""File helpers (role of verl/utils/fs.py, hdfs_io.py): ``copy_to_local`` resolves a model / data path to a local
one. HDFS needs the hadoop client, which this image does not have: ``hdfs://`` paths raise with that explanation;
local paths can be staged into shared memory (``use_shm``) as the reference does for fast multi-process loading."""

from __future__ import annotations

import hashlib
import os
import shutil
from typing import Optional

_HDFS_PREFIX = "hdfs://"


def is_non_local(path: str) -> bool:
    return str(path).startswith(_HDFS_PREFIX)


def md5_encode(path: str) -> str:
    return hashlib.md5(path.encode()).hexdigest()


def get_local_temp_path(hdfs_path: str, cache_dir: str) -> str:
    return os.path.join(cache_dir, md5_encode(hdfs_path), os.path.basename(hdfs_path.rstrip("/")))


def copy_to_shm(src: str) -> str:
    """Copy a file or directory under /dev/shm/verl-cache and return the new path."""
    src = os.path.abspath(os.path.expanduser(src))
    root = os.path.join("/dev/shm", "verl-cache", md5_encode(src))
    dest = os.path.join(root, os.path.basename(src.rstrip("/")))
    if os.path.exists(dest):
        return dest
    os.makedirs(root, exist_ok=True)
    if os.path.isdir(src):
        shutil.copytree(src, dest, symlinks=False, dirs_exist_ok=True)
    else:
        shutil.copy2(src, dest)
    return dest


def copy_to_local(src: str, cache_dir: Optional[str] = None, filelock: str = ".file.lock", verbose: bool = False,
                  always_recopy: bool = False, use_shm: bool = False) -> str:
    if src is None:
        return src
    if is_non_local(src):
        raise RuntimeError(f"{src}: HDFS access needs the hadoop command-line client, which is not installed here")
    src = os.path.expanduser(str(src))
    if use_shm and os.path.exists(src):
        return copy_to_shm(src)
    return src


def local_mkdir_safe(path: str) -> str:
    os.makedirs(os.path.expanduser(path), exist_ok=True)
    return path


def verify_copy(src: str, dest: str) -> bool:
    """True when ``dest`` looks like a complete copy of ``src``: the same kind, the same relative file tree, the same
    file sizes."""
    if not (os.path.exists(src) and os.path.exists(dest)) or os.path.isfile(src) != os.path.isfile(dest):
        return False
    if os.path.isfile(src):
        return os.path.getsize(src) == os.path.getsize(dest)

    def tree(root):
        out = {}
        for d, _, files in os.walk(root):
            for f in files:
                p = os.path.join(d, f)
                out[os.path.relpath(p, root)] = os.path.getsize(p)
        return out

    return tree(src) == tree(dest)


def copy_local_path_from_hdfs(src: str, cache_dir: Optional[str] = None, filelock: str = ".file.lock", verbose: bool = False,
                              always_recopy: bool = False) -> str:
    """Historical name of :func:`copy_to_local`."""
    return copy_to_local(src, cache_dir=cache_dir, filelock=filelock, verbose=verbose, always_recopy=always_recopy)
