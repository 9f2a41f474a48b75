"""In-tree build of the native library (CUDA kernels for sm_100a + C++ runtime).

Every ``csrc/*.cu`` is compiled with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` and every
``csrc/*.cpp`` with g++, then linked into ``verl_b200/lib/libverl_b200.so``.
The library exposes a C ABI that :mod:`verl_b200.ops._lib` binds through ctypes,
so no torch headers are needed and a full rebuild takes well under a minute.
nvcc cross-compiles without a GPU, so this also runs on a CPU-only machine.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = CSRC / "build"
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "libverl_b200.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--use_fast_math",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-Wno-unused-function",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the native library cannot be built")
    return cand


def _sources():
    cu = sorted(CSRC.glob("*.cu"))
    cpp = sorted(CSRC.glob("*.cpp"))
    return cu, cpp


def _digest(path: Path, extra: str) -> str:
    h = hashlib.sha1()
    h.update(extra.encode())
    h.update(path.read_bytes())
    for hdr in sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(hdr.read_bytes())
    return h.hexdigest()


# Build flavours: "" = the library every run uses; "jitter" = the same sources with -DVB_JITTER=1 (blocks of the
# communication kernels and of the GEMM sleep a pseudo-random time before they start), for race hunting in tests.
FLAVOUR_FLAGS = {"": [], "jitter": ["-DVB_JITTER=1"]}


def lib_path(flavour: str = "") -> Path:
    return LIB_DIR / (f"libverl_b200_{flavour}.so" if flavour else "libverl_b200.so")


def _compile_one(src: Path, verbose: bool, ptxas_verbose: bool, flavour: str = "") -> Path:
    is_cu = src.suffix == ".cu"
    flags = (NVCC_FLAGS if is_cu else CXX_FLAGS) + FLAVOUR_FLAGS[flavour]
    obj_dir = OBJ_DIR if not flavour else OBJ_DIR.parent / f"build_{flavour}"
    obj = obj_dir / (src.name + ".o")
    stamp = obj_dir / (src.name + ".sha1")
    dig = _digest(src, " ".join(flags))
    if obj.exists() and stamp.exists() and stamp.read_text() == dig and not ptxas_verbose:
        return obj
    if is_cu:
        cmd = [_nvcc(), *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if ptxas_verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
    else:
        cuda_inc = str(Path(_nvcc()).resolve().parent.parent / "include")
        cmd = ["g++", *flags, "-I", str(CSRC), "-I", cuda_inc, "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"compile failed: {src.name}\n{res.stdout}\n{res.stderr}")
    if ptxas_verbose or verbose:
        sys.stderr.write(res.stderr)
    stamp.write_text(dig)
    return obj


def build(force: bool = False, verbose: bool = False, ptxas_verbose: bool = False, flavour: str = "") -> Path:
    """Compile all native sources and link the shared library (of the given flavour). Returns its path."""
    obj_dir = OBJ_DIR if not flavour else OBJ_DIR.parent / f"build_{flavour}"
    out = lib_path(flavour)
    obj_dir.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    if force:
        for f in obj_dir.glob("*.sha1"):
            f.unlink()
    cu, cpp = _sources()
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, verbose, ptxas_verbose, flavour), cu + cpp))
    newest = max(o.stat().st_mtime for o in objs)
    if force or not out.exists() or out.stat().st_mtime < newest:
        cmd = [_nvcc(), "-shared", "-o", str(out), *map(str, objs), "-lcudart", "-lpthread"]
        if verbose:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed\n{res.stdout}\n{res.stderr}")
    return out


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="-v" in sys.argv, ptxas_verbose="--ptxas" in sys.argv,
              flavour="jitter" if "--jitter" in sys.argv else "")
    print(p)
