"""Environment report for bug reports (role of the reference's ``scripts/diagnose.py``): python / torch / CUDA
versions, GPUs with memory and clocks (read-only queries), the native library and whether its kernels load.

    python -m verl_b200.utils.diagnose
"""

from __future__ import annotations

import json
import os
import platform
import shutil
import subprocess
import sys


def collect() -> dict:
    info: dict = {"python": sys.version.split()[0], "platform": platform.platform(), "cpu_count": os.cpu_count()}
    try:
        import torch

        info["torch"] = torch.__version__
        info["torch_cuda"] = torch.version.cuda
        info["cuda_available"] = torch.cuda.is_available()
        info["nccl"] = ".".join(map(str, torch.cuda.nccl.version())) if torch.cuda.is_available() else None
        info["gpus"] = [{"index": i, "name": torch.cuda.get_device_name(i), "capability": list(torch.cuda.get_device_capability(i)),
                         "memory_gb": round(torch.cuda.get_device_properties(i).total_memory / 2**30, 1)}
                        for i in range(torch.cuda.device_count())] if torch.cuda.is_available() else []
    except Exception as e:  # noqa: BLE001
        info["torch_error"] = repr(e)
    for mod in ("numpy", "transformers", "safetensors", "pyarrow", "fastapi", "uvicorn", "aiohttp"):
        try:
            info[mod] = __import__(mod).__version__
        except Exception:  # noqa: BLE001
            info[mod] = None
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if os.path.exists(nvcc):
        out = subprocess.run([nvcc, "--version"], capture_output=True, text=True).stdout.strip().splitlines()
        info["nvcc"] = out[-2] if len(out) >= 2 else out
    if shutil.which("nvidia-smi"):
        q = "index,name,driver_version,clocks.sm,clocks.max.sm,power.limit,memory.used,memory.total"
        r = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader"], capture_output=True, text=True)
        info["nvidia_smi"] = r.stdout.strip().splitlines()
    try:
        from ..ops import _lib

        path = _lib.lib_path()
        info["native_library"] = {"path": str(path), "present": os.path.exists(str(path))}
    except Exception as e:  # noqa: BLE001
        info["native_library"] = {"error": repr(e)}
    info["env"] = {k: v for k, v in os.environ.items() if k.startswith(("VERL_", "NCCL_", "CUDA_", "TORCH_"))}
    return info


def main() -> dict:
    info = collect()
    print(json.dumps(info, indent=2, default=str))
    return info


if __name__ == "__main__":
    main()
