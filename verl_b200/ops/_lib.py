"""ctypes binding of the native library (``verl_b200/lib/libverl_b200.so``).

The library is plain C ABI: every launcher takes raw device pointers, sizes and a
``cudaStream_t`` and returns 0 or an error code. On a machine with a GPU a missing
library is an error (no silent eager fallback); on a CPU-only machine the library
still loads (it does not link libcuda) but the ops that need it are never called.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p
from pathlib import Path

import torch

_LIB = None
_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libverl_b200.so"

P, I, L, F, U = c_void_p, c_int, c_longlong, c_float, c_ulonglong

_SIGS = {
    "vb_abi_version": ([], I),
    "vb_launch_count": ([], L),
    "vb_launch_count_reset": ([], None),
    "vb_set_pdl": ([I], None),
    # gemm
    "vb_gemm_bf16": ([P, P, P, P, I, I, I, L, L, L, I, I, I, I, P, P], I),
    "vb_gemm_bf16_ws": ([P, P, P, P, I, I, I, L, L, L, I, I, I, I, P, L, P, I, P, P], I),
    "vb_lmhead_num_splits": ([I, I], I),
    "vb_lmhead_logprob_fwd": ([P, P, P, I, I, I, F, P, P, P, P, P, P, P], I),
    "vb_lmhead_dlogits": ([P, P, P, I, I, I, I, F, P, P, P, P, P, L, P, P], I),
    # elementwise
    "vb_rmsnorm_fwd": ([P, P, P, P, P, P, L, I, F, P], I),
    "vb_rmsnorm_bwd_parts": ([L], I),
    "vb_rmsnorm_bwd": ([P, P, P, P, P, P, P, P, I, L, I, P], I),
    "vb_rope": ([P, P, L, L, P, P, P, I, I, I, I, I, P], I),
    "vb_mrope": ([P, P, L, L, P, P, P, I, I, I, I, I, I, I, P], I),
    "vb_swiglu_fwd": ([P, P, L, I, P], I),
    "vb_swiglu_bwd": ([P, P, P, L, I, P], I),
    "vb_embedding_fwd": ([P, P, P, L, I, P], I),
    "vb_embedding_bwd": ([P, P, P, L, I, P], I),
    "vb_adamw": ([P, P, I, P, P, P, L, F, F, F, F, F, I, P, P, P], I),
    "vb_sumsq": ([P, I, L, P, P], I),
    "vb_clip_coef": ([P, F, F, P, P, P, P], I),
    "vb_cast_f32_bf16": ([P, P, L, P], I),
    # rl ops
    "vb_ppo_loss": ([P, P, P, P, P, P, P, P, P, P, L, F, F, F, F, I, F, F, P], I),
    "vb_gae": ([P, P, P, P, P, I, I, F, F, P], I),
    "vb_grpo_adv": ([P, P, P, P, P, I, I, I, F, I, P], I),
    "vb_sample": ([P, I, L, I, I, P, P, P, U, P, P, P, P], I),
    "vb_decode_advance": ([P, P, P, P, P, P, P, I, I, P, P, P, L, P, P, P, P, I, I, P], I),
    # attention
    "vb_decode_num_splits": ([I, I, I], I),
    "vb_grouped_gemm_bf16": ([P, P, P, I, I, I, L, L, L, I, I, I, I, I, I, P, P, P, P], I),
    "vb_fp8_quant_weight": ([P, L, I, I, P, L, P, I, P], I),
    "vb_fp8_quant_act": ([P, L, L, I, P, L, P, I, P], I),
    "vb_fp8_gemm_blockscale": ([P, P, P, P, P, P, I, I, I, L, L, L, P, P], I),
    "vb_flash_bwd_delta": ([P, P, L, L, P, L, I, P], I),
    "vb_flash_bwd_dq": ([P, P, P, P, L, L, L, L, P, I, L, I, I, I, F, I, P, P, P, L, P, P], I),
    "vb_flash_bwd_dkv": ([P, P, P, P, L, L, L, L, P, I, L, I, I, I, F, I, P, P, P, P, L, P, P], I),
    "vb_flash_fwd": ([P, P, P, L, L, L, P, P, I, L, L, I, I, I, F, I, P, L, P, P, P], I),
    "vb_paged_decode_tc_supported": ([I, I, I, I], I),
    "vb_paged_decode_tc": ([P, L, P, P, I, P, I, P, I, I, I, I, F, I, P, L, P, P, P], I),
    "vb_paged_decode": ([P, L, P, P, P, I, P, I, I, I, I, I, F, I, P, L, P, P], I),
    "vb_kv_cache_write": ([P, P, L, L, P, P, P, L, I, I, I, P], I),
}


class NativeLibraryError(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def load(build_if_missing: bool = True):
    """Load (building first if necessary) and return the ctypes handle."""
    global _LIB, _LIB_PATH
    if _LIB is not None:
        return _LIB
    flavour = "jitter" if os.environ.get("VERL_B200_JITTER") == "1" else ""
    if flavour:  # the race-hunting build: blocks of the communication kernels start after pseudo-random sleeps
        _LIB_PATH = _LIB_PATH.with_name(f"libverl_b200_{flavour}.so")
    if not _LIB_PATH.exists():
        if not build_if_missing:
            raise NativeLibraryError(f"native library missing: {_LIB_PATH}; run `python -m verl_b200._build`"
                                     + (" --jitter" if flavour else ""))
        from verl_b200 import _build

        _build.build(flavour=flavour)
    lib = ctypes.CDLL(str(_LIB_PATH), mode=os.RTLD_NOW | os.RTLD_GLOBAL)
    for name, (argtypes, restype) in _SIGS.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue  # optional symbol (older build); the op that needs it raises on use
        fn.argtypes = argtypes
        fn.restype = restype
    _LIB = lib
    return lib


def available() -> bool:
    try:
        load(build_if_missing=False)
        return True
    except Exception:
        return False


def fn(name: str):
    lib = load()
    try:
        return getattr(lib, name)
    except AttributeError as e:
        raise NativeLibraryError(f"symbol {name} not in {_LIB_PATH}; rebuild the native library") from e


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for the kernels that support it (default on; VERL_B200_PDL=0 turns it off):
    each such kernel may start while the kernel before it in the stream still runs, and waits for it only before
    its first access to global memory. Applies to launches and graph captures made after the call."""
    fn("vb_set_pdl")(1 if on else 0)


def ptr(t) -> int | None:
    """Device pointer of a tensor (None passes a null pointer)."""
    if t is None:
        return None
    return t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeLibraryError(f"{what} failed with code {rc}")


def launch_count() -> int:
    return int(fn("vb_launch_count")())


def reset_launch_count() -> None:
    fn("vb_launch_count_reset")()


_status_words = {}


def status_word(device=None) -> torch.Tensor:
    """Per-device int32[4] status word written by kernels whose bounded waits ran out."""
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    key = (dev.type, dev.index)
    if key not in _status_words:
        _status_words[key] = torch.zeros(4, dtype=torch.int32, device=dev)
    return _status_words[key]


def read_status(device=None) -> tuple[int, int, int]:
    """Synchronising read of the status word: (code, block, detail); code 0 = no error."""
    w = status_word(device).tolist()
    return w[0], w[1], w[2]


def clear_status(device=None) -> None:
    status_word(device).zero_()
