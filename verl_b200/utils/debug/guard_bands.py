"""Guard bands around device allocations: a memory-safety check for hand-written kernels that needs no sanitizer.

Inside ``with guard_allocations() as g:`` every tensor that ``torch.empty`` / ``empty_like`` / ``zeros`` / ``zeros_like``
/ ``empty_strided`` hands out on the chosen device sits between two bands of a canary byte; ``g.check()`` (also run on
exit) reads the bands back and raises with the offending allocation if a kernel wrote before the start or past the
end of its buffer. The ops of this package allocate their outputs and workspaces through these calls, so wrapping an op
in the context checks every buffer the op created. Reads out of bounds are not caught (they change no canary): those
are covered by comparing results with a reference on tile-edge shapes.

The reference has no counterpart (it ships no kernels of its own that would need one).
"""

from __future__ import annotations

import contextlib
from typing import Optional

import torch

CANARY = 0xA5
BAND_BYTES = 4096  # a multiple of every alignment the kernels ask for (TMA: 16 B, vector loads: 16 B, swizzle: 1024 B)


class GuardError(AssertionError):
    pass


class _Guard:
    def __init__(self, device: torch.device, band: int):
        self.device, self.band = device, band
        self.allocs: list[tuple[torch.Tensor, int, str]] = []  # (flat uint8 base, payload bytes, description)
        self.count = 0

    def _alloc(self, shape, dtype, zero: bool) -> torch.Tensor:
        dtype = dtype or torch.get_default_dtype()
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * _ORIG["empty"](0, dtype=dtype).element_size()
        pad = (-nbytes) % 16  # keep the trailing band 16-byte aligned as well
        base = _ORIG["empty"](self.band + nbytes + pad + self.band, dtype=torch.uint8, device=self.device)
        base[: self.band].fill_(CANARY)
        base[self.band + nbytes :].fill_(CANARY)
        body = base[self.band : self.band + nbytes]
        if zero:
            body.zero_()
        self.allocs.append((base, nbytes, f"{tuple(shape)} {dtype}"))
        self.count += 1
        return body.view(dtype).view(*shape) if len(shape) else body.view(dtype).view(())

    def check(self) -> int:
        """Verify every band; returns the number of allocations checked."""
        torch.cuda.synchronize(self.device) if self.device.type == "cuda" else None
        for base, nbytes, what in self.allocs:
            lo = base[: self.band]
            hi = base[self.band + nbytes :]
            for name, band in (("before the start", lo), ("past the end", hi)):
                bad = (band != CANARY).nonzero()
                if bad.numel():
                    first = int(bad[0])
                    off = first - self.band if name == "before the start" else first
                    raise GuardError(f"a kernel wrote {name} of an allocation {what}: first damaged byte at offset "
                                     f"{off} relative to that edge, {int(bad.numel())} byte(s) damaged")
        return len(self.allocs)


_ORIG: dict = {}


def _shape_of(args, kwargs):
    if "size" in kwargs:
        return tuple(kwargs["size"])
    if len(args) == 1 and isinstance(args[0], (tuple, list, torch.Size)):
        return tuple(args[0])
    return tuple(int(a) for a in args)


@contextlib.contextmanager
def guard_allocations(device: Optional[torch.device | str] = None, band_bytes: int = BAND_BYTES, check_on_exit: bool = True):
    """Route the allocation calls named above through guarded allocations on ``device`` (default: the current CUDA
    device, or the CPU when there is none). Dense, contiguous requests only; anything else (sparse layouts, pinned
    memory, other devices, ``out=``) falls through to torch. Not thread-safe: for tests."""
    dev = torch.device(device) if device is not None else (
        torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
    g = _Guard(dev, band_bytes)
    names = ("empty", "zeros", "empty_like", "zeros_like", "empty_strided")
    for n in names:
        _ORIG[n] = getattr(torch, n)

    def same_device(d) -> bool:
        if d is None:
            return dev.type == "cpu"  # torch's default device is the CPU
        d = torch.device(d)
        if d.type != dev.type:
            return False
        return d.index is None or dev.index is None or d.index == dev.index

    def plain(kwargs) -> bool:
        return not (kwargs.get("pin_memory") or kwargs.get("out") is not None or kwargs.get("requires_grad")
                    or kwargs.get("layout", torch.strided) is not torch.strided
                    or kwargs.get("memory_format", torch.contiguous_format) not in (torch.contiguous_format, torch.preserve_format))

    def make(zero: bool, orig):
        def fn(*args, **kwargs):
            if same_device(kwargs.get("device")) and plain(kwargs):
                try:
                    shape = _shape_of(args, kwargs)
                except Exception:
                    return orig(*args, **kwargs)
                return g._alloc(shape, kwargs.get("dtype"), zero)
            return orig(*args, **kwargs)

        return fn

    def make_like(zero: bool, orig):
        def fn(t, **kwargs):
            d = kwargs.get("device", t.device)
            if same_device(d) and plain(kwargs) and t.is_contiguous() and t.layout is torch.strided:
                return g._alloc(tuple(t.shape), kwargs.get("dtype", t.dtype), zero)
            return orig(t, **kwargs)

        return fn

    def strided(size, stride, **kwargs):
        want = []
        acc = 1
        for s in reversed(tuple(size)):
            want.append(acc)
            acc *= int(s)
        if same_device(kwargs.get("device")) and plain(kwargs) and tuple(stride) == tuple(reversed(want)):
            return g._alloc(tuple(size), kwargs.get("dtype"), False)
        return _ORIG["empty_strided"](size, stride, **kwargs)

    torch.empty, torch.zeros = make(False, _ORIG["empty"]), make(True, _ORIG["zeros"])
    torch.empty_like, torch.zeros_like = make_like(False, _ORIG["empty_like"]), make_like(True, _ORIG["zeros_like"])
    torch.empty_strided = strided
    try:
        yield g
        if check_on_exit:
            g.check()
    finally:
        for n in names:
            setattr(torch, n, _ORIG[n])
