"""Per-kernel device-time breakdown of a region (``torch.profiler`` device activities; no ncu).

Used to see how a training phase divides between GEMMs, attention, the fused lm_head, elementwise kernels, the
optimizer and communication. The times are taken while a profiler is attached, so they are for SHARES only; the
phase's duration comes from an un-profiled run (CUDA events).

``exposed`` communication is the time during which only communication kernels (peer-memory collectives, copy-engine
transfers, NCCL) were running on the device: intervals of communication kernels minus their overlap with compute
kernels of any stream.
"""

from __future__ import annotations

import re
from collections import defaultdict
from typing import Callable

import torch

# first match wins
_CLASSES = [
    ("attention_fwd", re.compile(r"flash_fwd|flash_attention_fwd|paged_decode|paged_attention")),
    ("attention_bwd", re.compile(r"flash_bwd")),
    ("grouped_gemm", re.compile(r"grouped|grp")),
    ("fp8_gemm", re.compile(r"fp8")),
    ("gemm", re.compile(r"gemm_kernel|gemm_pair|splitk|lse_merge|cutlass|cublas|gemm")),
    ("comm", re.compile(r"peer_|nvls_|moe_dispatch|moe_combine|tp_allreduce|nccl|Memcpy PtoP|Memcpy DtoD.*Peer|segment_copy")),
    ("optimizer", re.compile(r"adamw|sumsq|clip_coef|cast_f32")),
    ("norm_rope_act", re.compile(r"rmsnorm|rope|swiglu|embedding")),
    ("rl_loss", re.compile(r"ppo_loss|gae|grpo|sample")),
    ("memcpy_memset", re.compile(r"Memcpy|Memset")),
]


def classify(name: str) -> str:
    for cls, pat in _CLASSES:
        if pat.search(name):
            return cls
    return "other_torch"


def _union(intervals):
    out = []
    for s, e in sorted(intervals):
        if out and s <= out[-1][1]:
            out[-1][1] = max(out[-1][1], e)
        else:
            out.append([s, e])
    return out


def _subtract(a, b):
    """Total length of the union ``a`` not covered by the union ``b`` (both sorted, disjoint)."""
    total, j = 0.0, 0
    for s, e in a:
        cur = s
        while j < len(b) and b[j][1] <= cur:
            j += 1
        k = j
        while k < len(b) and b[k][0] < e:
            if b[k][0] > cur:
                total += b[k][0] - cur
            cur = max(cur, b[k][1])
            k += 1
        if cur < e:
            total += e - cur
    return total


def kernel_breakdown(fn: Callable[[], None], top: int = 25) -> dict:
    """Run ``fn`` once under the profiler. Returns ``{"total_device_ms", "by_class": {class: ms}, "top_kernels":
    [(name, ms, calls)], "comm_ms", "exposed_comm_ms", "busy_ms"}`` (device times of this process's GPU)."""
    from torch.profiler import ProfilerActivity, profile

    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU], record_shapes=False) as prof:
        fn()
        torch.cuda.synchronize()
    by_name: dict = defaultdict(lambda: [0.0, 0])
    by_class: dict = defaultdict(float)
    comm_iv, comp_iv = [], []
    for ev in prof.events():
        if getattr(ev, "device_type", None) is None or "cuda" not in str(ev.device_type).lower():
            continue
        dur_us = float(getattr(ev, "device_time_total", 0.0) or getattr(ev, "cuda_time_total", 0.0) or 0.0)
        if dur_us <= 0 and ev.time_range is not None:
            dur_us = float(ev.time_range.end - ev.time_range.start)
        if dur_us <= 0:
            continue
        name = ev.name
        cls = classify(name)
        by_name[name][0] += dur_us / 1e3
        by_name[name][1] += 1
        by_class[cls] += dur_us / 1e3
        if ev.time_range is not None:
            (comm_iv if cls == "comm" else comp_iv).append((float(ev.time_range.start), float(ev.time_range.end)))
    cu, pu = _union(comm_iv), _union(comp_iv)
    busy = sum(e - s for s, e in _union(comm_iv + comp_iv)) / 1e3
    topk = sorted(((n, round(v[0], 3), v[1]) for n, v in by_name.items()), key=lambda t: -t[1])[:top]
    return {"total_device_ms": round(sum(by_class.values()), 3), "busy_ms": round(busy, 3),
            "by_class": {k: round(v, 3) for k, v in sorted(by_class.items(), key=lambda kv: -kv[1])},
            "comm_ms": round(sum(e - s for s, e in cu) / 1e3, 3), "exposed_comm_ms": round(_subtract(cu, pu) / 1e3, 3),
            "top_kernels": [(n[:120], ms, c) for n, ms, c in topk]}
