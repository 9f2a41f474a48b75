"""Peer-memory collectives for one NVSwitch domain (kernels in ``csrc/comm.cu``).

Buffers that peers must read (parameter shards, per-unit gradient buffers, signal pads) are allocated from
torch's symmetric-memory allocator, which maps every rank's allocation into every process and, where the
fabric supports it, creates an NVLS multicast mapping. That is the only service taken from the library: the
data movement and the synchronisation are this package's own kernels (plain peer loads or
``multimem.ld_reduce``; never NCCL, never TMA on peer memory).

In the reference all of this is NCCL inside torch FSDP (all-gather / reduce-scatter per layer) and NCCL /
CUDA-IPC copies for weight sync (verl/workers/fsdp_workers.py:677-756).
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _lib

_SIGS_BOUND = False


def _bind():
    global _SIGS_BOUND
    lib = _lib.load()
    if _SIGS_BOUND:
        return lib
    c = ctypes
    P, I, L, U, F = c.c_void_p, c.c_int, c.c_longlong, c.c_uint, c.c_float
    lib.vb_peer_max_ranks.argtypes, lib.vb_peer_max_ranks.restype = [], I
    lib.vb_peer_barrier.argtypes, lib.vb_peer_barrier.restype = [P, I, I, I, U, P, P], I
    lib.vb_peer_all_gather.argtypes, lib.vb_peer_all_gather.restype = [P, P, L, P, L, I, I, I, U, P, P, P], I
    lib.vb_peer_all_gather_ce.argtypes, lib.vb_peer_all_gather_ce.restype = [P, P, L, P, L, I, I, I, U, P, P], I
    lib.vb_ag_gemm_bf16.argtypes = [P, P, P, P, I, I, I, L, L, P, I, L, L, P, I, P, P]
    lib.vb_ag_gemm_bf16.restype = I
    lib.vb_peer_reduce_scatter_add.argtypes = [P, P, P, L, P, L, F, I, I, I, U, P, P, P]
    lib.vb_peer_reduce_scatter_add.restype = I
    lib.vb_peer_segment_copy.argtypes, lib.vb_peer_segment_copy.restype = [P, P, P, I, P, I, I, I, U, P, P, P], I
    lib.vb_gemm_rs_bf16.argtypes = [P, P, P, I, I, I, L, L, L, P, I, I, I, P, L, P, I, P, P]
    lib.vb_gemm_rs_bf16.restype = I
    lib.vb_peer_sum_slots.argtypes, lib.vb_peer_sum_slots.restype = [P, P, P, P, L, I, I, I, I, U, P, P, P], I
    lib.vb_peer_a2a_chunks.argtypes = [P, P, L, P, P, P, L, L, I, I, I, I, I, U, P, P, P]
    lib.vb_peer_a2a_chunks.restype = I
    lib.vb_tp_allreduce_rmsnorm.argtypes = [P, P, L, P, P, P, P, I, I, F, I, I, I, P, P, P]
    lib.vb_tp_allreduce_rmsnorm.restype = I
    _SIGS_BOUND = True
    return lib


class _Alloc:
    """One symmetric allocation: the local tensor plus every rank's base pointer."""

    def __init__(self, tensor: torch.Tensor, ptrs: list[int], multicast_ptr: int):
        self.tensor = tensor
        self.base = tensor.data_ptr()
        self.nbytes = tensor.numel() * tensor.element_size()
        self.ptrs = (ctypes.c_void_p * len(ptrs))(*ptrs)
        self.multicast_ptr = multicast_ptr

    def offset_of(self, t: torch.Tensor) -> Optional[int]:
        off = t.data_ptr() - self.base
        if 0 <= off and off + t.numel() * t.element_size() <= self.nbytes:
            return off
        return None


class PeerComm:
    CH_GATHER, CH_REDUCE, CH_COPY, CH_BARRIER = 0, 1, 2, 3
    CH_TP = 4  # epoch kept on the device (tp_allreduce_rmsnorm): never used with host-side epochs

    def __init__(self, group=None, use_nvls: Optional[bool] = None):
        import torch.distributed._symmetric_memory as symm_mem

        self.symm_mem = symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.lib = _bind()
        assert self.world <= self.lib.vb_peer_max_ranks()
        if use_nvls is None:
            use_nvls = os.environ.get("VERL_B200_NVLS", "0") == "1"  # measured: plain peer loads match or beat the in-switch reduction at 2 and 8 GPUs
        self.use_nvls = use_nvls
        self.allocs: list[_Alloc] = []
        self.epochs = [0, 0, 0, 0]
        self.gates = torch.zeros(8, dtype=torch.int32, device=self.device)
        self.tp_ctrs = torch.zeros(4, dtype=torch.int32, device=self.device)  # epoch, done counter, gate of CH_TP
        self.pads = self.alloc(1024, torch.int32, zero=True)
        self.pad_alloc = self.allocs[-1]
        self._grad_bufs: list[torch.Tensor] = []
        self._grad_next = 0
        self.barrier()

    # -------------------------------------------------------------- allocation
    def alloc(self, numel: int, dtype: torch.dtype, zero: bool = True) -> torch.Tensor:
        """Symmetric allocation (collective: every rank must call it with the same size, in the same order)."""
        sm = self.symm_mem
        group_name = self.group.group_name
        try:
            sm.enable_symm_mem_for_group(group_name)
        except Exception:
            pass
        t = sm.empty(int(numel), dtype=dtype, device=self.device)
        if zero:
            t.zero_()
        torch.cuda.synchronize(self.device)
        hdl = sm.rendezvous(t, group_name)
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
        self.allocs.append(_Alloc(t, ptrs, mc))
        self._handles = getattr(self, "_handles", []) + [hdl]
        return t

    def _find(self, t: torch.Tensor) -> tuple[_Alloc, int]:
        for a in self.allocs:
            off = a.offset_of(t)
            if off is not None:
                return a, off
        raise ValueError("tensor is not inside a symmetric allocation of this communicator")

    def is_symmetric(self, t: torch.Tensor) -> bool:
        return any(a.offset_of(t) is not None for a in self.allocs)

    def reserve_grad_buffers(self, numel: int, count: int = 2):
        """Rotating fp32 buffers for per-unit gradients. While one is being reduced by slower peers the next
        unit's backward writes another; the caller reuses a buffer only after a later reduce-scatter proved
        that every peer finished reading it."""
        if len(self._grad_bufs) >= count and self._grad_bufs[0].numel() >= numel:
            return
        self._grad_bufs = [self.alloc(numel, torch.float32) for _ in range(count)]
        self._grad_next = 0

    def grad_buffer(self, numel: int) -> torch.Tensor:
        assert self._grad_bufs and self._grad_bufs[0].numel() >= numel, "reserve_grad_buffers() first"
        buf = self._grad_bufs[self._grad_next][:numel]
        self._grad_next = (self._grad_next + 1) % len(self._grad_bufs)
        buf.zero_()
        return buf

    # -------------------------------------------------------------- collectives
    def _epoch(self, ch: int) -> int:
        self.epochs[ch] += 1
        return self.epochs[ch]

    def _gate(self, ch: int) -> int:
        return self.gates.data_ptr() + 4 * ch

    def _status(self) -> int:
        return _lib.status_word(self.device).data_ptr()

    def barrier(self):
        rc = self.lib.vb_peer_barrier(self.pad_alloc.ptrs, self.rank, self.world, self.CH_BARRIER,
                                      self._epoch(self.CH_BARRIER), self._status(), _lib.stream())
        _lib.check(rc, "vb_peer_barrier")

    def all_gather(self, out: torch.Tensor, src: torch.Tensor, copy_engine: Optional[bool] = None):
        """out[r * n : (r+1) * n] = rank r's ``src`` (n = src.numel()); ``src`` must be symmetric memory.

        ``copy_engine`` (default: payloads of 1 MiB and more) moves the shards with asynchronous peer copies
        after a one-block handshake kernel instead of with SM loads."""
        a, off = self._find(src)
        nbytes = src.numel() * src.element_size()
        assert out.numel() * out.element_size() == nbytes * self.world
        if copy_engine is None:
            copy_engine = nbytes >= (1 << 20)
        if copy_engine:
            rc = self.lib.vb_peer_all_gather_ce(a.ptrs, self.pad_alloc.ptrs, off, out.data_ptr(), nbytes, self.rank,
                                                self.world, self.CH_GATHER, self._epoch(self.CH_GATHER), self._status(),
                                                _lib.stream())
            _lib.check(rc, "vb_peer_all_gather_ce")
            return
        rc = self.lib.vb_peer_all_gather(a.ptrs, self.pad_alloc.ptrs, off, out.data_ptr(), nbytes, self.rank, self.world,
                                         self.CH_GATHER, self._epoch(self.CH_GATHER), self._gate(self.CH_GATHER),
                                         self._status(), _lib.stream())
        _lib.check(rc, "vb_peer_all_gather")

    def reduce_scatter_add(self, dst: torch.Tensor, full: torch.Tensor, scale: float = 1.0):
        """dst += scale * sum over ranks of full[rank * n : (rank+1) * n]  (fp32; ``full`` symmetric)."""
        a, off = self._find(full)
        n = dst.numel()
        assert full.numel() == n * self.world and dst.dtype == torch.float32 and full.dtype == torch.float32
        mc = a.multicast_ptr if self.use_nvls else 0
        rc = self.lib.vb_peer_reduce_scatter_add(a.ptrs, self.pad_alloc.ptrs, ctypes.c_void_p(mc) if mc else None, off,
                                                 dst.data_ptr(), n, float(scale), self.rank, self.world, self.CH_REDUCE,
                                                 self._epoch(self.CH_REDUCE), self._gate(self.CH_REDUCE), self._status(),
                                                 _lib.stream())
        _lib.check(rc, "vb_peer_reduce_scatter_add")

    def segment_copy(self, dst: torch.Tensor, src_alloc_tensor: torch.Tensor, seg_table: torch.Tensor, nseg: int):
        """Table-driven gather from peers' copies of ``src_alloc_tensor`` into ``dst`` (see :mod:`.reshard`)."""
        a, off0 = self._find(src_alloc_tensor)
        assert off0 == 0, "pass the allocation's base tensor"
        rc = self.lib.vb_peer_segment_copy(a.ptrs, self.pad_alloc.ptrs, seg_table.data_ptr(), int(nseg), dst.data_ptr(),
                                           self.rank, self.world, self.CH_COPY, self._epoch(self.CH_COPY),
                                           self._gate(self.CH_COPY), self._status(), _lib.stream())
        _lib.check(rc, "vb_peer_segment_copy")

    def ag_gemm(self, x: torch.Tensor, shard: torch.Tensor, w_off: int, N: int, K: int, bias: Optional[torch.Tensor] = None,
                w_full: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16, barrier: bool = True):
        """Fused all-gather + GEMM: ``x [M, K] @ W^T`` where ``W [N, K]`` starts at element ``w_off`` of the flat bf16
        vector whose rank-r slice is ``shard`` (symmetric memory, same size on every rank). The gather runs inside the
        GEMM kernel (copy warps pull the peers' slices over NVLink chunk by chunk in tile order) and leaves the
        assembled matrix in ``w_full`` for later use. Returns (out [M, N], w_full [N, K]).

        ``barrier=True`` first runs the cross-rank handshake that makes every rank's slice final; pass False when a
        previous collective of the same step already did."""
        a, off = self._find(shard)
        assert shard.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and x.stride(1) == 1
        M = x.shape[0]
        if w_full is None:
            w_full = torch.empty((N, K), dtype=torch.bfloat16, device=x.device)
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        ready = torch.empty((N + 255) // 256, dtype=torch.int32, device=x.device)
        if barrier:
            self.barrier()
        srcs = (ctypes.c_void_p * self.world)(*[int(p) + off for p in a.ptrs])
        rc = self.lib.vb_ag_gemm_bf16(x.data_ptr(), w_full.data_ptr(), out.data_ptr(), _lib.ptr(bias), M, N, K, x.stride(0),
                                      out.stride(0), srcs, self.world, shard.numel(), int(w_off), ready.data_ptr(),
                                      int(out_dtype == torch.float32), self._status(), _lib.stream())
        _lib.check(rc, "vb_ag_gemm_bf16")
        return out, w_full

    def gemm_rs(self, x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor] = None,
                bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Fused GEMM -> reduce-scatter of a row-parallel linear layer: every rank holds ``x [M, K_local]`` and
        ``w [N, K_local]`` (its slice of the contraction); returns rows ``[rank * M / world, (rank + 1) * M / world)``
        of ``sum_ranks x @ w^T`` (+ ``residual`` for those rows; ``bias`` is added by rank 0's partial).

        The GEMM epilogue stores each finished tile into the owning rank's receive slot over NVLink while later tiles
        are still being computed; a second kernel waits for all ranks (bounded handshake) and adds the slots up from
        local memory. Collective: every rank calls it with the same shapes. Two receive buffers alternate, so a slot
        is rewritten only after every peer has passed the handshake of the following call."""
        from ..ops.gemm import _SPLITK_COUNTERS, _SPLITK_MAX_M, _splitk_workspace

        assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
        M, K = x.shape
        N = w.shape[0]
        W = self.world
        assert M % W == 0 and N % 8 == 0 and w.shape[1] == K, (M, N, K, W)
        rows = M // W
        n = rows * N
        key = ("gemm_rs", n)
        bufs = self.__dict__.setdefault("_rs_slots", {})
        if key not in bufs:
            bufs[key] = [self.alloc(W * n, torch.bfloat16, zero=False) for _ in range(2)] + [0]
            self.barrier()
        ent = bufs[key]
        slots = ent[ent[2] & 1]
        ent[2] += 1
        a, off = self._find(slots)
        dsts = (ctypes.c_void_p * W)(*[int(p) + off + self.rank * n * 2 for p in a.ptrs])
        stream = _lib.stream()
        ws, counters = _splitk_workspace(x.device, stream) if M <= _SPLITK_MAX_M else (None, None)
        use_bias = bias if self.rank == 0 else None
        rc = self.lib.vb_gemm_rs_bf16(x.data_ptr(), w.data_ptr(), _lib.ptr(use_bias), M, N, K, x.stride(0), w.stride(0), N,
                                      dsts, W, rows, 0, _lib.ptr(ws), ws.numel() * 4 if ws is not None else 0,
                                      _lib.ptr(counters), _SPLITK_COUNTERS if ws is not None else 0, self._status(),
                                      stream)
        _lib.check(rc, "vb_gemm_rs_bf16")
        out = torch.empty((rows, N), dtype=torch.bfloat16, device=x.device)
        if residual is not None:
            assert residual.shape == out.shape and residual.is_contiguous() and residual.dtype == out.dtype
        rc = self.lib.vb_peer_sum_slots(slots.data_ptr(), self.pad_alloc.ptrs, out.data_ptr(), _lib.ptr(residual), n, 0,
                                        self.rank, W, self.CH_REDUCE, self._epoch(self.CH_REDUCE),
                                        self._gate(self.CH_REDUCE), self._status(), stream)
        _lib.check(rc, "vb_peer_sum_slots")
        return out

    def tp_allreduce_rmsnorm(self, partial: torch.Tensor, residual: Optional[torch.Tensor],
                             weight: Optional[torch.Tensor], eps: float = 1e-6):
        """Row-parallel epilogue of a tensor-parallel block in one launch: ``h = sum_ranks partial (+ residual)``,
        returns ``(rmsnorm(h) * weight, h)`` (``(None, h)`` without ``weight``). ``partial [rows, H]`` (bf16) is this
        rank's partial product at the same offset of a symmetric buffer on every rank; the sums are bit-identical on
        all ranks. The kernel keeps its epoch on the device, so it can be captured in and replayed from a CUDA graph.
        The caller must not rewrite ``partial``'s buffer before a later call of this method has run on this rank
        (alternate two buffers)."""
        a, off = self._find(partial)
        rows, H = partial.shape
        assert partial.dtype == torch.bfloat16 and partial.is_contiguous()
        h = torch.empty((rows, H), dtype=torch.bfloat16, device=partial.device)
        y = torch.empty_like(h) if weight is not None else None
        if residual is not None:
            assert residual.shape == h.shape and residual.is_contiguous() and residual.dtype == torch.bfloat16
        rc = self.lib.vb_tp_allreduce_rmsnorm(a.ptrs, self.pad_alloc.ptrs, off, _lib.ptr(residual), _lib.ptr(weight),
                                              _lib.ptr(y), h.data_ptr(), rows, H, float(eps), self.rank, self.world,
                                              self.CH_TP, self.tp_ctrs.data_ptr(), self._status(), _lib.stream())
        _lib.check(rc, "vb_tp_allreduce_rmsnorm")
        return y, h

    def all_to_all_heads(self, x: torch.Tensor, gather_seq: bool) -> torch.Tensor:
        """The two exchanges of Ulysses sequence parallelism on ``x [rows, heads, D]`` (16-bit elements), one kernel each,
        pulled over peer memory straight into the output layout:

        * ``gather_seq=True``:  ``[T / W, H, D]`` (this rank's tokens, all heads) -> ``[T, H / W, D]`` (all tokens, this
          rank's heads), rank r's tokens at rows ``[r T / W, (r + 1) T / W)``;
        * ``gather_seq=False``: ``[T, H / W, D]`` -> ``[T / W, H, D]``, rank r's heads at ``[r H / W, (r + 1) H / W)``.

        The input is staged in one of two alternating symmetric buffers (rewritten only after a later exchange of this
        communicator has passed its handshake). Collective: same shapes on every rank."""
        W, me = self.world, self.rank
        assert x.dim() == 3 and x.element_size() == 2
        x = x.contiguous()
        n = x.numel()
        key = ("a2a", n, x.dtype)
        bufs = self.__dict__.setdefault("_a2a_bufs", {})
        if key not in bufs:
            bufs[key] = [self.alloc(n, x.dtype, zero=False) for _ in range(2)] + [0]
            self.barrier()
        ent = bufs[key]
        stage = ent[ent[2] & 1]
        ent[2] += 1
        stage.copy_(x.view(-1))
        D = x.shape[2]
        if gather_seq:
            Tl, H = x.shape[0], x.shape[1]
            assert H % W == 0
            Hl = H // W
            chunk = Hl * D
            out = torch.empty((W * Tl, Hl, D), dtype=x.dtype, device=x.device)
            src_base = [me * chunk] * W
            dst_base = [r * Tl * chunk for r in range(W)]
            src_stride, dst_stride, rows = H * D, chunk, Tl
        else:
            T, Hl = x.shape[0], x.shape[1]
            assert T % W == 0
            Tl = T // W
            chunk = Hl * D
            out = torch.empty((Tl, W * Hl, D), dtype=x.dtype, device=x.device)
            src_base = [me * Tl * chunk] * W
            dst_base = [r * chunk for r in range(W)]
            src_stride, dst_stride, rows = chunk, W * chunk, Tl
        assert (chunk * 2) % 16 == 0, "heads-per-rank x head_dim must be a multiple of 8 elements"
        to16 = lambda v: [int(e) * 2 // 16 for e in v]  # noqa: E731
        a, off = self._find(stage)
        LL = ctypes.c_longlong * W
        rc = self.lib.vb_peer_a2a_chunks(a.ptrs, self.pad_alloc.ptrs, off, out.data_ptr(), LL(*to16(src_base)),
                                         LL(*to16(dst_base)), src_stride * 2 // 16, dst_stride * 2 // 16, rows, chunk * 2 // 16,
                                         me, W, self.CH_COPY, self._epoch(self.CH_COPY), self._gate(self.CH_COPY),
                                         self._status(), _lib.stream())
        _lib.check(rc, "vb_peer_a2a_chunks")
        return out

    def check(self):
        """Synchronising read of the status word; raises if a bounded wait ran out."""
        code, blk, detail = _lib.read_status(self.device)
        if code != 0:
            _lib.clear_status(self.device)
            raise RuntimeError(f"peer collective timed out (code {code}, block {blk}, peer/detail {detail})")
