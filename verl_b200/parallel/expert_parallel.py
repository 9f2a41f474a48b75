"""Expert-parallel MoE layer over peer memory (inference: the rollout's EP layout).

Role of DeepEP / vLLM fused-MoE all-to-all under the reference's rollout. Rank ``r`` of the group owns experts
``[r * E / W, (r + 1) * E / W)``; every rank routes its own tokens:

1. the per-rank expert histograms are all-gathered (``E`` ints per rank, peer-memory all-gather), after which every
   rank can compute, on the device and without a host read-back, where its rows of expert ``e`` start in the owner's
   receive buffer. That buffer has the grouped-GEMM layout (rows sorted by expert, every expert padded to 128 rows),
   so nothing is sorted or copied again on the owner;
2. ``vb_moe_dispatch``: a warp per (token, slot) pair stores the token's hidden vector into its row of the owner's
   buffer (512-byte warp stores over NVLink);
3. after a handshake the owner runs its experts with two grouped GEMMs (all local experts in one launch each);
4. ``vb_moe_combine``: after a second handshake a warp per token pulls its ``k`` expert outputs from the owners'
   buffers and writes the routing-weighted sum.

Buffers (symmetric memory): histogram ``[E]``, receive rows ``[cap, H]``, expert outputs ``[cap, H]`` with
``cap = W * max_tokens * k + E_local * 127`` rounded up to 128: the worst case, all tokens of all ranks on one owner.
A smaller ``capacity_rows`` may be given; rows that do not fit are dropped and reported through the status word
(:meth:`PeerComm.check`).
"""

from __future__ import annotations

import ctypes
from typing import Callable, Optional

import torch

from ..ops import _lib
from ..ops.moe import BLK, _grouped

_BOUND = False


def _bind(lib):
    global _BOUND
    if not _BOUND:
        P, I, L, U = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_uint
        lib.vb_moe_dispatch.argtypes, lib.vb_moe_dispatch.restype = [P, P, I, I, I, I, P, P, P, I, P, L, P, P], I
        lib.vb_moe_combine.argtypes, lib.vb_moe_combine.restype = [P, P, P, P, P, I, I, I, I, P, I, I, I, U, P, P, P], I
        lib.vb_moe_hist.argtypes, lib.vb_moe_hist.restype = [P, I, I, P, P], I
        lib.vb_moe_layout.argtypes, lib.vb_moe_layout.restype = [P, I, I, I, I, I, P, P, P, I, P, P], I
        _BOUND = True
    return lib


class ExpertParallelMoE:
    def __init__(self, comm, num_experts: int, hidden: int, top_k: int, max_tokens: int,
                 capacity_rows: Optional[int] = None):
        W = comm.world
        assert num_experts % W == 0 and hidden % 8 == 0 and 1 <= top_k <= 8
        self.comm, self.lib = comm, _bind(comm.lib)
        self.E, self.E_local, self.H, self.k, self.max_tokens = num_experts, num_experts // W, hidden, top_k, max_tokens
        cap = capacity_rows if capacity_rows is not None else W * max_tokens * top_k + self.E_local * (BLK - 1)
        self.cap = (cap + BLK - 1) // BLK * BLK
        dev = comm.device
        # collective allocations: same order and sizes on every rank
        self.hist_sym = comm.alloc(max(num_experts, 64), torch.int32)
        self.recv_x = comm.alloc(self.cap * hidden, torch.bfloat16)
        self.y_sym = comm.alloc(self.cap * hidden, torch.bfloat16)
        self.hist_all = torch.zeros(W * self.hist_sym.numel(), dtype=torch.int32, device=dev)
        self.cursor = torch.zeros(num_experts, dtype=torch.int32, device=dev)
        self.base = torch.zeros(num_experts, dtype=torch.int32, device=dev)
        self.expert_off = torch.zeros(self.E_local + 1, dtype=torch.int32, device=dev)
        self.blk_expert = torch.full((self.cap // BLK,), -1, dtype=torch.int32, device=dev)
        a, off = comm._find(self.recv_x)
        self._recv_ptrs = (ctypes.c_void_p * W)(*[int(p) + off for p in a.ptrs])
        a, off = comm._find(self.y_sym)
        self._y_ptrs = (ctypes.c_void_p * W)(*[int(p) + off for p in a.ptrs])
        comm.barrier()

    def layout(self, top_i32: torch.Tensor):
        """All-gather the histograms of ``top_i32`` ([T, k] int32); returns (base [E] int32: first row of this rank's
        rows of expert e at its owner, blk_expert [cap / 128] int32 and expert_off [E_local + 1] int32 of the rows this
        rank receives). Three launches (histogram, all-gather, layout); also zeroes the dispatch cursors."""
        c, W, E, El = self.comm, self.comm.world, self.E, self.E_local
        stream = _lib.stream()
        rc = self.lib.vb_moe_hist(top_i32.data_ptr(), top_i32.numel(), E, self.hist_sym.data_ptr(), stream)
        _lib.check(rc, "vb_moe_hist")
        c.all_gather(self.hist_all, self.hist_sym, copy_engine=False)  # handshake inside: also orders the buffers' reuse
        rc = self.lib.vb_moe_layout(self.hist_all.data_ptr(), self.hist_sym.numel(), E, El, c.rank, W, self.base.data_ptr(),
                                    self.expert_off.data_ptr(), self.blk_expert.data_ptr(), self.cap // BLK,
                                    self.cursor.data_ptr(), stream)
        _lib.check(rc, "vb_moe_layout")
        return self.base, self.blk_expert, self.expert_off

    @torch.no_grad()
    def forward(self, x: torch.Tensor, top_i: torch.Tensor, top_w: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor,
                act: Callable[[torch.Tensor], torch.Tensor]) -> torch.Tensor:
        """x [T, H] bf16 (this rank's tokens), top_i / top_w [T, k] (global expert ids), gate_up [E_local, 2I, H] and
        down [E_local, H, I] (this rank's experts), ``act``: [P, 2I] -> [P, I]. Returns [T, H]."""
        c = self.comm
        T, H = x.shape
        assert H == self.H and T <= self.max_tokens and top_i.shape == (T, self.k) and x.dtype == torch.bfloat16
        x = x.contiguous()
        ti = top_i.to(torch.int32).contiguous()
        tw = top_w.float().contiguous()
        base, blk_expert, expert_off = self.layout(ti)
        where = torch.empty(T * self.k, dtype=torch.int32, device=x.device)
        status, stream = c._status(), _lib.stream()
        rc = self.lib.vb_moe_dispatch(x.data_ptr(), ti.data_ptr(), T, self.k, H, self.E_local, base.data_ptr(),
                                      self.cursor.data_ptr(), self._recv_ptrs, c.world, where.data_ptr(), self.cap,
                                      status, stream)
        _lib.check(rc, "vb_moe_dispatch")
        c.barrier()  # every rank's rows have arrived
        xs = self.recv_x.view(self.cap, H)
        I2 = gate_up.shape[1]
        h = torch.empty((self.cap, I2), dtype=x.dtype, device=x.device)
        _grouped(xs, gate_up, h, self.cap, I2, H, False, False, False, 1, self.E_local, blk_expert, None)
        a = act(h)
        y = self.y_sym.view(self.cap, H)
        _grouped(a, down, y, self.cap, H, a.shape[1], False, False, False, 1, self.E_local, blk_expert, None)
        out = torch.empty((T, H), dtype=x.dtype, device=x.device)
        rc = self.lib.vb_moe_combine(self._y_ptrs, c.pad_alloc.ptrs, ti.data_ptr(), tw.data_ptr(), where.data_ptr(), T,
                                     self.k, H, self.E_local, out.data_ptr(), c.rank, c.world, c.CH_COPY,
                                     c._epoch(c.CH_COPY), c._gate(c.CH_COPY), status, stream)
        _lib.check(rc, "vb_moe_combine")
        return out


# ---------------------------------------------------------------------------------------------------------------
# Training-side expert parallelism: every rank routes its OWN tokens, sends each (token, slot) pair to the rank that
# owns the expert, runs its experts on what arrives and sends the results back (role of Megatron's token dispatcher
# under the reference's ``expert_model_parallel_size``, verl/workers/config/engine.py:80). Differentiable: the
# backward of an all-to-all is the all-to-all with the split sizes swapped.
import torch.distributed as dist  # noqa: E402


def _all_to_all_rows(x: torch.Tensor, send: list, recv: list, group) -> torch.Tensor:
    """Rows ``x[sum(send[:r]) : sum(send[:r + 1])]`` go to rank r; returns the rows received, in rank order."""
    out = x.new_empty((sum(recv),) + tuple(x.shape[1:]))
    if dist.get_backend(group) == "gloo":
        # gloo has no all-to-all: every rank gathers all buffers and keeps the rows addressed to it (CPU tests)
        W, me = dist.get_world_size(group), dist.get_rank(group)
        cap = torch.tensor([x.shape[0]], dtype=torch.long)
        caps = [torch.zeros(1, dtype=torch.long) for _ in range(W)]
        dist.all_gather(caps, cap, group=group)
        m = int(max(c.item() for c in caps))
        pad = x.new_zeros((m,) + tuple(x.shape[1:]))
        pad[: x.shape[0]] = x
        bufs = [torch.empty_like(pad) for _ in range(W)]
        dist.all_gather(bufs, pad, group=group)
        splits = [None] * W
        dist.all_gather_object(splits, list(send), group=group)
        o = 0
        for r in range(W):
            lo = sum(splits[r][:me])
            n = splits[r][me]
            out[o : o + n] = bufs[r][lo : lo + n]
            o += n
        return out
    dist.all_to_all_single(out, x.contiguous(), output_split_sizes=list(recv), input_split_sizes=list(send), group=group)
    return out


class _AllToAllRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, send, recv, group):
        ctx.send, ctx.recv, ctx.group = send, recv, group
        return _all_to_all_rows(x, send, recv, group)

    @staticmethod
    def backward(ctx, g):
        return _all_to_all_rows(g.contiguous(), ctx.recv, ctx.send, ctx.group), None, None, None


def ep_moe_mlp(x: torch.Tensor, top_i: torch.Tensor, top_w: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, act,
               group, num_experts: int) -> torch.Tensor:
    """Expert-parallel routed MLP for training. ``x [T, H]``: this rank's tokens; ``top_i / top_w [T, k]``: global expert
    ids and weights; ``gate_up [E / W, 2I, H]``, ``down [E / W, H, I]``: this rank's experts (rank r owns experts
    ``[r E / W, (r + 1) E / W)``). Returns ``[T, H]``."""
    from ..ops.moe import moe_mlp

    W = dist.get_world_size(group)
    T, k = top_i.shape
    E_local = num_experts // W
    flat_e = top_i.reshape(-1)
    dest = torch.div(flat_e, E_local, rounding_mode="floor")
    order = torch.argsort(dest, stable=True)
    send = torch.bincount(dest, minlength=W).tolist()          # pairs this rank sends to every rank
    counts = torch.tensor(send, dtype=torch.long, device=x.device)
    got = torch.empty_like(counts)
    if dist.get_backend(group) == "gloo":
        allc = [torch.empty_like(counts) for _ in range(W)]
        dist.all_gather(allc, counts, group=group)
        got = torch.stack(allc)[:, dist.get_rank(group)].contiguous()
    else:
        dist.all_to_all_single(got, counts, group=group)
    recv = got.tolist()
    tok = torch.div(order, k, rounding_mode="floor")
    xs = x.index_select(0, tok)                                 # rows in destination order
    x_in = _AllToAllRows.apply(xs, send, recv, group)
    e_in = _all_to_all_rows((flat_e[order] % E_local).contiguous(), send, recv, group)
    if x_in.shape[0] > 0:
        y_in = moe_mlp(x_in, e_in[:, None], torch.ones(x_in.shape[0], 1, dtype=torch.float32, device=x.device), gate_up, down, act)
    else:  # no token for this rank's experts: keep the graph (and the collectives) alive
        y_in = x_in * 0.0 + 0.0 * (gate_up.sum() + down.sum()).to(x_in.dtype)
    ys = _AllToAllRows.apply(y_in, recv, send, group)           # back in this rank's destination order
    w = top_w.reshape(-1)[order].to(ys.dtype).unsqueeze(-1)
    return torch.zeros_like(x).index_add(0, tok, ys * w)
