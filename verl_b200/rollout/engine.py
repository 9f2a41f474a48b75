"""Native continuous-batching rollout engine with a paged KV cache.

Replaces the vLLM / SGLang servers the reference launches (verl/workers/rollout/vllm_rollout/
vllm_async_server.py, sglang_rollout/*). The scheduler and block manager are C++
(``csrc/scheduler.cpp``); the model runner executes the same transformer weights as the training
engine with the hand-written kernels: prefill = packed varlen attention + KV-cache write, decode =
paged-KV attention, one CUDA graph per padded batch size, sampling fused into one kernel that also
returns the log-prob of the sampled token (what the trainer stores as ``rollout_log_probs``).

Token-in / token-out API: :meth:`add_request`, :meth:`step`, :meth:`generate`, :meth:`abort_request`,
:meth:`sleep` / :meth:`wake_up` (drop / re-create the KV cache), :meth:`update_weights`.
"""

from __future__ import annotations

import os

import ctypes
import time
from dataclasses import dataclass, field
from typing import Iterable, Optional

import numpy as np
import torch

from .. import ops
from ..models import CausalLM, ModelConfig
from ..models.hf_io import hf_to_native_state_dict
from ..ops import _lib


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_k: int = -1
    top_p: float = 1.0
    max_tokens: int = 512
    logprobs: bool = True
    ignore_eos: bool = False
    stop_token_ids: tuple = ()
    n: int = 1

    @classmethod
    def from_dict(cls, d: Optional[dict]) -> "SamplingParams":
        d = dict(d or {})
        if "max_new_tokens" in d and "max_tokens" not in d:
            d["max_tokens"] = d.pop("max_new_tokens")
        if d.get("logprobs") is None:
            d.pop("logprobs", None)
        elif not isinstance(d["logprobs"], bool):
            d["logprobs"] = d["logprobs"] not in (0, False)
        known = {f for f in cls.__dataclass_fields__}
        return cls(**{k: v for k, v in d.items() if k in known})


@dataclass
class TokenOutput:
    """Result of one request (verl/workers/rollout/replica.py:32)."""

    token_ids: list
    log_probs: Optional[list] = None
    routed_experts: Optional[object] = None
    stop_reason: Optional[str] = None  # completed | aborted | length
    num_preempted: int = 0
    request_id: Optional[str] = None


@dataclass
class _Request:
    rid: str
    sid: int
    params: SamplingParams
    prompt_len: int
    logprobs: list = field(default_factory=list)
    done: bool = False
    stop_reason: Optional[str] = None


def _sched_lib():
    lib = _lib.load()
    if not getattr(lib, "_sched_bound", False):
        c = ctypes
        P, I, L = c.c_void_p, c.c_int, c.c_longlong
        lib.vb_sched_create.argtypes, lib.vb_sched_create.restype = [I, I, I, I, I, I], P
        lib.vb_sched_destroy.argtypes, lib.vb_sched_destroy.restype = [P], None
        lib.vb_sched_add.argtypes, lib.vb_sched_add.restype = [P, L, P, I, I], I
        lib.vb_sched_step.argtypes, lib.vb_sched_step.restype = [P], I
        lib.vb_sched_get_step.argtypes, lib.vb_sched_get_step.restype = [P] * 10 + [I], I
        lib.vb_sched_commit.argtypes, lib.vb_sched_commit.restype = [P, P, P, P], None
        lib.vb_sched_output.argtypes, lib.vb_sched_output.restype = [P, L, P, I], I
        lib.vb_sched_preempt_count.argtypes, lib.vb_sched_preempt_count.restype = [P, L], I
        lib.vb_sched_remove.argtypes, lib.vb_sched_remove.restype = [P, L], I
        lib.vb_sched_reset_prefix_cache.argtypes, lib.vb_sched_reset_prefix_cache.restype = [P], None
        lib.vb_sched_stats.argtypes, lib.vb_sched_stats.restype = [P, P], None
        lib.vb_sched_reserve_burst.argtypes, lib.vb_sched_reserve_burst.restype = [P, I], I
        lib.vb_sched_commit_burst.argtypes, lib.vb_sched_commit_burst.restype = [P, P, I, P, P, P], None
        lib.vb_sched_step_limits.argtypes, lib.vb_sched_step_limits.restype = [P, P], None
        lib._sched_bound = True
    return lib


class Scheduler:
    """Thin Python handle on the C++ scheduler."""

    def __init__(self, num_blocks, block_size, max_num_seqs, max_batched_tokens, max_model_len, prefix_caching=True):
        self.lib = _sched_lib()
        self.h = self.lib.vb_sched_create(num_blocks, block_size, max_num_seqs, max_batched_tokens, max_model_len,
                                          int(prefix_caching))
        self.block_size = block_size
        self.max_blocks = (max_model_len + block_size - 1) // block_size
        cap_s, cap_t = max_num_seqs + 8, max_batched_tokens + max_num_seqs + 8
        self.seq_ids = np.zeros(cap_s, np.int64)
        self.seq_ntok = np.zeros(cap_s, np.int32)
        self.seq_start = np.zeros(cap_s, np.int32)
        self.seq_prefill = np.zeros(cap_s, np.int32)
        self.seq_total = np.zeros(cap_s, np.int32)
        self.tokens = np.zeros(cap_t, np.int64)
        self.positions = np.zeros(cap_t, np.int64)
        self.slots = np.zeros(cap_t, np.int64)
        self.block_tables = np.zeros((cap_s, self.max_blocks), np.int32)
        self.done = np.zeros(cap_s, np.int32)
        self.accepted = np.zeros(cap_s, np.int32)
        self.limits = np.zeros(cap_s, np.int32)

    def __del__(self):
        try:
            if self.h:
                self.lib.vb_sched_destroy(self.h)
                self.h = None
        except Exception:
            pass

    def add(self, sid: int, prompt: list[int], max_new_tokens: int) -> int:
        arr = np.asarray(prompt, dtype=np.int32)
        return self.lib.vb_sched_add(self.h, sid, arr.ctypes.data, len(arr), max_new_tokens)

    def step(self) -> tuple[int, int]:
        n = self.lib.vb_sched_step(self.h)
        if n == 0:
            return 0, 0
        p = lambda a: a.ctypes.data  # noqa: E731
        t = self.lib.vb_sched_get_step(self.h, p(self.seq_ids), p(self.seq_ntok), p(self.seq_start), p(self.seq_prefill),
                                       p(self.seq_total), p(self.tokens), p(self.positions), p(self.slots),
                                       p(self.block_tables), self.max_blocks)
        return n, t

    def _fetch(self) -> int:
        p = lambda a: a.ctypes.data  # noqa: E731
        return self.lib.vb_sched_get_step(self.h, p(self.seq_ids), p(self.seq_ntok), p(self.seq_start), p(self.seq_prefill),
                                          p(self.seq_total), p(self.tokens), p(self.positions), p(self.slots),
                                          p(self.block_tables), self.max_blocks)

    def reserve_burst(self, k: int) -> int:
        """Pages for up to ``k`` consecutive decode steps of the planned (pure decode) step; returns the number of
        steps covered (1 = no burst) and refreshes the block tables."""
        got = self.lib.vb_sched_reserve_burst(self.h, int(k))
        if got > 1:
            self._fetch()
        return got

    def step_limits(self, n: int) -> np.ndarray:
        self.lib.vb_sched_step_limits(self.h, self.limits.ctypes.data)
        return self.limits[:n]

    def commit_burst(self, toks: np.ndarray, finished_at: np.ndarray):
        """toks [k, n] int64, finished_at [n] int32 (1-based step of the caller's stop, 0 = none) -> (accepted, done)."""
        k, n = toks.shape
        toks = np.ascontiguousarray(toks, dtype=np.int64)
        finished_at = np.ascontiguousarray(finished_at, dtype=np.int32)
        self.lib.vb_sched_commit_burst(self.h, toks.ctypes.data, int(k), finished_at.ctypes.data, self.accepted.ctypes.data,
                                       self.done.ctypes.data)
        return self.accepted[:n], self.done[:n]

    def commit(self, new_tokens: np.ndarray, finished: np.ndarray) -> np.ndarray:
        n = len(new_tokens)
        self.lib.vb_sched_commit(self.h, new_tokens.ctypes.data, finished.ctypes.data, self.done.ctypes.data)
        return self.done[:n]

    def output(self, sid: int, cap: int) -> list[int]:
        buf = np.zeros(max(cap, 1), np.int32)
        n = self.lib.vb_sched_output(self.h, sid, buf.ctypes.data, len(buf))
        return buf[: max(n, 0)].tolist()

    def preempt_count(self, sid: int) -> int:
        return self.lib.vb_sched_preempt_count(self.h, sid)

    def remove(self, sid: int) -> bool:
        return bool(self.lib.vb_sched_remove(self.h, sid))

    def reset_prefix_cache(self):
        self.lib.vb_sched_reset_prefix_cache(self.h)

    def stats(self) -> dict:
        out = np.zeros(6, np.int64)
        self.lib.vb_sched_stats(self.h, out.ctypes.data)
        return dict(zip(("waiting", "running", "free_pages", "preempted", "prefix_hits", "prefix_queries"), out.tolist()))


class NativeRolloutEngine:
    def __init__(self, model: CausalLM, *, max_num_seqs: int = 256, max_model_len: int = 2048,
                 max_num_batched_tokens: int = 8192, block_size: int = 16, num_blocks: Optional[int] = None,
                 gpu_memory_utilization: float = 0.5, enable_prefix_caching: bool = True, enforce_eager: bool = False,
                 seed: int = 0, eos_token_id: Optional[int] = None, cudagraph_capture_sizes: Optional[list] = None,
                 quantization: Optional[str] = None, tp_group=None, tp_comm=None, full_config: Optional[ModelConfig] = None,
                 decode_burst: int = 16, record_routing: bool = False):
        """``model``: the whole model, or (tensor parallelism) this rank's slice of it as laid out by
        :func:`verl_b200.parallel.reshard.tp_model_config`, with ``tp_group`` the replica's process group, ``tp_comm``
        its peer-memory communicator (CUDA) and ``full_config`` the architecture of the whole model. Every rank of a
        replica runs the same scheduler on the same requests and samples the same tokens (the all-reduced activations
        are bit-identical on all ranks), so the ranks need no control traffic besides the activation all-reduces."""
        self.model = model
        # up to this many decode steps run back to back on the device (each step's last kernel prepares the next
        # step's inputs); the host reads their tokens in one go. 1 = the host takes part in every step.
        self.decode_burst = max(1, min(int(decode_burst), 64))
        self.tp_group, self.tp_comm = tp_group, tp_comm
        self.tp = 1
        if tp_group is not None:
            import torch.distributed as dist

            self.tp = dist.get_world_size(tp_group)
            self.tp_rank = dist.get_rank(tp_group)
        self.full_cfg: ModelConfig = full_config if full_config is not None else model.cfg
        self._tp_bufs: list = []
        if quantization not in (None, "", "fp8"):
            raise ValueError(f"unsupported rollout quantization {quantization!r} (supported: fp8)")
        self.quantization = quantization or None
        self._fp8: dict[int, tuple] = {}
        self.cfg: ModelConfig = model.cfg
        self.device = model.embed_tokens.weight.device
        self.dtype = model.embed_tokens.weight.dtype
        self.on_gpu = self.device.type == "cuda"
        self.max_num_seqs = max_num_seqs
        self.max_model_len = max_model_len
        self.max_num_batched_tokens = max(max_num_batched_tokens, 16)
        self.block_size = block_size
        self.enable_prefix_caching = enable_prefix_caching
        # mixture-of-experts models: keep, per request, the experts every INPUT token was routed to in every layer
        # (``TokenOutput.routed_experts [prompt + response tokens, layers, top-k]``; the trainer replays them, router
        # replay mode R3). Tokens served from the prefix cache are never routed, so the cache is off while recording.
        self.record_routing = bool(record_routing) and self.cfg.is_moe
        self._routing: dict[int, np.ndarray] = {}
        if self.record_routing:
            self.enable_prefix_caching = False
        self.enforce_eager = enforce_eager or not self.on_gpu
        self.seed = seed
        self.eos = self.cfg.eos_token_id if eos_token_id is None else eos_token_id
        self.gpu_memory_utilization = gpu_memory_utilization
        self._num_blocks_arg = num_blocks
        self.k_cache: list = []
        self._kv_store = None  # one allocation behind the per-layer K / V views
        self.v_cache: list = []
        self.sched: Optional[Scheduler] = None
        self.requests: dict[int, _Request] = {}
        self._mmreq: dict[int, dict] = {}  # per-request multimodal state of vision-language models
        self.by_rid: dict[str, int] = {}
        self._next_sid = 0
        self._graphs: dict[int, tuple] = {}
        self._capture_sizes = cudagraph_capture_sizes
        self.step_counter = torch.zeros(1, dtype=torch.long, device=self.device)
        self.stats = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "decode_steps": 0, "step_s": 0.0,
                      "decode_wait_s": 0.0, "prefill_s": 0.0}
        if self.tp > 1 and self.on_gpu:
            if tp_comm is None:
                raise ValueError("a tensor-parallel rollout replica on CUDA needs its peer-memory communicator (tp_comm)")
            # Partial products of the row-parallel GEMMs, read by the peers' all-reduce kernels: two alternating buffers
            # for the decode path and two for the prefill path (a buffer is rewritten only after a later all-reduce of
            # the replica has passed its handshake; both paths run an even number of all-reduces)
            rows = max(self.max_num_batched_tokens + self.max_num_seqs, self.max_num_seqs) + 8
            self._tp_rows = rows
            self._tp_bufs = [tp_comm.alloc(rows * self.cfg.hidden_size, torch.bfloat16, zero=False) for _ in range(4)]
            tp_comm.barrier()
        self.wake_up()
        self.refresh_quantization()

    # ----------------------------------------------------------------- memory
    def _page_bytes(self) -> int:
        c = self.cfg
        return 2 * c.num_hidden_layers * c.num_key_value_heads * self.block_size * c.head_dim * 2

    def wake_up(self, tags: Optional[list] = None):
        """(Re-)create the KV cache and scheduler state. ``tags`` may name "kv_cache" / "weights" as in the
        reference's multi-stage wake-up; weights are owned by the caller, so only "kv_cache" acts here."""
        if tags is not None and "kv_cache" not in tags:
            return
        if self.sched is not None and self.k_cache:
            return
        if self._num_blocks_arg is not None:
            nb = self._num_blocks_arg
        elif self.on_gpu:
            free, total = torch.cuda.mem_get_info(self.device)
            budget = int(min(free * 0.9, total * self.gpu_memory_utilization))
            nb = max(budget // self._page_bytes(), 64)
            nb = min(nb, self.max_num_seqs * ((self.max_model_len + self.block_size - 1) // self.block_size) + 64)
        else:
            nb = self.max_num_seqs * ((self.max_model_len + self.block_size - 1) // self.block_size) + 8
        if self.tp > 1:  # the ranks of a replica must run identical schedulers: agree on the smallest cache
            import torch.distributed as dist

            t = torch.tensor([int(nb)], dtype=torch.int64, device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.tp_group)
            nb = int(t.item())
        self.num_blocks = int(nb)
        c = self.cfg
        shape = (self.num_blocks, c.num_key_value_heads, self.block_size, c.head_dim)
        # ONE allocation for the K and V pages of all layers: freeing it on sleep() is one driver call instead of one
        # per layer and side (with peer access enabled every cudaFree of a large block is expensive)
        L = c.num_hidden_layers
        self._kv_store = torch.zeros((2 * L,) + shape, dtype=self.dtype, device=self.device)
        self.k_cache = [self._kv_store[i] for i in range(L)]
        self.v_cache = [self._kv_store[L + i] for i in range(L)]
        self.sched = Scheduler(self.num_blocks, self.block_size, self.max_num_seqs, self.max_num_batched_tokens,
                               self.max_model_len, self.enable_prefix_caching)
        self._graphs = {}

    def sleep(self):
        """Free the KV cache (and captured graphs). Running requests must have been drained or aborted."""
        self.abort_all_requests()
        self.k_cache, self.v_cache, self._graphs = [], [], {}
        self._kv_store = None
        self.sched = None
        if self.on_gpu:
            torch.cuda.empty_cache()

    def clear_kv_cache(self):
        if self.sched is not None:
            self.sched.reset_prefix_cache()

    # ---------------------------------------------------------------- weights
    @torch.no_grad()
    def update_weights(self, weights: Iterable[tuple[str, torch.Tensor]], **kwargs):
        """Load HF-named tensors into the engine's (fused-layout) parameters. When the engine shares its
        module with the trainer on the same device this is unnecessary; it serves separate replicas."""
        hf = {k: v for k, v in weights}
        native = hf_to_native_state_dict(self.full_cfg, hf)
        if self.tp > 1:
            from ..parallel.reshard import shard_state_dict

            native = shard_state_dict(self.full_cfg, native, self.tp_rank, self.tp)
        own = dict(self.model.named_parameters())
        for k, v in native.items():
            if k in own:
                own[k].data.copy_(v.to(own[k].dtype))
        self.refresh_quantization()
        self.clear_kv_cache()

    # --------------------------------------------------------------- requests
    def add_request(self, request_id: str, prompt_ids: list[int], sampling_params=None,
                    multi_modal_inputs: Optional[dict] = None) -> None:
        """``multi_modal_inputs`` (vision-language models): ``{"pixel_values": [patches, C * T * P * P],
        "image_grid_thw": [n_images, 3]}`` for the image placeholder tokens of ``prompt_ids``, as an HF image processor
        returns them (role of the multimodal inputs of verl/workers/rollout/vllm_rollout/vllm_async_server.py:445-547)."""
        if self.sched is None:
            self.wake_up()
        sp = sampling_params if isinstance(sampling_params, SamplingParams) else SamplingParams.from_dict(sampling_params)
        max_new = min(sp.max_tokens, self.max_model_len - len(prompt_ids))
        sid = self._next_sid
        self._next_sid += 1
        sched_ids = list(prompt_ids)
        mm = None
        if multi_modal_inputs and (multi_modal_inputs.get("pixel_values") is not None
                                   or multi_modal_inputs.get("pixel_values_videos") is not None):
            mm, sched_ids = self._prepare_multimodal(prompt_ids, multi_modal_inputs)
        rc = self.sched.add(sid, sched_ids, max_new)
        if rc != 0:
            raise ValueError(f"request {request_id}: prompt of {len(prompt_ids)} tokens does not fit (code {rc})")
        self.requests[sid] = _Request(request_id, sid, sp, len(prompt_ids))
        self.by_rid[request_id] = sid
        if self.record_routing:
            self._routing[sid] = np.zeros((len(prompt_ids) + max(max_new, 0), self.cfg.num_hidden_layers,
                                           self.cfg.num_experts_per_tok), np.int16)
        if mm is not None:
            self._mmreq[sid] = mm

    @torch.no_grad()
    def _prepare_multimodal(self, prompt_ids: list[int], inputs: dict):
        """Run the vision tower once for the request and keep what prefill and decode need: the image embeddings, the
        prompt indices of the placeholder tokens, the [3, L] multimodal RoPE positions and the offset of later text
        positions. The scheduler sees salted ids (>= vocabulary size, derived from the pixels) in place of the
        placeholder tokens, so that prompts with the same text but other images never share prefix-cache pages."""
        from ..models.vision import get_rope_index

        cfg = self.full_cfg
        if getattr(self.model, "visual", None) is None:
            raise ValueError("multi_modal_inputs were given but the model has no vision tower")
        img_grid = inputs["image_grid_thw"] if inputs.get("pixel_values") is not None else None
        vid_grid = inputs["video_grid_thw"] if inputs.get("pixel_values_videos") is not None else None
        # one tower call over the images' patches followed by the videos' (as the training forward does)
        pv = torch.cat([inputs[k] for k, g in (("pixel_values", img_grid), ("pixel_values_videos", vid_grid))
                        if g is not None], 0).to(self.device)
        grid = torch.cat([g for g in (img_grid, vid_grid) if g is not None], 0).to(self.device)
        taps = []
        if self.model.visual.num_deepstack:  # Qwen3-VL: features for the image tokens' hidden states after the first layers
            emb, taps = self.model.visual(pv, grid, return_deepstack=True)
            taps = [t.to(self.dtype) for t in taps]
        else:
            emb = self.model.visual(pv, grid)
        emb = emb.to(self.dtype)
        ids = torch.tensor(prompt_ids, dtype=torch.long)
        vid_tok = cfg.extra.get("video_token_id")
        where = torch.nonzero(ids == cfg.image_token_id, as_tuple=True)[0] if img_grid is not None else ids.new_zeros(0)
        if vid_grid is not None:
            where = torch.cat([where, torch.nonzero(ids == int(vid_tok), as_tuple=True)[0]])
        if where.numel() != emb.shape[0]:
            raise ValueError(f"{where.numel()} vision placeholder tokens but {emb.shape[0]} vision embeddings")
        # prefill looks rows up by position: keep them (and their embeddings) in prompt order
        where, order = torch.sort(where)
        emb = emb[order.to(emb.device)]
        taps = [t[order.to(t.device)] for t in taps]
        merge = int(cfg.extra["vision_config"].get("spatial_merge_size", 2))
        pos3, delta = get_rope_index(ids, img_grid.cpu() if img_grid is not None else None, cfg.image_token_id, merge,
                                     video_grid_thw=vid_grid.cpu() if vid_grid is not None else None,
                                     video_token_id=None if vid_tok is None else int(vid_tok))
        salt = int(pv.float().sum().item() * 1000003) & 0x3FFFFFFF
        room = (1 << 31) - 1 - cfg.vocab_size
        sched = list(prompt_ids)
        for j, w in enumerate(where.tolist()):
            sched[w] = cfg.vocab_size + (salt + 7919 * j) % room
        return {"emb": emb, "taps": taps, "where": where.numpy(), "pos3": pos3.numpy(), "delta": int(delta)}, sched

    def _finish(self, sid: int, reason: str) -> TokenOutput:
        req = self.requests.pop(sid)
        self._mmreq.pop(sid, None)
        self.by_rid.pop(req.rid, None)
        toks = self.sched.output(sid, self.max_model_len)
        pre = self.sched.preempt_count(sid)
        self.sched.remove(sid)
        lps = req.logprobs[: len(toks)] if req.params.logprobs else None
        routed = self._routing.pop(sid, None)
        if routed is not None:
            routed = routed[: req.prompt_len + len(toks)]
            if len(toks):
                routed[-1] = 0  # the last token was never an input (a burst that ran past the end may have fed it)
        return TokenOutput(token_ids=toks, log_probs=lps, routed_experts=routed, stop_reason=reason,
                           num_preempted=max(pre, 0), request_id=req.rid)

    def abort_request(self, request_id: str) -> Optional[TokenOutput]:
        """Stop a request; the partial output is returned with ``stop_reason="aborted"``."""
        sid = self.by_rid.get(request_id)
        if sid is None:
            return None
        return self._finish(sid, "aborted")

    def abort_all_requests(self) -> list[TokenOutput]:
        if self.sched is None:
            return []
        return [self._finish(sid, "aborted") for sid in list(self.requests.keys())]

    def has_unfinished(self) -> bool:
        return bool(self.requests)

    # ------------------------------------------------------------ model pieces
    def _layer_attn_in(self, layer, x, positions):
        c = self.cfg
        att = layer.self_attn
        qkv = self._mm(x, att.qkv_proj.weight, att.qkv_proj.bias)
        T = x.shape[0]
        if c.qk_norm:
            q, k, v = qkv.split([c.q_size, c.kv_size, c.kv_size], dim=-1)
            q, _ = ops.rmsnorm(q.reshape(T * c.num_attention_heads, c.head_dim).contiguous(), att.q_norm.weight, c.rms_norm_eps)
            k, _ = ops.rmsnorm(k.reshape(T * c.num_key_value_heads, c.head_dim).contiguous(), att.k_norm.weight, c.rms_norm_eps)
            qkv = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v], dim=-1)
        rope = self.model.rope(self.device)
        qkv = ops.rope_qkv(qkv, positions, rope[0], rope[1], c.num_attention_heads, c.num_key_value_heads, c.head_dim,
                           mrope_section=c.mrope_section if positions.dim() == 2 else None,
                           mrope_interleaved=bool(getattr(c, "mrope_interleaved", False)))
        q = qkv[:, : c.q_size].view(T, c.num_attention_heads, c.head_dim)
        k = qkv[:, c.q_size : c.q_size + c.kv_size].view(T, c.num_key_value_heads, c.head_dim)
        v = qkv[:, c.q_size + c.kv_size :].view(T, c.num_key_value_heads, c.head_dim)
        return q, k, v

    def refresh_quantization(self) -> None:
        """fp8 rollout (``rollout.quantization = fp8``): block-quantise the projection weights of every layer (e4m3,
        one scale per 128 x 128 block). Call after every weight sync: the trainer's bf16 weights are the source
        (quantise-on-resync of verl/utils/vllm/vllm_fp8_utils.py:182-431)."""
        self._fp8.clear()
        if self.quantization != "fp8" or not self.on_gpu:
            return
        from ..ops import fp8

        # routed experts (no grouped fp8 GEMM) and the two-matrix xIELU MLP stay in bf16: for those models the
        # attention projections alone are quantised
        dense_mlp = not self.cfg.is_moe and self.cfg.mlp_gated
        for layer in self.model.layers:
            ws = [layer.self_attn.qkv_proj.weight, layer.self_attn.o_proj.weight]
            if dense_mlp:
                ws += [layer.mlp.gate_up_proj.weight, layer.mlp.down_proj.weight]
            for w in ws:
                if w.numel():
                    self._fp8[id(w)] = fp8.quantize_weight(w.data)

    def _mm(self, x, w, bias=None):
        q = self._fp8.get(id(w))
        if q is not None:
            from ..ops import fp8

            return fp8.fp8_linear(x, q[0], q[1], bias)
        if self.on_gpu:
            return ops.gemm(x, w, bias=bias)
        return torch.nn.functional.linear(x, w, bias)

    def _mm_partial(self, x, w, slot: int, path: int):
        """Row-parallel GEMM. Tensor parallelism on CUDA: the partial product goes straight into the symmetric buffer
        ``2 * path + slot`` (path 0 = decode, 1 = prefill) that the peers' all-reduce kernels read."""
        if self.tp == 1 or not self.on_gpu:
            return self._mm(x, w)
        buf = self._tp_bufs[2 * path + slot][: x.shape[0] * w.shape[0]].view(x.shape[0], w.shape[0])
        q = self._fp8.get(id(w))
        if q is not None:
            from ..ops import fp8

            buf.copy_(fp8.fp8_linear(x, q[0], q[1], None))
        else:
            ops.gemm(x, w, out=buf)
        return buf

    def _to_partial(self, y, slot: int, path: int):
        if self.tp == 1 or not self.on_gpu:
            return y
        buf = self._tp_bufs[2 * path + slot][: y.numel()].view(y.shape)
        buf.copy_(y)
        return buf

    def _reduce_norm(self, partial, norm_w, residual):
        """(rmsnorm(h) * norm_w, h) with h = sum over the replica's ranks of ``partial`` + ``residual``: one fused
        all-reduce + residual + RMSNorm kernel over peer memory; plain RMSNorm without tensor parallelism."""
        eps = self.cfg.rms_norm_eps
        if self.tp == 1:
            return ops.rmsnorm(partial, norm_w, eps, residual)
        if self.on_gpu:
            return self.tp_comm.tp_allreduce_rmsnorm(partial, residual, norm_w, eps)
        import torch.distributed as dist

        partial = partial.contiguous()
        dist.all_reduce(partial, group=self.tp_group)
        return ops.rmsnorm(partial, norm_w, eps, residual)

    def _forward_layers(self, h, attend, path: int, inject: Optional[dict] = None):
        """Decoder stack on embedded tokens ``h [T, H]``; ``attend(li, layer, x)`` returns the attention output of the
        layer's (local) heads for the normalised input ``x``. Returns the final-norm hidden states. Every RMSNorm after
        the first one is fused with the residual add (and, under tensor parallelism, with the all-reduce of the
        preceding row-parallel GEMM). ``inject[li] = (rows, values)``: added to the hidden states of ``rows`` after
        layer ``li`` (the deepstack vision features of Qwen3-VL)."""
        c = self.cfg
        layers = self.model.layers
        T = h.shape[0]
        x, residual = ops.rmsnorm(h, layers[0].input_layernorm.weight, c.rms_norm_eps, None)
        for li, layer in enumerate(layers):
            attn = attend(li, layer, x)
            o = self._mm_partial(attn.reshape(T, c.q_size), layer.self_attn.o_proj.weight, 0, path)
            x, residual = self._reduce_norm(o, layer.post_attention_layernorm.weight, residual)
            if c.is_moe or not c.mlp_gated:  # routed experts / the two-matrix xIELU MLP: the module's own forward
                d = self._to_partial(layer.mlp(x), 1, path)
            else:
                d = self._mm_partial(ops.swiglu(self._mm(x, layer.mlp.gate_up_proj.weight)), layer.mlp.down_proj.weight,
                                     1, path)
            if inject and li in inject and (self.tp == 1 or self.tp_rank == 0):
                # ``d`` is this rank's partial sum under tensor parallelism: one rank adds the (replicated) values
                d.index_add_(0, inject[li][0], inject[li][1].to(d.dtype))
            nw = layers[li + 1].input_layernorm.weight if li + 1 < len(layers) else self.model.norm.weight
            x, residual = self._reduce_norm(d, nw, residual)
        return x

    def _routing_snapshot(self) -> torch.Tensor:
        """[tokens of the latest forward, layers, top-k] expert ids (int16, on the device)."""
        return torch.stack([layer.mlp.last_routing for layer in self.model.layers], dim=1).to(torch.int16)

    def _routing_store(self, sid: int, start: int, rows: np.ndarray) -> None:
        buf = self._routing.get(sid)
        if buf is not None and start < buf.shape[0]:
            n = min(rows.shape[0], buf.shape[0] - start)
            buf[start : start + n] = rows[:n]

    def _final_logits(self, x):
        w = self.model.lm_head_weight
        logits = ops.gemm(x, w, out_dtype=torch.float32) if self.on_gpu else x.float() @ w.float().t()
        ban = getattr(self, "_banned_ids", None)
        if ban is None:
            # vision-language models: the image placeholder id stands for pixels and is never a token to generate (a
            # sampled one would be taken for an image by every later consumer of the sequence)
            c = self.full_cfg
            ids = [c.image_token_id] if getattr(c, "is_vl", False) and c.image_token_id is not None else []
            if ids and c.extra.get("video_token_id") is not None:
                ids.append(int(c.extra["video_token_id"]))
            ban = self._banned_ids = torch.tensor(ids, dtype=torch.long, device=self.device)
        if ban.numel():
            logits.index_fill_(1, ban, float("-inf"))
        return logits

    # ------------------------------------------------------------------ decode
    @torch.no_grad()
    def _decode_forward(self, ids, positions, slots, block_table, seq_lens, splits, work):
        h = ops.embedding(ids, self.model.embed_tokens.weight)

        def attend(li, layer, x):
            q, k, v = self._layer_attn_in(layer, x, positions)
            ops.kv_cache_write(k, v, slots, self.k_cache[li], self.v_cache[li])
            return ops.paged_decode_attention(q, self.k_cache[li], self.v_cache[li], block_table, seq_lens,
                                              num_splits=splits, work=work)

        return self._final_logits(self._forward_layers(h, attend, 0))

    def _graph_sizes(self):
        if self._capture_sizes:
            return sorted(self._capture_sizes)
        sizes, b = [], 1
        while b < self.max_num_seqs:
            sizes.append(b)
            b *= 2
        sizes.append(self.max_num_seqs)
        return sizes

    def _get_graph(self, B: int):
        """Static buffers + captured graph for a padded decode batch of B sequences."""
        if B in self._graphs:
            return self._graphs[B]
        dev, c = self.device, self.cfg
        mb = self.sched.max_blocks
        # All per-step inputs live in ONE device buffer that is filled by ONE copy from a pinned host mirror, the
        # two outputs in one more buffer that comes back in one copy: a decode step costs two small transfers.
        fields = [("ids", np.int64, (B,), 0), ("pos", np.int64, (B,), 0), ("slots", np.int64, (B,), -1),
                  ("lens", np.int32, (B,), 1), ("temp", np.float32, (B,), 1.0), ("topk", np.int32, (B,), -1),
                  ("topp", np.float32, (B,), 1.0), ("limit", np.int32, (B,), 0), ("alive", np.int32, (B,), 0),
                  ("flags", np.int32, (B,), 0), ("bpos", np.int32, (1,), 0), ("bt", np.int32, (B, mb), 0)]
        off, layout = 0, {}
        for name, dt, shape, _ in fields:
            nb = int(np.prod(shape)) * np.dtype(dt).itemsize
            layout[name] = (off, nb)
            off = (off + nb + 255) // 256 * 256
        pin = dev.type == "cuda"
        K = self.decode_burst
        host = torch.zeros(off, dtype=torch.uint8, pin_memory=pin)
        devbuf = torch.zeros(off, dtype=torch.uint8, device=dev)
        # ring of the burst's results: K rows of B tokens (int64) followed by K rows of B log-probs (fp32)
        out_dev = torch.zeros(K * B * 12, dtype=torch.uint8, device=dev)
        out_host = torch.zeros(K * B * 12, dtype=torch.uint8, pin_memory=pin)
        tdt = {np.int64: torch.int64, np.int32: torch.int32, np.float32: torch.float32}
        st = {"host": {}, "pad": {}, "host_buf": host, "dev_buf": devbuf, "out_dev": out_dev, "out_host": out_host,
              "sig": None}
        hnp = host.numpy()
        for name, dt, shape, pad in fields:
            o, nb = layout[name]
            st[name] = devbuf[o : o + nb].view(tdt[dt]).view(shape)
            st["host"][name] = hnp[o : o + nb].view(dt).reshape(shape)
            st["host"][name][...] = pad
            st["pad"][name] = pad
        devbuf.copy_(host)
        st["ring_tok"] = out_dev[: K * B * 8].view(torch.int64).view(K, B)
        st["ring_lp"] = out_dev[K * B * 8 :].view(torch.float32).view(K, B)
        st["host_tok"] = out_host.numpy()[: K * B * 8].view(np.int64).reshape(K, B)
        st["host_lp"] = out_host.numpy()[K * B * 8 :].view(np.float32).reshape(K, B)
        st["tok"] = torch.zeros(B, dtype=torch.int64, device=dev)
        st["lp"] = torch.zeros(B, dtype=torch.float32, device=dev)
        if self.record_routing:  # the burst's routing records: row s = step s of the burst
            shape = (K, B, c.num_hidden_layers, c.num_experts_per_tok)
            st["ring_rt"] = torch.zeros(shape, dtype=torch.int16, device=dev)
            st["rt_host"] = torch.zeros(shape, dtype=torch.int16, pin_memory=pin)
        splits, work = ops.decode_workspace(B, c.num_attention_heads, c.num_key_value_heads, c.head_dim,
                                            self.max_model_len, dev)
        st["splits"], st["work"] = splits, work
        eos = -1 if self.eos is None else int(self.eos)

        def run():
            logits = self._decode_forward(st["ids"], st["pos"], st["slots"], st["bt"], st["lens"], splits, work)
            if self.record_routing:  # before decode_advance moves the burst position on
                st["ring_rt"].index_copy_(0, st["bpos"].long(), self._routing_snapshot().unsqueeze(0))
            ops.sample(logits, temperature=st["temp"], top_k=st["topk"], top_p=st["topp"], seed=self.seed,
                       step=self.step_counter, out_tokens=st["tok"], out_logprobs=st["lp"])
            ops.decode_advance(st["tok"], st["lp"], st["ids"], st["pos"], st["slots"], st["lens"], st["bt"],
                               self.block_size, st["limit"], st["alive"], st["flags"], eos, st["ring_tok"], st["ring_lp"],
                               st["bpos"], self.step_counter)

        graph = None
        if not self.enforce_eager:
            s = torch.cuda.Stream(device=dev)
            s.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(s):
                run()  # warm-up (also sets func attributes, fills caches)
            torch.cuda.current_stream(dev).wait_stream(s)
            torch.cuda.synchronize(dev)
            graph = torch.cuda.CUDAGraph()
            # thread-local capture mode: CUDA calls made by other threads of the process (a checkpoint writer, a
            # profiler, another engine's loop) must not invalidate this capture
            mode = os.environ.get("VERL_B200_GRAPH_CAPTURE_MODE", "thread_local")
            # Cyclic garbage (an earlier engine with its graphs and pinned buffers) must not be finalised in the
            # middle of the capture: destroying graphs or freeing memory there invalidates it. Collect now, and
            # keep the collector off until the capture has ended.
            import gc

            gc.collect()
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph, capture_error_mode=mode):
                    run()
            finally:
                if gc_was_on:
                    gc.enable()
        self._graphs[B] = (st, graph, run)
        return self._graphs[B]

    def _pad_batch(self, n: int) -> int:
        for b in self._graph_sizes():
            if b >= n:
                return b
        return n

    # ----------------------------------------------------------------- prefill
    @torch.no_grad()
    def _prefill_forward(self, seq_idx: list[int], tok_lo: list[int]):
        """Run the scheduled prefill chunks. Returns logits [num_prefill_seqs, V] at each chunk's last token."""
        sc, c, dev = self.sched, self.cfg, self.device
        ids_l, pos_l, slot_l, cu, ctx_lens = [], [], [], [0], []
        for i, lo in zip(seq_idx, tok_lo):
            n = int(sc.seq_ntok[i])
            ids_l.append(sc.tokens[lo : lo + n])
            pos_l.append(sc.positions[lo : lo + n])
            slot_l.append(sc.slots[lo : lo + n])
            cu.append(cu[-1] + n)
            ctx_lens.append(int(sc.seq_start[i]))
        ids = torch.from_numpy(np.concatenate(ids_l)).to(dev)
        pos = torch.from_numpy(np.concatenate(pos_l)).to(dev)
        slots = torch.from_numpy(np.concatenate(slot_l)).to(dev)
        T = ids.numel()
        cu_q = torch.tensor(cu, dtype=torch.int32, device=dev)
        max_q = max(b - a for a, b in zip(cu[:-1], cu[1:]))
        has_ctx = any(x > 0 for x in ctx_lens)
        if has_ctx:
            # gather indices of the cached context (block, offset) and the order that interleaves
            # [context | new tokens] per sequence for the key/value side
            blk_l, off_l, order, cu_k = [], [], [], [0]
            n_ctx_total = sum(ctx_lens)
            ctx_off = 0
            for j, (i, ctx) in enumerate(zip(seq_idx, ctx_lens)):
                if ctx:
                    p = np.arange(ctx)
                    blk_l.append(sc.block_tables[i, p // self.block_size])
                    off_l.append(p % self.block_size)
                    order.append(np.arange(ctx_off, ctx_off + ctx))
                    ctx_off += ctx
                order.append(n_ctx_total + np.arange(cu[j], cu[j + 1]))
                cu_k.append(cu_k[-1] + ctx + cu[j + 1] - cu[j])
            blk = torch.from_numpy(np.concatenate(blk_l).astype(np.int64)).to(dev)
            off = torch.from_numpy(np.concatenate(off_l).astype(np.int64)).to(dev)
            order_t = torch.from_numpy(np.concatenate(order)).to(dev)
            cu_k_t = torch.tensor(cu_k, dtype=torch.int32, device=dev)
            max_k = max(b - a for a, b in zip(cu_k[:-1], cu_k[1:]))
        vl = bool(self.full_cfg.is_vl)
        inject = None
        if vl:
            # salted placeholder ids (>= vocabulary) look up row 0; their embeddings are replaced below
            ids = torch.where(ids < self.full_cfg.vocab_size, ids, torch.zeros_like(ids))
        h = ops.embedding(ids, self.model.embed_tokens.weight)
        if vl:
            # multimodal RoPE: [3, T] positions; a request with images takes them from its table (its text after the
            # images is offset by the request's delta), the others advance all three axes together
            pos3 = pos.unsqueeze(0).repeat(3, 1)
            ds_rows, ds_vals = [], []
            for j, i in enumerate(seq_idx):
                mm = self._mmreq.get(int(sc.seq_ids[i]))
                if mm is None:
                    continue
                st, n = int(sc.seq_start[i]), cu[j + 1] - cu[j]
                L = mm["pos3"].shape[1]
                tok = np.arange(st, st + n)
                p3 = np.where(tok[None, :] < L, mm["pos3"][:, np.minimum(tok, L - 1)], tok[None, :] + mm["delta"])
                pos3[:, cu[j] : cu[j + 1]] = torch.from_numpy(p3).to(dev)
                hit = (mm["where"] >= st) & (mm["where"] < st + n)
                if hit.any():
                    k0 = int(np.searchsorted(mm["where"], st))
                    rows_ = torch.from_numpy(mm["where"][hit] - st + cu[j]).to(dev)
                    h = h.index_put((rows_,), mm["emb"][k0 : k0 + int(hit.sum())])
                    if mm.get("taps"):
                        ds_rows.append(rows_)
                        ds_vals.append([t[k0 : k0 + int(hit.sum())] for t in mm["taps"]])
            pos = pos3
            if ds_rows:
                rows_all = torch.cat(ds_rows)
                inject = {li: (rows_all, torch.cat([v[li] for v in ds_vals])) for li in range(len(ds_vals[0]))}

        def attend(li, layer, x):
            q, k, v = self._layer_attn_in(layer, x, pos)
            ops.kv_cache_write(k, v, slots, self.k_cache[li], self.v_cache[li])
            if not has_ctx:
                return ops.attention_varlen(q, k, v, cu_q, max_q, causal=True)
            k_all = torch.cat([self.k_cache[li][blk, :, off], k], dim=0)[order_t]
            v_all = torch.cat([self.v_cache[li][blk, :, off], v], dim=0)[order_t]
            return _varlen_attention_kv(q, k_all, v_all, cu_q, cu_k_t, max_q, max_k)

        x = self._forward_layers(h, attend, 1, inject)
        if self.record_routing:
            rt = self._routing_snapshot().cpu().numpy()
            for j, i in enumerate(seq_idx):
                self._routing_store(int(sc.seq_ids[i]), int(sc.seq_start[i]), rt[cu[j] : cu[j + 1]])
        last = torch.tensor([b - 1 for b in cu[1:]], dtype=torch.long, device=dev)
        return self._final_logits(x[last])

    # -------------------------------------------------------------------- step
    @torch.no_grad()
    def step(self) -> list[TokenOutput]:
        """One scheduler iteration. Returns the requests that finished in it."""
        sc = self.sched
        t_step = time.perf_counter()
        n, _ = sc.step()
        if n == 0:
            return []
        self.stats["steps"] += 1
        lo, tok_lo = 0, []
        for i in range(n):
            tok_lo.append(lo)
            lo += int(sc.seq_ntok[i])
        dec = [i for i in range(n) if not sc.seq_prefill[i]]
        pre = [i for i in range(n) if sc.seq_prefill[i]]
        new_tokens = np.full(n, -1, np.int64)
        new_lps = np.zeros(n, np.float32)
        dev = self.device
        burst = None
        if dec:
            nd = len(dec)
            B = self._pad_batch(nd)
            st, graph, run = self._get_graph(B)
            di = np.asarray(dec)
            sids_d = sc.seq_ids[di]
            sps = [self.requests[int(sid)].params for sid in sids_d]
            k = 1
            if not pre and self.decode_burst > 1 and not any(p.stop_token_ids for p in sps):
                k = sc.reserve_burst(self.decode_burst)
            t_idx = np.asarray([tok_lo[i] for i in dec])
            hp, pad = st["host"], st["pad"]
            sig = (nd, sids_d.tobytes())
            fresh = st["sig"] != sig  # batch membership changed: rewrite the padding and the per-request constants
            dec_pos = sc.positions[t_idx]
            if self._mmreq:  # after its images a request's text positions are offset (all three RoPE axes are equal then)
                dec_pos = dec_pos + np.asarray([self._mmreq.get(int(sid), {}).get("delta", 0) for sid in sids_d])
            for name, arr in (("ids", sc.tokens[t_idx]), ("pos", dec_pos), ("slots", sc.slots[t_idx]),
                              ("bt", sc.block_tables[di]), ("lens", sc.seq_total[di])):
                hp[name][:nd] = arr
                if fresh:
                    hp[name][nd:] = pad[name]
            if fresh:
                for name, vals in (("temp", [p.temperature for p in sps]), ("topk", [p.top_k for p in sps]),
                                   ("topp", [p.top_p for p in sps]), ("flags", [int(p.ignore_eos) for p in sps]),
                                   ("limit", sc.step_limits(n)[di]), ("alive", 1)):
                    hp[name][:nd] = vals
                    hp[name][nd:] = pad[name]
                st["sig"] = sig
            st["dev_buf"].copy_(st["host_buf"], non_blocking=True)
            for _ in range(k):
                if graph is not None:
                    graph.replay()
                else:
                    run()
            st["out_host"].copy_(st["out_dev"], non_blocking=True)
            if self.record_routing:
                st["rt_host"].copy_(st["ring_rt"], non_blocking=True)
            t_wait = time.perf_counter()
            if dev.type == "cuda":
                torch.cuda.current_stream(dev).synchronize()
            if self.record_routing:
                # step s of the burst read the token at text position (position of the first step) + s; rows past a
                # sequence's end are cut off when the request finishes
                rt = st["rt_host"].numpy()
                for j, sid in enumerate(sids_d.tolist()):
                    self._routing_store(int(sid), int(sc.positions[t_idx[j]]), rt[:k, j])
            self.stats["decode_wait_s"] += time.perf_counter() - t_wait
            self.stats["decode_steps"] += k
            if k > 1:
                burst = (k, st["host_tok"][:k, :nd].copy(), st["host_lp"][:k, :nd].copy(), sps)
            else:
                new_tokens[di] = st["host_tok"][0, :nd]
                new_lps[di] = st["host_lp"][0, :nd]
            self.stats["decode_tokens"] += nd * k
        if burst is not None:
            outs = self._commit_burst(n, *burst)
            self.stats["step_s"] += time.perf_counter() - t_step
            return outs
        if pre:
            t_pre = time.perf_counter()
            logits = self._prefill_forward(pre, [tok_lo[i] for i in pre])
            # only chunks that complete their sequence sample a token
            sps = [self.requests[int(sc.seq_ids[i])].params for i in pre]
            temp = torch.tensor([p.temperature for p in sps], dtype=torch.float32, device=dev)
            topk = torch.tensor([p.top_k for p in sps], dtype=torch.int32, device=dev)
            topp = torch.tensor([p.top_p for p in sps], dtype=torch.float32, device=dev)
            tok, lp = ops.sample(logits, temperature=temp, top_k=topk, top_p=topp, seed=self.seed, step=self.step_counter)
            self.step_counter.add_(1)
            new_tokens[np.asarray(pre)] = tok.cpu().numpy()
            new_lps[np.asarray(pre)] = lp.cpu().numpy()
            self.stats["prefill_tokens"] += int(sum(sc.seq_ntok[i] for i in pre))
            self.stats["prefill_s"] += time.perf_counter() - t_pre
        # stop criteria
        finished = np.zeros(n, np.int32)
        reasons = {}
        sids = sc.seq_ids[:n].tolist()
        reqs = [self.requests[sid] for sid in sids]
        toks = new_tokens.tolist()
        eos = self.eos
        for i, (req, t) in enumerate(zip(reqs, toks)):
            prm = req.params
            if not prm.ignore_eos and (t == eos or (prm.stop_token_ids and t in prm.stop_token_ids)):
                finished[i] = 1
                reasons[sids[i]] = "completed"
        done = sc.commit(new_tokens, finished).tolist()
        partial = (sc.seq_prefill[:n] == 2).tolist()  # partial prefill chunk: its sampled token is discarded
        lps = new_lps.tolist()
        outs = []
        for i, req in enumerate(reqs):
            if toks[i] >= 0 and not partial[i]:
                req.logprobs.append(lps[i])
            if done[i]:
                outs.append(self._finish(sids[i], reasons.get(sids[i], "length")))
        self.stats["step_s"] += time.perf_counter() - t_step
        return outs

    def _commit_burst(self, n: int, k: int, toks: np.ndarray, lps: np.ndarray, sps: list) -> list[TokenOutput]:
        """Book-keeping of a burst of ``k`` decode steps over the ``n`` planned sequences (toks / lps are [k, n])."""
        sc = self.sched
        eos = self.eos
        finished_at = np.zeros(n, np.int32)
        if eos is not None:
            hit = toks == eos
            ign = np.asarray([p.ignore_eos for p in sps])
            hit[:, ign] = False
            any_hit = hit.any(0)
            finished_at[any_hit] = hit.argmax(0)[any_hit] + 1
        sids = sc.seq_ids[:n].tolist()
        accepted, done = sc.commit_burst(toks, finished_at)
        accepted, done = accepted.tolist(), done.tolist()
        outs = []
        for i, sid in enumerate(sids):
            req = self.requests[sid]
            a = accepted[i]
            if a:
                req.logprobs.extend(lps[:a, i].tolist())
            if done[i]:
                outs.append(self._finish(sid, "completed" if 0 < finished_at[i] <= a else "length"))
        return outs

    def _was_sampled(self, i: int) -> bool:
        """False for a partial prefill chunk: its sampled token is discarded by the scheduler."""
        return int(self.sched.seq_prefill[i]) != 2

    # ---------------------------------------------------------------- generate
    def generate(self, prompts: list[list[int]], sampling_params=None, request_ids: Optional[list[str]] = None,
                 multi_modal_inputs: Optional[list] = None):
        """Blocking batch generation. ``sampling_params``: one for all or a list; ``multi_modal_inputs``: per prompt a
        dict (``pixel_values`` / ``image_grid_thw``) or None. Returns TokenOutputs in order."""
        n = len(prompts)
        sps = sampling_params if isinstance(sampling_params, list) else [sampling_params] * n
        rids = request_ids or [f"gen-{self._next_sid + i}-{time.monotonic_ns()}" for i in range(n)]
        mms = multi_modal_inputs if multi_modal_inputs is not None else [None] * n
        for rid, p, sp, mm in zip(rids, prompts, sps, mms):
            self.add_request(rid, p, sp, multi_modal_inputs=mm)
        results: dict[str, TokenOutput] = {}
        want = set(rids)
        idle = 0
        while want - results.keys():
            outs = self.step()
            if not outs and not self.requests:
                break
            idle = idle + 1 if not outs and self.sched.stats()["running"] == 0 else 0
            if idle > 1000:
                raise RuntimeError("rollout engine made no progress (KV cache too small for the waiting requests?)")
            for o in outs:
                results[o.request_id] = o
        return [results[r] for r in rids]


def _varlen_attention_kv(q, k, v, cu_q, cu_k, max_q, max_k):
    """Causal attention where each sequence's queries are the last ``len_q`` positions of its keys."""
    if q.is_cuda:
        from ..ops.attention import _native_fwd_ok, flash_fwd

        k, v = k.contiguous(), v.contiguous()
        if _native_fwd_ok(q, k, v):
            return flash_fwd(q, k, v, cu_q, max_q, True, q.shape[-1] ** -0.5, need_lse=False, cu_seqlens_k=cu_k)[0]
        from flash_attn import flash_attn_varlen_func  # library kernel (head dims other than 128)

        return flash_attn_varlen_func(q, k, v, cu_q, cu_k, max_q, max_k, causal=True)
    out = torch.empty_like(q)
    G = q.shape[1] // k.shape[1]
    for (qs, qe), (ks, ke) in zip(zip(cu_q[:-1].tolist(), cu_q[1:].tolist()), zip(cu_k[:-1].tolist(), cu_k[1:].tolist())):
        lq, lk = qe - qs, ke - ks
        qq = q[qs:qe].transpose(0, 1).float()
        kk = k[ks:ke].repeat_interleave(G, 1).transpose(0, 1).float()
        vv = v[ks:ke].repeat_interleave(G, 1).transpose(0, 1).float()
        s = qq @ kk.transpose(1, 2) * q.shape[-1] ** -0.5
        mask = torch.arange(lk)[None, :] <= (torch.arange(lq)[:, None] + (lk - lq))
        s = s.masked_fill(~mask, float("-inf"))
        out[qs:qe] = (torch.softmax(s, -1) @ vv).transpose(0, 1).to(q.dtype)
    return out
