"""The native training engine: packed-sequence transformer on hand-written kernels, ZeRO-3
sharding with per-layer gather / recompute / reduce-scatter, fused AdamW on fp32 master shards.

It fills the role of ``FSDPEngine`` / ``FSDPEngineWithLMHead`` / ``FSDPEngineWithValueHead``
(verl/workers/engine/fsdp/transformer_impl.py:77-1057) and of the FSDP parts of
``ActorRolloutRefWorker._build_model_optimizer`` (verl/workers/fsdp_workers.py:275-611).

Differences by design:
  * inputs are always packed (remove-padding) and only the positions that predict response tokens go
    through the lm_head, which is fused with log-softmax / entropy (no logits tensor);
  * mixed precision = bf16 working weights + fp32 master / moments / gradient shards;
    weight-gradient GEMMs accumulate in fp32 directly into the gradient shard on one GPU;
  * activation checkpointing and parameter gathering are the same mechanism (``unit_call``).
"""

from __future__ import annotations

import json
import os
from contextlib import contextmanager
from pathlib import Path
from typing import Callable, Optional

import torch
import torch.distributed as dist

from ... import ops
from ...models import CausalLM, ModelConfig, PackedBatch
from ...models.hf_io import native_to_hf_items
from ...parallel.zero import ZeroShardedParams, unit_call
from .base import BaseEngine, EngineRegistry

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "float16": torch.float16, "fp16": torch.float16}


def _cfg(obj, key, default=None):
    if obj is None:
        return default
    if isinstance(obj, dict):
        v = obj.get(key, default)
    else:
        v = getattr(obj, key, default)
    return default if v is None else v


class _SumOverGroup(torch.autograd.Function):
    """Sum of per-rank partial results whose non-zero rows are disjoint. Every rank goes on to compute the same
    loss from the sum, so the backward is the identity on this rank's rows: no communication."""

    @staticmethod
    def forward(ctx, x, group):
        import torch.distributed as dist

        y = x.clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, grad):
        return grad, None


class NativeEngine(BaseEngine):
    def __init__(self, model_config: ModelConfig, engine_config=None, optimizer_config=None, *, value_head: bool = False,
                 device: Optional[str] = None, trainable: bool = True, group=None, seed: int = 0,
                 state_dict: Optional[dict] = None, comm=None, gradient_checkpointing: bool = True,
                 tiled_mlp_shards: int = 0, lora: Optional[dict] = None, frozen_prefixes: tuple = ()):
        self.model_config = model_config
        # parameters whose name starts with one of these stay as loaded (``("visual.",)``: a frozen vision tower)
        self.frozen_prefixes = tuple(frozen_prefixes or ())
        self._frozen: list = []
        self.tiled_mlp_shards = int(tiled_mlp_shards)
        # LoRA (``{"rank", "alpha", "target_modules", "exclude_modules"}``): the base weights are frozen and keep no
        # optimizer state; the adapters are replicated fp32 tensors trained by their own AdamW
        self.lora = dict(lora) if lora and int(lora.get("rank", 0) or 0) > 0 else None
        self._lora_params: list = []
        self._lora_opt = None
        self._keep_cap: Optional[int] = None  # set to 0 after an out-of-memory error with kept activations
        self.engine_config = engine_config
        self.optimizer_config = optimizer_config
        self.value_head = value_head
        if device is None:
            device = f"cuda:{torch.cuda.current_device()}" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        self.trainable = trainable and not _cfg(engine_config, "forward_only", False)
        self.group = group
        self.seed = seed
        self._init_state = state_dict
        self.comm = comm
        self.gradient_checkpointing = gradient_checkpointing
        self.work_dtype = _DTYPES[_cfg(engine_config, "dtype", "bfloat16")] if self.device.type == "cuda" else torch.float32
        self.step_count = 0
        self.lr_step = 0
        # gradient-norm clip of the role that owns this engine (``actor.grad_clip`` / ``critic.grad_clip`` of the
        # reference's FSDP workers) when it is to replace ``optim.clip_grad``
        self.clip_grad_override: Optional[float] = None
        if _cfg(engine_config, "full_determinism", False):
            from .utils import enable_full_determinism

            enable_full_determinism(int(seed))
        self.model: Optional[CausalLM] = None
        self.zero: Optional[ZeroShardedParams] = None
        self._offloaded = False

    # ------------------------------------------------------------------- build
    def initialize(self):
        cfg = self.model_config
        self._setup_pipeline()
        self._setup_tensor_parallel()
        if self.tp_size > 1 or self.pp_size > 1:
            self._build_parallel_model()
        else:
            self.model = CausalLM(cfg, dtype=self.work_dtype, device=self.device, value_head=self.value_head)
            self.model.init_weights(self.seed)
            if self._init_state is not None:
                missing, unexpected = self.model.load_state_dict(
                    {k: v.to(self.work_dtype) for k, v in self._init_state.items()}, strict=False)
        self._init_state = None
        if self.tiled_mlp_shards > 1:
            from ...models.tiled_mlp import apply_tiled_mlp

            apply_tiled_mlp(self.model, self.tiled_mlp_shards)
        if self.lora is not None and self.trainable:
            from ...models.lora import apply_lora, lora_named_parameters

            if self.device.type == "cuda":
                assert int(self.lora["rank"]) % 8 == 0, "lora_rank must be a multiple of 8 (GEMM row alignment)"
            for p in self.model.parameters():
                p.requires_grad_(False)
            apply_lora(self.model, int(self.lora["rank"]), float(self.lora.get("alpha", 16) or 16),
                       self.lora.get("target_modules", "all-linear"), self.lora.get("exclude_modules"), seed=self.seed)
            self._lora_params = [p for _, p in lora_named_parameters(self.model)]
        m = self.model
        first, last = self.pp_rank == 0, self.pp_rank == self.pp_size - 1
        tied = last and m.lm_head is None and not m.value_head
        units = []
        # a vision tower lives (and is gathered) with the embedding: its outputs replace placeholder-token embeddings
        vis = [("visual." + n, p) for n, p in m.visual.named_parameters()] if getattr(m, "visual", None) is not None else []
        if tied:
            units.append(("", [("embed_tokens.weight", m.embed_tokens.weight), ("norm.weight", m.norm.weight)] + vis))
        elif first:
            units.append(("", [("embed_tokens.weight", m.embed_tokens.weight)] + vis))
        # expert parallelism: the stacked expert matrices form units of their own that are never gathered (rank r's
        # shard IS experts [r E / W, (r + 1) E / W)); they go to the end of the list so that the layer units stay
        # neighbours for the gather prefetch
        ep = int(_cfg(self.engine_config, "expert_model_parallel_size", 1) or 1)
        self.ep_size = ep if (cfg.is_moe and ep > 1) else 1
        expert_units = []
        for i, layer in enumerate(m.layers):
            name = f"layers.{i + m.layer_offset}"
            if self.ep_size > 1:
                skip = {id(layer.mlp.gate_up_proj), id(layer.mlp.down_proj)}
                units.append((name, [(n, p) for n, p in layer.named_parameters() if id(p) not in skip]))
                expert_units.append((name, [("mlp.gate_up_proj", layer.mlp.gate_up_proj)], {"local": True}))
                expert_units.append((name, [("mlp.down_proj", layer.mlp.down_proj)], {"local": True}))
            else:
                units.append((name, layer))
        if last and not tied:
            head = [("norm.weight", m.norm.weight)]
            if m.value_head:
                head.append(("score.weight", m.score.weight))
            else:
                head.append(("lm_head.weight", m.lm_head.weight))
            units.append(("", head))
        n_plain = len(units)
        units += expert_units
        self._setup_hybrid_sharding()
        self.zero = ZeroShardedParams(units, group=self.shard_group, work_dtype=self.work_dtype, device=self.device,
                                      trainable=self.trainable and not self._lora_params, comm=self.comm)
        if self.ep_size > 1:
            if self.tp_size > 1 or self.lora is not None:
                raise ValueError("expert_model_parallel_size > 1 cannot be combined with tensor parallelism (which already "
                                 "splits the experts over its group) or LoRA")
            if self.zero.world > 1 and self.ep_size != self.zero.world:
                raise ValueError(f"expert_model_parallel_size {self.ep_size} must equal the size of the sharding group "
                                 f"({self.zero.world}): every rank of the group owns E / {self.zero.world} experts")
            if self.zero.world > 1:
                for layer in m.layers:
                    layer.mlp.ep_group = self.shard_group
        self.zero.frozen_grad = bool(self._lora_params)
        if self.frozen_prefixes and self.trainable and not self._lora_params:
            self._freeze(self.frozen_prefixes)
        self._setup_sequence_parallel()
        self._setup_context_parallel()
        n0 = 1 if (first or tied) else 0
        self._embed_unit = self.zero.units[0] if (first or tied) else None
        self._layer_units = self.zero.units[n0 : n0 + len(m.layers)]
        self._head_unit = (self.zero.units[0] if tied else self.zero.units[n_plain - 1]) if last else None
        if self.device.type == "cuda":
            torch.cuda.empty_cache()
        if self._lora_params:
            oc = self.optimizer_config
            self._lora_opt = torch.optim.AdamW(self._lora_params, lr=float(_cfg(oc, "lr", 1e-6)),
                                               betas=tuple(_cfg(oc, "betas", (0.9, 0.999))), eps=float(_cfg(oc, "eps", 1e-8)),
                                               weight_decay=float(_cfg(oc, "weight_decay", 0.01)))
        if self.trainable:
            dev = self.device
            self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
            self._scale = torch.ones(1, dtype=torch.float32, device=dev)
            self._skip = torch.zeros(1, dtype=torch.int32, device=dev)
            self._norm = torch.zeros(1, dtype=torch.float32, device=dev)
        return self

    @property
    def world(self) -> int:
        """Ranks of the engine's group (data parallel x sequence parallel); under hybrid sharding this is larger than
        ``zero.world``, the number of ranks over which the parameters are sharded."""
        return self.dp_world

    def _block_groups(self, k: int, strided: bool):
        """This rank's group among the groups of ``k`` ranks inside its block of ranks (the engine's group, or this
        pipeline stage's part of it): consecutive ranks ``[g k, (g + 1) k)``, or (``strided``) the ranks with the same
        index inside those. Process-group creation is collective over the whole job, so the groups of EVERY pipeline
        stage's block are created here, in the same order on every rank."""
        import torch.distributed as dist

        if self.pp_size > 1:
            full = dist.get_process_group_ranks(self.full_group)
            S = len(full) // self.pp_size
            blocks = [full[st * S : (st + 1) * S] for st in range(self.pp_size)]
        else:
            blocks = [dist.get_process_group_ranks(self.group)]
        me = dist.get_rank()
        mine = None
        for block in blocks:
            W = len(block)
            lists = ([[block[g * k + i] for g in range(W // k)] for i in range(k)] if strided
                     else [[block[g * k + i] for i in range(k)] for g in range(W // k)])
            for members in lists:
                grp = dist.new_group(members)
                if me in members:
                    mine = grp
        return mine

    def _setup_tensor_parallel(self):
        """``tensor_model_parallel_size`` > 1 (the Megatron-style training layout, verl/workers/config/engine.py
        McoreEngineConfig): ``tp`` consecutive ranks hold column / row slices of every block, 1 / tp of the experts and of
        an untied lm_head's vocabulary rows; activations between blocks are replicated over the group. Parameters,
        gradients and optimizer state of a slice are ZeRO-sharded over the ranks with the same slice."""
        import torch.distributed as dist

        self.tp_size, self.tp_rank, self.tp_group = 1, 0, None
        tp = int(_cfg(self.engine_config, "tensor_model_parallel_size", 1) or 1)
        W = dist.get_world_size(self.group) if self.group is not None else 1
        if tp <= 1:
            return
        if W % tp != 0:
            raise ValueError(f"tensor_model_parallel_size {tp} does not divide the {W} ranks of the engine's group")
        cfg = self.model_config
        if cfg.num_key_value_heads % tp != 0:
            raise ValueError(f"training with tensor_model_parallel_size {tp} needs it to divide the {cfg.num_key_value_heads} "
                             "KV heads (replicated KV heads would need their gradients summed between the replicas)")
        if int(_cfg(self.engine_config, "ulysses_sequence_parallel_size", 1) or 1) > 1:
            raise ValueError("tensor_model_parallel_size > 1 and ulysses_sequence_parallel_size > 1 cannot be combined")
        if self.lora is not None:
            raise ValueError("LoRA adapters are not sliced: use tensor_model_parallel_size = 1 with model.lora_rank > 0")
        r = dist.get_rank(self.group)
        self.tp_group = self._block_groups(tp, strided=False)
        self._tp_dp_group = self._block_groups(tp, strided=True)
        self.tp_size, self.tp_rank = tp, r % tp

    def _setup_pipeline(self):
        """``pipeline_model_parallel_size`` > 1: the engine's group is cut into ``pp`` consecutive blocks of ranks, block
        ``s`` holds stage ``s`` (a contiguous run of decoder layers; embedding on the first, final norm and head on the
        last stage). Everything else (tensor parallelism, sharding, data parallelism) is set up inside a stage's block;
        rank ``i`` of a block exchanges the residual stream with rank ``i`` of the neighbouring blocks."""
        import torch.distributed as dist

        self.full_group = self.group
        self.full_world = dist.get_world_size(self.group) if self.group is not None else 1
        self.full_rank = dist.get_rank(self.group) if self.group is not None else 0
        self.pp_size, self.pp_rank, self.pp_group = 1, 0, None
        pp = int(_cfg(self.engine_config, "pipeline_model_parallel_size", 1) or 1)
        if pp <= 1:
            return
        W, r = self.full_world, self.full_rank
        cfg = self.model_config
        if W % pp != 0:
            raise ValueError(f"pipeline_model_parallel_size {pp} does not divide the {W} ranks of the engine's group")
        if pp > cfg.num_hidden_layers:
            raise ValueError(f"pipeline_model_parallel_size {pp} exceeds the {cfg.num_hidden_layers} decoder layers")
        if cfg.tie_word_embeddings and not self.value_head:
            raise ValueError("tied input / output embeddings cannot be split over pipeline stages")
        if self.lora is not None or int(_cfg(self.engine_config, "ulysses_sequence_parallel_size", 1) or 1) > 1:
            raise ValueError("pipeline_model_parallel_size > 1 cannot be combined with LoRA or Ulysses")
        S = W // pp
        ranks_of = dist.get_process_group_ranks(self.group)
        stage_group = None
        for st in range(pp):  # collective: every rank creates every group
            grp = dist.new_group(ranks_of[st * S : (st + 1) * S])
            if r // S == st:
                stage_group = grp
        for i in range(S):
            grp = dist.new_group([ranks_of[st * S + i] for st in range(pp)])
            if r % S == i:
                self.pp_group = grp
        self.pp_size, self.pp_rank = pp, r // S
        self.pp_prev = ranks_of[r - S] if self.pp_rank > 0 else None           # global ranks of the neighbours
        self.pp_next = ranks_of[r + S] if self.pp_rank < pp - 1 else None
        self.pp_last = ranks_of[(pp - 1) * S + r % S]
        self.pp_stage_ranks = [ranks_of[st * S + r % S] for st in range(pp)]
        self.group = stage_group  # may hold this rank alone

    def _build_parallel_model(self):
        """This rank's part of the model: the whole model is initialised (or given), cut to the stage's layers and
        sliced for the tensor-parallel rank."""
        from ...parallel.pipeline import stage_layers
        from ...parallel.reshard import shard_state_dict, tp_model_config

        cfg, tp, r = self.model_config, self.tp_size, self.tp_rank
        state = self._init_state
        if state is None:
            full = CausalLM(cfg, dtype=self.work_dtype, device=self.device, value_head=self.value_head).init_weights(self.seed)
            state = dict(full.state_dict())
            del full
        lo, hi = stage_layers(cfg.num_hidden_layers, self.pp_size, self.pp_rank)
        first, last = self.pp_rank == 0, self.pp_rank == self.pp_size - 1
        if self.pp_size > 1:  # keep this stage's tensors; layers are renumbered from 0 inside the stage's module
            kept = {}
            for k, v in state.items():
                if k.startswith("layers."):
                    i = int(k.split(".")[1])
                    if lo <= i < hi:
                        kept[f"layers.{i - lo}." + k.split(".", 2)[2]] = v
                elif k.startswith("embed_tokens."):
                    if first:
                        kept[k] = v
                elif last:
                    kept[k] = v
            state = kept
        vp = last and (not self.value_head) and (not cfg.tie_word_embeddings) and tp > 1 and cfg.vocab_size % tp == 0
        self._vocab_parallel_head = vp
        tcfg = tp_model_config(cfg, r, tp)
        if vp:
            tcfg.extra["lm_head_rows"] = cfg.vocab_size // tp
        self.model = CausalLM(tcfg, dtype=self.work_dtype, device=self.device, value_head=self.value_head,
                              layer_range=(lo, hi), has_embed=first or (last and cfg.tie_word_embeddings and not self.value_head),
                              has_head=last)
        sl = shard_state_dict(cfg, {k: v.to(self.work_dtype) for k, v in state.items()}, r, tp, vocab_parallel_head=vp)
        self.model.load_state_dict(sl, strict=False)
        if tp > 1:
            for layer in self.model.layers:
                layer.self_attn.tp_group = self.tp_group
                layer.mlp.tp_group = self.tp_group
        if vp:
            self.model.tp_group = self.tp_group
            self.model.vocab_offset = r * (cfg.vocab_size // tp)

    def _setup_hybrid_sharding(self):
        """``fsdp_size`` < world (HSDP, verl/workers/fsdp_workers.py:98-108 ``create_device_mesh``): parameters,
        gradients and optimizer state are sharded over ``fsdp_size`` consecutive ranks and replicated across the
        ``world / fsdp_size`` groups; the replicas' gradient shards are summed before the optimizer step."""
        import torch.distributed as dist

        self.dp_world = dist.get_world_size(self.group) if self.group is not None else 1
        self.dp_rank_all = dist.get_rank(self.group) if self.group is not None else 0
        self.shard_group, self.replica_group, self.hsdp = self.group, None, False
        fs = int(_cfg(self.engine_config, "fsdp_size", -1) or -1)
        W = self.dp_world
        if self.tp_size > 1:
            # the slices are sharded over the ranks that hold the same slice
            if 0 < fs < W // self.tp_size:
                raise ValueError("fsdp_size (hybrid sharding) cannot be combined with tensor_model_parallel_size > 1")
            self.shard_group = self._tp_dp_group  # may hold this rank alone
            if self.comm is not None and self.device.type == "cuda":
                from ...parallel.peer_comm import PeerComm

                self.comm = PeerComm(self.shard_group) if W // self.tp_size > 1 else None
            return
        if fs <= 0 or fs >= W:
            return
        if W % fs != 0:
            raise ValueError(f"fsdp_size {fs} does not divide the {W} ranks of the engine's group")
        r = self.dp_rank_all
        self.shard_group = self._block_groups(fs, strided=False)
        self.replica_group = self._block_groups(fs, strided=True)
        self.hsdp = True
        self.replica_index = r // fs
        if self.comm is not None and self.device.type == "cuda":
            from ...parallel.peer_comm import PeerComm

            self.comm = PeerComm(self.shard_group) if fs > 1 else None  # the sharder's collectives stay in the group
        if fs == 1:
            self.comm = None

    def _setup_sequence_parallel(self):
        """Ulysses: ``ulysses_sequence_parallel_size`` consecutive ranks form a group that works on the same
        micro-batch, each on a slice of the packed token stream (mesh (dp, sp) of verl/workers/fsdp_workers.py:146-273).
        Parameters stay sharded over all ranks; the gradient reduce-scatter over all ranks then sums the partial
        gradients of the slices as well as those of the data-parallel replicas."""
        import torch.distributed as dist

        sp = int(_cfg(self.engine_config, "ulysses_sequence_parallel_size", 1) or 1)
        self.sp_size, self.sp_group, self.sp_rank = 1, None, 0
        if sp <= 1 or self.dp_world <= 1:
            return
        W, r = self.dp_world, self.dp_rank_all
        assert W % sp == 0, f"world size {W} is not a multiple of ulysses_sequence_parallel_size {sp}"
        from ...utils.ulysses import validate_ulysses_config

        validate_ulysses_config(self.model_config.num_attention_heads, sp)
        self.sp_group = self._block_groups(sp, strided=False)
        self.sp_size, self.sp_rank = sp, r % sp
        if self.device.type == "cuda" and self.comm is not None:
            # the exchanges around attention run as peer-memory kernels of the sequence-parallel group
            from ...parallel.peer_comm import PeerComm
            from ...utils.ulysses import register_peer_comm

            register_peer_comm(self.sp_group, self.comm if sp == self.dp_world else PeerComm(self.sp_group))
        for layer in self.model.layers:
            layer.self_attn.sp_group = self.sp_group

    def _setup_context_parallel(self):
        """``context_parallel_size`` consecutive ranks share a micro-batch; each holds two zig-zag chunks of every
        sequence (``parallel/context_parallel.py``; the reference reaches this through Megatron's
        ``context_parallel_size``, verl/workers/config/engine.py + verl/models/mcore/util.py:25-116). Parameters stay
        sharded over all ranks, as under Ulysses."""
        cp = int(_cfg(self.engine_config, "context_parallel_size", 1) or 1)
        self.cp_size, self.cp_group, self.cp_rank = 1, None, 0
        if cp <= 1 or self.dp_world <= 1:
            return
        if self.sp_size > 1 or self.tp_size > 1 or self.pp_size > 1:
            raise ValueError("context_parallel_size > 1 cannot be combined with Ulysses, tensor or pipeline parallelism")
        if getattr(self.model_config, "is_vl", False):
            raise ValueError("context_parallel_size > 1 is not supported for vision-language models")
        W, r = self.dp_world, self.dp_rank_all
        assert W % cp == 0, f"world size {W} is not a multiple of context_parallel_size {cp}"
        self.cp_group = self._block_groups(cp, strided=False)
        self.cp_size, self.cp_rank = cp, r % cp
        for layer in self.model.layers:
            layer.self_attn.cp_group = self.cp_group

    @property
    def model_parallel(self) -> bool:
        """The model itself is split over ranks (tensor or pipeline parallelism), not only its storage."""
        return self.tp_size > 1 or self.pp_size > 1

    @property
    def mp_size(self) -> int:
        """Ranks that work on the same samples: a sequence-parallel or a tensor-parallel group."""
        return self._mp_inner * max(self.pp_size, 1)

    @property
    def _mp_inner(self) -> int:
        return max(self.sp_size, 1) * max(self.tp_size, 1) * max(getattr(self, "cp_size", 1), 1)

    @property
    def mp_group(self):
        """Group of the ranks that work on the same samples (created on first use: a collective)."""
        if self.pp_size <= 1:
            if getattr(self, "cp_size", 1) > 1:
                return self.cp_group
            return self.tp_group if self.tp_size > 1 else self.sp_group
        if getattr(self, "_pool_group", None) is None:
            import torch.distributed as dist

            ranks_of = dist.get_process_group_ranks(self.full_group)
            S, inner = self.full_world // self.pp_size, self._mp_inner
            for d in range(S // inner):
                members = [ranks_of[st * S + d * inner + i] for st in range(self.pp_size) for i in range(inner)]
                grp = dist.new_group(members)
                if (self.full_rank % S) // inner == d:
                    self._pool_group, self._pool_rank = grp, members.index(ranks_of[self.full_rank])
        return self._pool_group

    @property
    def mp_rank(self) -> int:
        if self.pp_size > 1:
            _ = self.mp_group
            return self._pool_rank
        return self.tp_rank if self.tp_size > 1 else self.sp_rank

    def get_data_parallel_size(self) -> int:
        return self.dp_world // self._mp_inner

    def get_data_parallel_rank(self) -> int:
        return self.dp_rank_all // self._mp_inner

    def get_data_parallel_group(self):
        return self.group

    # -------------------------------------------------------------- mode / offload
    @contextmanager
    def train_mode(self, **kwargs):
        self._enter_mode("train")
        try:
            yield self
        finally:
            self._exit_mode("train")

    @contextmanager
    def eval_mode(self, **kwargs):
        self._enter_mode("eval")
        try:
            yield self
        finally:
            self._exit_mode("eval")

    def _enter_mode(self, mode, **kwargs):
        if self._offloaded:
            self.to(str(self.device))

    def _exit_mode(self, mode):
        if _cfg(self.engine_config, "param_offload", False) or _cfg(self.engine_config, "optimizer_offload", False):
            self.to("cpu", model=_cfg(self.engine_config, "param_offload", False),
                    optimizer=_cfg(self.engine_config, "optimizer_offload", False))

    def to(self, device: str, model: bool = True, optimizer: bool = True, grad: bool = True):
        if torch.device(device).type == "cpu" and self.device.type == "cuda":
            self.zero.offload(params=model, optimizer=optimizer)
            self._offloaded = True
        else:
            self.zero.reload()
            self._offloaded = False

    # ------------------------------------------------------------------ forward
    def _forward_hidden_rows(self, batch: PackedBatch, rows: Optional[torch.Tensor]):
        """Final-norm input pieces (hidden, residual) restricted to ``rows`` of the packed stream."""
        m, z = self.model, self.zero
        rope = m.rope(self.device)
        sp_lo = 0
        if self.sp_size > 1:
            # this rank's slice of the packed stream; attention re-assembles the sequences per head group
            from ...utils.ulysses import ulysses_pad_and_slice_inputs

            T = batch.input_ids.shape[0]
            ids_l, pos_l, _ = ulysses_pad_and_slice_inputs(batch.input_ids, batch.position_ids, self.sp_size, self.sp_group)
            sp_lo = self.sp_rank * ids_l.shape[0]
            batch = PackedBatch(ids_l, pos_l, batch.cu_seqlens, batch.max_seqlen, total_tokens=T)
        cp_inv = None
        if self.cp_size > 1:
            # this rank's two zig-zag chunks of every sequence, chunk-major; padding rows (index -1) sit past the end
            # of their sequence, so no real query ever attends to them
            from ...parallel.context_parallel import cp_local_index

            T = batch.input_ids.shape[0]
            idx, cu_chunk, offs = cp_local_index(batch.cu_seqlens, self.cp_rank, self.cp_size)
            held = idx >= 0
            safe = idx.clamp(min=0)
            ids_l = torch.where(held, batch.input_ids[safe], torch.zeros_like(safe))
            pos_l = torch.where(held, batch.position_ids[safe], offs)
            cp_inv = torch.full((T,), -1, dtype=torch.long, device=idx.device)
            cp_inv[idx[held]] = torch.nonzero(held, as_tuple=True)[0]
            batch = PackedBatch(ids_l, pos_l, cu_chunk, int((cu_chunk[1:] - cu_chunk[:-1]).max()), total_tokens=T)
        taps = ()
        if self.pp_rank > 0:
            from ...parallel.pipeline import pipe_recv

            hidden = pipe_recv(self.pp_prev, (batch.input_ids.shape[0], self.model_config.hidden_size), self.work_dtype,
                               self.device, need_grad=self.trainable)
        elif m.num_deepstack:
            # Qwen3-VL: the vision tower's deepstack features come out of the embedding unit with the embeddings and are
            # added to the image tokens' hidden states after the first layers
            if self.sp_size > 1 or self.cp_size > 1 or self.pp_size > 1:
                raise NotImplementedError("deepstack vision features (Qwen3-VL) with sequence, context or pipeline parallelism")
            hidden, *taps = unit_call(z, self._embed_unit, lambda: m.embed(batch, with_deepstack=True))
        else:
            hidden = unit_call(z, self._embed_unit, lambda: m.embed(batch))
        residual = None
        n_layers = len(m.layers)
        n_keep = self._layers_to_keep(hidden.shape[0]) if (torch.is_grad_enabled() and self.trainable) else 0
        for i, (layer, unit) in enumerate(zip(m.layers, self._layer_units)):
            # the LAST n_keep layers keep their activations: their memory is the first to be freed in the backward
            hidden, residual = unit_call(z, unit, lambda h, r, layer=layer: layer(h, r, batch, rope), hidden, residual,
                                         keep_activations=i >= n_layers - n_keep)
            if i < len(taps):
                hidden = m.add_deepstack(hidden, batch, taps[i])
        if cp_inv is not None:
            all_rows = rows if rows is not None else torch.arange(batch.total_tokens, device=hidden.device)
            loc = cp_inv[all_rows]
            mine = loc >= 0
            self._sp_sel = (mine, all_rows.numel())
            return hidden[loc[mine]], residual[loc[mine]]
        if self.sp_size > 1:
            # keep the rows that live in this rank's slice; _sp_merge puts the per-row results back together
            n_l = hidden.shape[0]
            all_rows = rows if rows is not None else torch.arange(batch.total_tokens, device=hidden.device)
            mine = (all_rows >= sp_lo) & (all_rows < sp_lo + n_l)
            self._sp_sel = (mine, all_rows.numel())
            local = all_rows[mine] - sp_lo
            return hidden[local], residual[local]
        if self.pp_rank < self.pp_size - 1:
            from ...parallel.pipeline import pipe_send

            # one tensor travels: the next stage's first RMSNorm re-creates (normed, residual) from hidden + residual
            return "sent", pipe_send(hidden if residual is None else hidden + residual, self.pp_next)
        if rows is not None:
            hidden, residual = hidden[rows], (residual[rows] if residual is not None else None)
        return hidden, residual

    def _pp_share(self, outs: tuple, token, n: int):
        """Pipeline stages other than the last one return placeholders that carry the last stage's VALUES (broadcast
        over the stages) and, through ``token``, this stage's part of the graph: calling backward on a loss built from
        them runs the stage's backward (receive the gradient from the next stage, back-propagate, send it on)."""
        import torch.distributed as dist

        last = self.pp_rank == self.pp_size - 1
        shared = []
        for t in outs:
            vals = t.detach().float().clone() if last else torch.zeros(n, dtype=torch.float32, device=self.device)
            dist.broadcast(vals, src=self.pp_last, group=self.pp_group)
            shared.append(t if last else vals + 0.0 * token)
        return tuple(shared)

    def _layers_to_keep(self, tokens: int) -> int:
        """How many decoder layers keep their activations for the backward instead of recomputing them.

        ``gradient_checkpointing=False`` keeps all of them. Otherwise ``keep_activation_layers`` of the engine config
        decides: an integer, or ``auto`` (default on CUDA): as many layers as fit in the memory that is free right
        now, after a reserve for the backward's own temporaries. The answer may differ between ranks and between
        micro-batches; the sequence of collectives does not depend on it."""
        n_layers = len(self.model.layers)
        if self._keep_cap is not None:
            return min(n_layers, self._keep_cap)
        if not self.gradient_checkpointing:
            return n_layers
        policy = os.environ.get("VERL_B200_KEEP_ACTIVATION_LAYERS") or _cfg(self.engine_config, "keep_activation_layers", "auto")
        if str(policy) != "auto":
            return max(0, min(n_layers, int(policy)))
        if self.device.type != "cuda":
            return 0
        c = self.model_config
        if c.num_experts:  # routed activations depend on the routing: recompute
            return 0
        qkv = (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim
        per_token = 2 * (5 * c.hidden_size + qkv + c.num_attention_heads * c.head_dim + 3 * c.intermediate_size) + 64
        per_layer = int(tokens * per_token * 1.1)
        free, total = torch.cuda.mem_get_info(self.device)
        free += torch.cuda.memory_reserved(self.device) - torch.cuda.memory_allocated(self.device)
        reserve = max(12 << 30, total // 12) + 2 * per_layer
        n = int(max(0, free - reserve) // max(per_layer, 1))
        self.last_kept_layers = min(n_layers, n)
        self.last_keep_info = {"free_gb": round(free / 2**30, 1), "per_layer_gb": round(per_layer / 2**30, 2),
                               "reserve_gb": round(reserve / 2**30, 1), "tokens": int(tokens)}
        return self.last_kept_layers

    def _sp_merge(self, out):
        """Scatter this rank's per-row results into the full row order and sum over the sequence-parallel group
        (every row is owned by exactly one rank). The backward keeps the gradient of the rows this rank owns."""
        if self.sp_size <= 1 and self.cp_size <= 1:
            return out
        mine, n = self._sp_sel
        group = self.cp_group if self.cp_size > 1 else self.sp_group

        def one(t):
            full = torch.zeros((n,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
            full = full.index_put((torch.nonzero(mine, as_tuple=True)[0],), t)
            return _SumOverGroup.apply(full, group)

        return tuple(one(t) if isinstance(t, torch.Tensor) else t for t in out) if isinstance(out, tuple) else one(out)

    def _forward_hidden_rows_safe(self, batch: PackedBatch, rows: Optional[torch.Tensor]):
        """:meth:`_forward_hidden_rows`; on a single GPU an out-of-memory error in a training forward (nothing of this
        micro-batch has reached the gradient shard yet) switches the kept-activation policy off for the rest of the
        run and repeats the forward with every layer recomputed. With several ranks a one-sided repeat would
        desynchronise the collectives, so the error is raised."""
        try:
            return self._forward_hidden_rows(batch, rows)
        except torch.cuda.OutOfMemoryError:
            if not (torch.is_grad_enabled() and self.trainable and self.zero.world == 1 and self._keep_cap != 0):
                raise
            self._keep_cap = 0
            print("[verl_b200] out of memory with kept activations: recomputing all layers from now on", flush=True)
            torch.cuda.empty_cache()
            return self._forward_hidden_rows(batch, rows)

    def forward_logprob(self, batch: PackedBatch, rows: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0,
                        sum_pi_squared: bool = False):
        """Log-prob of ``labels[i]`` predicted at packed position ``rows[i]`` (+ entropy), both fp32.
        ``sum_pi_squared`` (forward-only passes of the optimal-token-baseline estimators): a third output, the sum over
        the vocabulary of the squared token probabilities at every row, from logits materialised 1024 rows at a time."""
        m, z = self.model, self.zero
        hidden, residual = self._forward_hidden_rows_safe(batch, rows)
        if isinstance(hidden, str):  # an earlier pipeline stage: the residual stream went to the next stage
            return self._pp_share((0, 0, 0) if sum_pi_squared else (0, 0), residual, rows.numel())

        if self.sp_size > 1 or self.cp_size > 1:
            labels = labels[self._sp_sel[0]]

        def head(h, r):
            x = m.final_norm(h, r)
            out = m.logprob_entropy(x, labels, temperature)
            if not sum_pi_squared:
                return out
            assert m.tp_group is None or m.lm_head is None or m.lm_head.weight.shape[0] == m.cfg.vocab_size, \
                "sum_pi_squared with a vocabulary-parallel lm_head is not supported"
            spp = []
            with torch.no_grad():
                for lo in range(0, x.shape[0], 1024):
                    p = torch.softmax(m.logits(x[lo : lo + 1024]).float() / temperature, dim=-1)
                    spp.append((p * p).sum(-1))
            return (*out, torch.cat(spp) if spp else x.new_zeros(0, dtype=torch.float32))

        out = self._sp_merge(unit_call(z, self._head_unit, head, hidden, residual))
        return self._pp_share(out, None, rows.numel()) if self.pp_size > 1 else out

    def forward_values(self, batch: PackedBatch, rows: torch.Tensor):
        m, z = self.model, self.zero
        hidden, residual = self._forward_hidden_rows_safe(batch, rows)
        if isinstance(hidden, str):
            return self._pp_share((0,), residual, rows.numel())[0]
        out = self._sp_merge(unit_call(z, self._head_unit, lambda h, r: m.values(m.final_norm(h, r)), hidden, residual))
        return self._pp_share((out,), None, rows.numel())[0] if self.pp_size > 1 else out

    def forward_logits(self, batch: PackedBatch, rows: Optional[torch.Tensor] = None):
        m, z = self.model, self.zero
        hidden, residual = self._forward_hidden_rows(batch, rows)
        return self._sp_merge(unit_call(z, self._head_unit, lambda h, r: m.logits(m.final_norm(h, r)), hidden, residual))

    # --------------------------------------------------------- response bookkeeping
    # ----------------------------------------------------------- TensorDict batch interface
    def forward_backward_batch(self, data, loss_function=None, forward_only: bool = False) -> dict:
        """One pass over a batch in the no-padding layout (verl/workers/engine/fsdp/transformer_impl.py:
        forward_backward_batch + prepare_model_inputs / prepare_model_outputs).

        ``data``: TensorDict with ``input_ids`` as a jagged nested tensor ``[bsz, j]`` (optionally ``position_ids``),
        the loss inputs (``loss_mask`` nested for SFT; ``prompts / responses / response_mask / attention_mask / ...``
        for RL losses), and the non-tensor knobs ``use_dynamic_bsz``, ``max_token_len_per_gpu``,
        ``micro_batch_size_per_gpu``, ``temperature``, ``calculate_entropy``.

        The model outputs handed to ``loss_function(model_output=..., data=micro_batch, dp_group=...)`` are nested
        tensors aligned with ``input_ids``: ``log_probs[i][t]`` is the log-probability of token ``t + 1`` of sample
        ``i`` (``entropy`` likewise), ``values[i][t]`` for a value head. Returns ``{"loss": [per micro-batch],
        "model_output": {...concatenated nested tensors...}, "metrics": {name: [per micro-batch]}}``."""
        import torch.distributed as dist

        from ...utils import tensordict_utils as tu

        ids = data["input_ids"]
        assert ids.is_nested, "the engine's batch interface takes input_ids as a jagged nested tensor (no padding)"
        temperature = float(tu.get(data, "temperature", 1.0) or 1.0)
        calc_ent = bool(tu.get(data, "calculate_entropy", False))
        lens = ids.offsets().diff()
        # global normalisers of the loss (sum over the data-parallel group): tokens that count, samples
        if "loss_mask" in data.keys():
            counted = float(data["loss_mask"].values().sum())
        elif "response_mask" in data.keys():
            counted = float(data["response_mask"].sum())
        else:
            counted = float(lens.sum())
        norm = torch.tensor([counted, float(len(lens))], dtype=torch.float64, device=self.device)
        dp_group = self.get_data_parallel_group()
        if self.dp_world > 1:
            dist.all_reduce(norm, group=self.group)
            norm = norm / self._mp_inner
        # micro-batches: fixed sample count, or packed up to a token budget
        n = len(lens)
        if tu.get(data, "use_dynamic_bsz", False):
            budget = int(tu.get(data, "max_token_len_per_gpu", 16384) or 16384)
            groups, cur, tok = [], [], 0
            for i, L in enumerate(lens.tolist()):
                if cur and tok + L > budget:
                    groups.append(cur)
                    cur, tok = [], 0
                cur.append(i)
                tok += L
            if cur:
                groups.append(cur)
        else:
            mb = int(tu.get(data, "micro_batch_size_per_gpu", None) or n)
            groups = [list(range(i, min(i + mb, n))) for i in range(0, n, mb)]
        out = {"loss": [], "metrics": {}, "model_output": {}}
        pieces: dict = {}
        pending: list = []
        for g in groups:
            micro = data[torch.tensor(g)]
            mids = micro["input_ids"]
            vals, offs = mids.values().to(self.device), mids.offsets().to(self.device)
            if "position_ids" in micro.keys() and micro["position_ids"].is_nested:
                pos = micro["position_ids"].values().to(self.device)
            else:
                mlens = offs.diff()
                pos = torch.arange(vals.numel(), device=self.device) - torch.repeat_interleave(offs[:-1], mlens)
            packed = PackedBatch(vals, pos, offs.int(), int(offs.diff().max().item()))
            rows = torch.arange(vals.numel(), device=self.device)

            def nest(t):
                return torch.nested.nested_tensor_from_jagged(t, offsets=offs)

            if self.model.value_head:
                model_output = {"values": nest(self.forward_values(packed, rows))}
            else:
                labels = torch.roll(vals, -1)
                lp, ent = self.forward_logprob(packed, rows, labels, temperature)
                model_output = {"log_probs": nest(lp)}
                if calc_ent and ent is not None:
                    model_output["entropy"] = nest(ent)
            for k, v in model_output.items():
                pieces.setdefault(k, []).append(v.detach())
            if loss_function is not None:
                # this engine SUMS the ranks' gradients (reduce-scatter without averaging), so the factor with which the
                # reference undoes its gradient averaging is 1: a rank's loss is its part of the global mean
                tu.assign_non_tensor(micro, dp_size=1, batch_num_tokens=float(norm[0]), global_batch_size=float(norm[1]))
                loss, metrics = loss_function(model_output=model_output, data=micro, dp_group=dp_group)
                if not forward_only:
                    if self.pp_size > 1:
                        pending.append(loss)  # pipelined: all forwards first, then the backwards in the same order
                    else:
                        loss.backward()
                out["loss"].append(float(loss.detach()))
                for k, v in (metrics or {}).items():
                    out["metrics"].setdefault(k, []).append(float(v) if not isinstance(v, (list, dict)) else v)
        for loss in pending:
            loss.backward()
        for k, v in pieces.items():
            out["model_output"][k] = tu.concat_nested_tensors(v) if len(v) > 1 else v[0]
        return out

    def train_batch(self, data, loss_function) -> dict:
        """zero-grad -> forward / backward over the micro-batches -> optimizer step (BaseEngine.train_batch of the
        reference); ``metrics["grad_norm"]`` is added."""
        self.optimizer_zero_grad()
        out = self.forward_backward_batch(data, loss_function, forward_only=False)
        out["metrics"]["grad_norm"] = float(self.optimizer_step())
        return out

    def infer_batch(self, data, loss_function=None) -> dict:
        with torch.no_grad():
            return self.forward_backward_batch(data, loss_function, forward_only=True)

    def is_mp_src_rank_with_outputs(self) -> bool:
        inner = self.tp_rank if self.tp_size > 1 else self.sp_rank
        return inner == 0 and self.pp_rank == self.pp_size - 1

    @staticmethod
    def response_rows(input_ids: torch.Tensor, attention_mask: torch.Tensor, response_length: int,
                      position_ids: Optional[torch.Tensor] = None):
        """Pack a left-padded-prompt / right-padded-response batch and locate, for every existing
        response token, the packed row that predicts it.

        Returns (packed batch, rows [N], labels [N], (b, j) coordinates of the N response tokens)."""
        B, S = input_ids.shape
        P = S - response_length
        packed, idx = PackedBatch.from_padded(input_ids, attention_mask, position_ids)
        inv = torch.full((B * S,), -1, dtype=torch.long, device=input_ids.device)
        inv[idx] = torch.arange(idx.numel(), device=input_ids.device)
        resp_exists = attention_mask[:, P:].bool()
        bj = torch.nonzero(resp_exists, as_tuple=False)
        src_flat = bj[:, 0] * S + (P - 1) + bj[:, 1]
        rows = inv[src_flat]
        labels = input_ids[:, P:][resp_exists]
        return packed, rows, labels, bj

    # ---------------------------------------------------------------- optimizer
    def optimizer_zero_grad(self):
        self.zero.zero_grad()
        for p in self._lora_params:
            p.grad = None

    def _lora_optimizer_step(self) -> torch.Tensor:
        """Sum the adapter gradients over the data-parallel group, clip by their global norm, AdamW. A non-finite
        norm skips the update."""
        oc = self.optimizer_config
        clip = float(_cfg(oc, "clip_grad", 1.0) if self.clip_grad_override is None else self.clip_grad_override)
        grads = [p.grad if p.grad is not None else torch.zeros_like(p) for p in self._lora_params]
        flat = torch.cat([g.reshape(-1) for g in grads])
        if self.dp_world > 1:
            dist.all_reduce(flat, group=self.group)
        norm = flat.double().norm().float()
        self.step_count += 1
        if bool(torch.isfinite(norm)):
            coef = min(1.0, clip / (float(norm) + 1e-6)) if clip > 0 else 1.0
            off = 0
            for p in self._lora_params:
                n = p.numel()
                p.grad = (flat[off:off + n] * coef).view_as(p)
                off += n
            for g in self._lora_opt.param_groups:
                g["lr"] = self._lr()
            self._lora_opt.step()
        else:
            self.step_count -= 1
        for p in self._lora_params:
            p.grad = None
        return norm.reshape(1)

    @contextmanager
    def disable_adapter(self):
        """Run the frozen base model (the reference policy under LoRA: verl's ``ref_in_actor``)."""
        mods = dict(self.model.named_modules())
        names = list(getattr(self.model, "lora_modules", []))
        for n in names:
            mods[n].__dict__["lora_off"] = True
        try:
            yield self
        finally:
            for n in names:
                mods[n].__dict__["lora_off"] = False

    def merge_lora_into(self, model) -> int:
        """Add the adapters' deltas to the weights of ``model`` (same module names, weights equal to the base)."""
        from ...models.lora import merge_lora_into

        return merge_lora_into(self.model, model) if self._lora_params else 0

    def _lr(self) -> float:
        oc = self.optimizer_config
        base = float(_cfg(oc, "lr", 1e-6))
        total = int(_cfg(oc, "total_training_steps", -1))
        warm = int(_cfg(oc, "lr_warmup_steps", -1))
        if warm < 0:
            warm = int(float(_cfg(oc, "lr_warmup_steps_ratio", 0.0)) * max(total, 0))
        step = self.lr_step
        kind = _cfg(oc, "lr_scheduler_type", "constant")
        if step < warm:
            return base * step / max(1, warm)
        if kind == "cosine" and total > 0:
            import math

            min_ratio = float(_cfg(oc, "min_lr_ratio", 0.0) or 0.0)
            prog = (step - warm) / max(1, total - warm)
            cyc = float(_cfg(oc, "num_cycles", 0.5))
            coef = (1 - min_ratio) * 0.5
            return base * max(min_ratio, math.cos(math.pi * cyc * 2.0 * prog) * coef + (1 + min_ratio) * 0.5)
        return base

    def lr_scheduler_step(self):
        self.lr_step += 1
        return self._lr()

    def _freeze(self, prefixes: tuple) -> None:
        """No gradient for the named parameters, and their slices of this rank's master / working shards are put back
        after every optimizer step (with zero gradients AdamW itself leaves them alone, the decoupled weight decay
        does not)."""
        z = self.zero
        for u in z.units:
            if u.local:
                continue
            lo, hi = z.rank * u.shard, (z.rank + 1) * u.shard
            for name, p, n, o in zip(u.names, u.params, u.numels, u.offsets):
                if not name.startswith(prefixes):
                    continue
                p.requires_grad_(False)
                s_, e_ = max(o, lo), min(o + n, hi)
                if s_ < e_:
                    a, b = u.offset + s_ - lo, u.offset + e_ - lo
                    self._frozen.append((a, b, z.master[a:b].clone()))
        if not any(not p.requires_grad for u in z.units for p in u.params):
            raise ValueError(f"no parameter name starts with {prefixes}")

    def optimizer_step(self) -> float:
        """Global grad-norm, clip, fused AdamW on the shards. Returns the (pre-clip) gradient norm; a
        non-finite norm skips the update (verl/workers/actor/dp_actor.py:391-415)."""
        if self._lora_params:
            return self._lora_optimizer_step()
        z, oc = self.zero, self.optimizer_config
        clip = float(_cfg(oc, "clip_grad", 1.0) if self.clip_grad_override is None else self.clip_grad_override)
        lr = self._lr()
        betas = tuple(_cfg(oc, "betas", (0.9, 0.999)))
        wd = float(_cfg(oc, "weight_decay", 0.01))
        eps = float(_cfg(oc, "eps", 1e-8))
        self.step_count += 1
        z.wait_comm()  # the last reduce-scatters run on the communication stream
        z.fold_local_units()
        if self.hsdp:  # hybrid sharding: add up the replicas' gradient shards (the loss is normalised globally)
            dist.all_reduce(z.grad, group=self.replica_group)
        if self.device.type == "cuda":
            self._sumsq.zero_()
            ops.sumsq_into(z.grad if self.tp_size == 1 else z.grad * self._tp_norm_weight(), self._sumsq)
            if z.world > 1:
                dist.all_reduce(self._sumsq, group=self.shard_group)
            if self.tp_size > 1:
                dist.all_reduce(self._sumsq, group=self.tp_group)
            if self.pp_size > 1:  # every stage holds its own layers: the norm is over all of them
                dist.all_reduce(self._sumsq, group=self.pp_group)
            ops.clip_coef(self._sumsq, clip, 1.0, self._scale, self._skip, self._norm)
            ops.adamw_step(z.master, z.grad, z.exp_avg, z.exp_avg_sq, z.shard16, lr=lr, betas=betas, eps=eps,
                           weight_decay=wd, step=self.step_count, scale=self._scale, skip=self._skip)
            norm = self._norm
            if int(self._skip.item()):  # a non-finite norm skipped the update: the step does not count
                self.step_count -= 1
        else:
            g_n = z.grad if self.tp_size == 1 else z.grad * self._tp_norm_weight()
            sq = g_n.double().pow(2).sum().reshape(1)
            if z.world > 1:
                dist.all_reduce(sq, group=self.shard_group)
            if self.tp_size > 1:
                dist.all_reduce(sq, group=self.tp_group)
            if self.pp_size > 1:
                dist.all_reduce(sq, group=self.pp_group)
            norm = sq.sqrt().float()
            if torch.isfinite(norm).all():
                coef = min(1.0, clip / (norm.item() + 1e-6)) if clip > 0 else 1.0
                g = z.grad * coef
                b1, b2 = betas
                z.exp_avg.mul_(b1).add_(g, alpha=1 - b1)
                z.exp_avg_sq.mul_(b2).addcmul_(g, g, value=1 - b2)
                bc1, bc2 = 1 - b1 ** self.step_count, 1 - b2 ** self.step_count
                z.master.mul_(1 - lr * wd)
                z.master.addcdiv_(z.exp_avg / bc1, (z.exp_avg_sq / bc2).sqrt() + eps, value=-lr)
                z.shard16.copy_(z.master.to(z.shard16.dtype))
            else:
                self.step_count -= 1
        for a, b, saved in self._frozen:
            z.master[a:b].copy_(saved)
            z.shard16[a:b].copy_(saved.to(z.shard16.dtype))
        z.zero_grad()
        return norm

    _TP_SLICED = ("qkv_proj.weight", "qkv_proj.bias", "gate_up_proj.weight", "o_proj.weight", "down_proj.weight",
                  "mlp.gate_up_proj", "mlp.down_proj")

    def _tp_is_sliced(self, name: str) -> bool:
        leaf = name.split(".")[-2] + "." + name.split(".")[-1] if "." in name else name
        return leaf in self._TP_SLICED or (getattr(self, "_vocab_parallel_head", False) and name.endswith("lm_head.weight"))

    def _tp_norm_weight(self) -> torch.Tensor:
        """Per-element factor of the gradient-norm sum over (shard group x tensor-parallel group): replicated
        parameters (norms, embeddings, routers) appear once per tensor-parallel rank, so their squares count 1 / tp."""
        w = getattr(self, "_tp_w", None)
        if w is None:
            z = self.zero
            w = torch.ones_like(z.grad)
            dup = (1.0 / self.tp_size) ** 0.5
            for u in z.units:
                lo, hi = z.rank * u.shard, (z.rank + 1) * u.shard
                for name, n, o in zip(u.names, u.numels, u.offsets):
                    if self._tp_is_sliced(name):
                        continue
                    s_, e_ = max(o, lo), min(o + n, hi)
                    if s_ < e_:
                        w[u.offset + s_ - lo : u.offset + e_ - lo] = dup
            self._tp_w = w
        return w

    # --------------------------------------------------------------- weights out
    def get_per_tensor_param(self, dtype: Optional[torch.dtype] = None):
        """Generator of (HF parameter name, full tensor): one unit is gathered at a time."""
        if self._offloaded:
            self.to(str(self.device))
        return native_to_hf_items(self.model_config, self._merged_named_tensors(dtype))

    def _merged_named_tensors(self, dtype=None):
        """(name, full tensor) of every parameter of the WHOLE model, in the same order on every rank: pipeline stages
        take turns broadcasting their tensors to the ranks at the same position of the other stages."""
        if self.pp_size <= 1:
            yield from self._stage_named_tensors(dtype)
            return
        import torch.distributed as dist

        for st in range(self.pp_size):
            src = self.pp_stage_ranks[st]
            mine = st == self.pp_rank
            it = self._stage_named_tensors(dtype) if mine else None
            while True:
                head = [None]
                if mine:
                    nxt = next(it, None)
                    head = [None if nxt is None else (nxt[0], tuple(nxt[1].shape), nxt[1].dtype)]
                dist.broadcast_object_list(head, src=src, group=self.pp_group)
                if head[0] is None:
                    break
                name, shape, dt = head[0]
                t = nxt[1].contiguous() if mine else torch.empty(shape, dtype=dt, device=self.device)
                dist.broadcast(t, src=src, group=self.pp_group)
                yield name, t

    def _stage_named_tensors(self, dtype=None):
        """(name, full tensor) of every parameter of this pipeline stage; adapted weights come out merged
        (W + (alpha / r) B A); tensor-parallel slices are gathered over the group and put back together."""
        if self.tp_size > 1:
            import torch.distributed as dist

            from ...parallel.reshard import unshard_state_dict

            for k, v in self.zero.named_full_tensors(dtype):
                if not self._tp_is_sliced(k):
                    yield k, v
                    continue
                parts = [torch.empty_like(v) for _ in range(self.tp_size)]
                dist.all_gather(parts, v.contiguous(), group=self.tp_group)
                yield k, unshard_state_dict(self.model_config, [{k: p} for p in parts],
                                            getattr(self, "_vocab_parallel_head", False))[k]
            return
        if not self._lora_params:
            yield from self.zero.named_full_tensors(dtype)
            return
        from ...models.lora import lora_delta

        mods = dict(self.model.named_modules())
        adapted = {n + ".weight": mods[n] for n in self.model.lora_modules}
        for k, v in self.zero.named_full_tensors(dtype):
            if k in adapted:
                v = (v.float() + lora_delta(adapted[k]).to(v.device)).to(v.dtype)
            yield k, v

    def native_named_tensors(self):
        return self._merged_named_tensors()

    def full_state_dict(self, dtype=torch.bfloat16, to_cpu: bool = True) -> dict:
        out = {}
        for k, v in self._merged_named_tensors():
            t = v.detach().to(dtype)
            out[k] = t.cpu() if to_cpu else t.clone()
        return out

    # ---------------------------------------------------------------- checkpoint
    def save_checkpoint(self, local_path: str, hdfs_path=None, global_step: int = 0, max_ckpt_to_keep=None,
                        save_contents=("model", "optimizer", "extra"), **kwargs):
        """verl FSDP layout: ``model_world_size_{W}_rank_{r}.pt``, ``optim_...``, ``extra_state_...``,
        ``fsdp_config.json``, ``huggingface/`` (verl/utils/checkpoint/fsdp_checkpoint_manager.py:56-362)."""
        from ...utils.checkpoint.checkpoint_manager import NativeCheckpointManager

        # the manager keeps the list of folders this engine has written: ``max_ckpt_to_keep`` removes the oldest before
        # a new save, ``hdfs_path`` receives a copy of the finished folder
        mgr = getattr(self, "_ckpt_manager", None)
        if mgr is None:
            mgr = self._ckpt_manager = NativeCheckpointManager(self)
        mgr.checkpoint_save_contents = list(save_contents)
        mgr.save_checkpoint(local_path, hdfs_path, global_step=global_step, max_ckpt_to_keep=max_ckpt_to_keep)

    def load_checkpoint(self, local_path: str, hdfs_path=None, del_local_after_load: bool = False,
                        load_contents=("model", "optimizer", "extra"), **kwargs):
        from ...utils.checkpoint.native_checkpoint import load_engine_checkpoint

        load_engine_checkpoint(self, local_path, load_contents=load_contents)


@EngineRegistry.register(model_type="language_model", backend=["fsdp", "fsdp2", "native", "megatron"], device=["cuda", "cpu"])
class NativeEngineWithLMHead(NativeEngine):
    pass


@EngineRegistry.register(model_type="value_model", backend=["fsdp", "fsdp2", "native", "megatron"], device=["cuda", "cpu"])
class NativeEngineWithValueHead(NativeEngine):
    def __init__(self, *args, **kwargs):
        kwargs["value_head"] = True
        super().__init__(*args, **kwargs)
