"""SPMD workers: the hybrid actor / rollout / reference worker, the critic worker and a
reward-model worker, all on the native engines.

RPC surface and semantics follow ``ActorRolloutRefWorker`` / ``CriticWorker`` / ``RewardModelWorker``
(verl/workers/fsdp_workers.py:140-1981, verl/workers/engine_workers.py:371-636): ``init_model,
generate_sequences, compute_log_prob, compute_ref_log_prob, update_actor, update_weights,
compute_values, update_critic, compute_rm_score, save_checkpoint, load_checkpoint``.

Hybrid engine on one box: the rollout engine runs on the same GPU as the trainer. With one rank it
reads the trainer's bf16 weights in place (weight sync is a no-op); with several ranks every rank
keeps a rollout copy that ``update_weights`` refreshes from the ZeRO shards over NVLink.
"""

from __future__ import annotations

import os
import time
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from ..models import CausalLM, ModelConfig, preset
from ..models.hf_io import load_hf_checkpoint
from ..protocol import DataProto
from ..single_controller.base import Dispatch, Worker, register
from ..single_controller.base.decorator import make_nd_compute_dataproto_dispatch_fn
from ..utils.config import omega_conf_to_dataclass
from ..utils.py_functional import append_to_dict
from .actor.dp_actor import DataParallelPPOActor
from .critic.dp_critic import DataParallelPPOCritic
from .engine.native import NativeEngine, _cfg

__all__ = ["ActorRolloutRefWorker", "AsyncActorRolloutRefWorker", "CriticWorker", "RewardModelWorker",
           "resolve_model_config"]


def resolve_model_config(model_cfg) -> tuple[ModelConfig, Optional[dict]]:
    """Model architecture (and weights, if the path holds any) from ``model.path``: an HF directory, a
    preset name (``preset:qwen2.5-7b``) for random-init runs, or ``override_config`` on top of either."""
    path = os.path.expanduser(str(_cfg(model_cfg, "path", "")))
    override = dict(_cfg(model_cfg, "override_config", {}) or {})
    override = dict(override.get("model_config", override))
    state = None
    if path.startswith("preset:"):
        cfg = preset(path[len("preset:"):], **override)
        return cfg, None
    if os.path.isdir(path):
        if any(f.endswith(".safetensors") for f in os.listdir(path)):
            cfg, state = load_hf_checkpoint(path)
        else:
            cfg = ModelConfig.from_pretrained(path)
        for k, v in override.items():
            setattr(cfg, k, v)
        return cfg, state
    raise FileNotFoundError(f"model path {path!r}: expected an HF directory or 'preset:<name>'")


def _role_clip(role_cfg):
    """``actor.grad_clip`` / ``critic.grad_clip`` (the knob of the reference's FSDP workers) replaces ``optim.clip_grad``
    (the knob of its engine workers) when only the former was changed from the common default of 1.0."""
    role, optim = _cfg(role_cfg, "grad_clip", None), _cfg(_cfg(role_cfg, "optim", None), "clip_grad", 1.0)
    if role is not None and float(role) != 1.0 and float(optim) == 1.0:
        return float(role)
    return None


def _init_dist(device_name: str, timeout_s: int = 600):
    if dist.is_initialized():
        return
    if int(os.environ.get("WORLD_SIZE", 1)) <= 1 and "MASTER_ADDR" not in os.environ:
        return
    from datetime import timedelta

    backend = "nccl" if device_name == "cuda" and torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group(backend=backend, timeout=timedelta(seconds=timeout_s))


class _WorkerBase(Worker):
    def __init__(self, config, device_name: Optional[str] = None):
        super().__init__()
        self.config = config
        self.device_name = device_name or ("cuda" if torch.cuda.is_available() else "cpu")
        _init_dist(self.device_name, int(_cfg(config, "nccl_timeout", 600)))
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.dp_rank = dist.get_rank() if dist.is_initialized() else 0
        if self.device_name == "cuda":
            self.device = torch.device("cuda", torch.cuda.current_device())
        else:
            self.device = torch.device("cpu")

    def _norm_batch(self, cfg, mini_key="ppo_mini_batch_size", micro_key="ppo_micro_batch_size", n: int = 1):
        """YAML batch sizes are global prompt counts; workers use per-rank sample counts. The ranks of a
        sequence-parallel group share their samples, so the divisor is the data-parallel size ``world // sp``
        (verl/workers/fsdp_workers.py:239-273)."""
        eng_cfg = _cfg(cfg, "fsdp_config", None) or _cfg(_cfg(cfg, "model", None), "fsdp_config", None)
        sp = int(_cfg(eng_cfg, "ulysses_sequence_parallel_size", 1) or 1) if eng_cfg is not None else 1
        sp = max(sp, int(_cfg(cfg, "ulysses_sequence_parallel_size", 1) or 1))
        if eng_cfg is not None:
            sp *= int(_cfg(eng_cfg, "tensor_model_parallel_size", 1) or 1) * int(_cfg(eng_cfg, "pipeline_model_parallel_size", 1) or 1)
            sp *= int(_cfg(eng_cfg, "context_parallel_size", 1) or 1)
        dp = max(self.world // max(sp, 1), 1)
        mini = int(getattr(cfg, mini_key)) * n // dp
        assert mini > 0, f"{mini_key} {getattr(cfg, mini_key)} * n {n} must be >= data-parallel size {dp}"
        object.__setattr__(cfg, mini_key, mini)
        micro = getattr(cfg, micro_key, None)
        if micro is not None:
            per = max(int(micro) // dp, 1)
            object.__setattr__(cfg, micro_key + "_per_gpu", per)
        per_gpu = getattr(cfg, micro_key + "_per_gpu", None)
        if per_gpu is not None and not getattr(cfg, "use_dynamic_bsz", False):
            assert mini % per_gpu == 0, f"normalized {mini_key} {mini} should be divisible by {micro_key}_per_gpu {per_gpu}"


def _spmd() -> bool:
    return os.environ.get("VERL_B200_SPMD") == "1"


def sp_pool(data: DataProto, engine) -> tuple[DataProto, Optional[tuple]]:
    """SPMD launch with Ulysses or tensor parallelism: every rank drives its own share of the batch, but the ranks of
    a sequence-parallel / tensor-parallel group must work on the same samples. Pool the group's shares (rank order); :func:`sp_unpool` hands every rank the
    rows of its own share back. A no-op under the dispatching worker group (the dispatch already sends a group the
    same samples) and without sequence parallelism."""
    sp = int(getattr(engine, "mp_size", getattr(engine, "sp_size", 1)) or 1)
    if sp <= 1 or not _spmd():
        return data, None
    parts = [None] * sp
    dist.all_gather_object(parts, data, group=engine.mp_group)
    pooled = DataProto.concat(parts)
    pooled.meta_info = dict(data.meta_info)
    tok = pooled.meta_info.get("global_token_num")
    if tok is not None and data.meta_info.get("token_num_is_local"):
        pooled.meta_info["global_token_num"] = [t for p in parts for t in (p.meta_info.get("global_token_num") or [])]
    lo = sum(len(p) for p in parts[: engine.mp_rank])
    return pooled, (lo, len(data))


def sp_unpool(out: DataProto, info: Optional[tuple]) -> DataProto:
    if info is None or out.batch is None:
        return out
    lo, n = info
    return out[lo : lo + n]


class ActorRolloutRefWorker(_WorkerBase):
    """role in {"actor", "rollout", "ref", "actor_rollout", "actor_rollout_ref"}."""

    def __init__(self, config, role: str = "actor_rollout_ref", device_name: Optional[str] = None, **kwargs):
        super().__init__(config, device_name)
        self.role = role
        assert role in ("actor", "rollout", "ref", "actor_rollout", "actor_rollout_ref")
        self._is_actor = role in ("actor", "actor_rollout", "actor_rollout_ref")
        self._is_rollout = role in ("rollout", "actor_rollout", "actor_rollout_ref")
        self._is_ref = role in ("ref", "actor_rollout_ref")
        self.actor_cfg = omega_conf_to_dataclass(config.actor) if self._is_actor else None
        self.ref_cfg = omega_conf_to_dataclass(config.ref) if self._is_ref and config.get("ref") is not None else None
        self.rollout_cfg = omega_conf_to_dataclass(config.rollout) if self._is_rollout else None
        n = int(_cfg(config.get("rollout", {}), "n", 1))
        if self._is_actor:
            self._norm_batch(self.actor_cfg, n=n)
        # Ulysses: the ranks of a sequence-parallel group share one data-parallel rank and the first one reports
        # (dispatch of verl/single_controller/base/decorator.py:297-328, registration of fsdp_workers.py:146-273)
        def mesh_of(c):
            """(data-parallel rank, reports results) of this rank under the engine's layout: pipeline stages are
            consecutive blocks of ranks; inside a block ``tp x sp x cp`` consecutive ranks share their samples; the last
            stage's first rank of such a group reports."""
            if c is None:
                return self.dp_rank, True
            ec = _cfg(c, "fsdp_config", None)
            inner = (int(_cfg(ec, "ulysses_sequence_parallel_size", 1) or 1) * int(_cfg(ec, "tensor_model_parallel_size", 1) or 1)
                     * int(_cfg(ec, "context_parallel_size", 1) or 1))
            pp = int(_cfg(ec, "pipeline_model_parallel_size", 1) or 1)
            S = max(self.world // pp, 1)
            local = self.dp_rank % S
            return local // inner, (local % inner == 0 and self.dp_rank // S == pp - 1)

        (dp_a, col_a), (dp_r, col_r) = mesh_of(self.actor_cfg), mesh_of(self.ref_cfg if self.ref_cfg is not None else self.actor_cfg)
        self._register_dispatch_collect_info("actor", dp_rank=dp_a, is_collect=col_a)
        self._register_dispatch_collect_info("ref", dp_rank=dp_r, is_collect=col_r)
        # a rollout replica spans `tensor_model_parallel_size` consecutive ranks: they receive the same prompts and
        # the first one reports (verl/workers/rollout/replica.py:96-143)
        self.rollout_tp = int(_cfg(self.rollout_cfg, "tensor_model_parallel_size", 1) or 1) if self._is_rollout else 1
        if self._is_rollout:
            self._check_rollout_parallelism()
        self._register_dispatch_collect_info("rollout", dp_rank=self.dp_rank // self.rollout_tp,
                                             is_collect=self.dp_rank % self.rollout_tp == 0)
        self.tp_group = self.tp_comm = None
        self.actor_engine = self.ref_engine = None
        self.actor = self.ref_policy = None
        self.rollout_engine = None
        self.rollout_model = None
        self._rollout_flat = None
        self.timing = {}

    # ------------------------------------------------------------------ build
    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def init_model(self):
        model_cfg, state = resolve_model_config(self.config.model)
        self.model_config = model_cfg
        gc = bool(_cfg(self.config.model, "enable_gradient_checkpointing", True))
        seed = int(_cfg(_cfg(self.actor_cfg, "fsdp_config", None), "seed", 42)) if self.actor_cfg else 42
        group = dist.group.WORLD if dist.is_initialized() and self.world > 1 else None
        comm = self._make_comm()
        tm = _cfg(self.config.model, "tiled_mlp", None) or {}
        tiled = int(_cfg(tm, "num_shards", 4)) if _cfg(tm, "enabled", False) else 0
        lora_rank = int(_cfg(self.config.model, "lora_rank", 0) or 0)
        lora = {"rank": lora_rank, "alpha": _cfg(self.config.model, "lora_alpha", 16),
                "target_modules": _cfg(self.config.model, "target_modules", "all-linear"),
                "exclude_modules": _cfg(self.config.model, "exclude_modules", None)} if lora_rank > 0 else None
        self._lora = lora is not None
        if self._lora and self._is_rollout and self.rollout_tp > 1:
            raise ValueError("LoRA training syncs merged weights into a whole-model rollout copy: set "
                             "rollout.tensor_model_parallel_size=1 with model.lora_rank > 0")
        if self._is_actor:
            self.actor_engine = NativeEngine(model_cfg, self.actor_cfg.fsdp_config, self.actor_cfg.optim,
                                             device=str(self.device), group=group, seed=seed, state_dict=state,
                                             comm=comm, gradient_checkpointing=gc, tiled_mlp_shards=tiled, lora=lora,
                                             frozen_prefixes=("visual.",) if _cfg(self.actor_cfg, "freeze_vision_tower", False)
                                             else ()).initialize()
            self.actor_engine.clip_grad_override = _role_clip(self.actor_cfg)
            self.actor = DataParallelPPOActor(self.actor_cfg, self.actor_engine)
        if self._is_ref and not (self._lora and self._is_actor):  # LoRA: the reference is the actor with adapters off
            ref_eng_cfg = self.ref_cfg.fsdp_config if self.ref_cfg is not None else None
            self.ref_engine = NativeEngine(model_cfg, ref_eng_cfg, None, device=str(self.device), group=group, seed=seed,
                                           state_dict=state, trainable=False, comm=comm).initialize()
            self.ref_policy = DataParallelPPOActor(self.ref_cfg or self.actor_cfg, self.ref_engine)
            self.ref_policy.record_routing = False
            if self.actor_cfg is not None:  # the reference policy evaluates the same batches: same layout choice
                self.ref_policy.use_prefix_grouper = bool(_cfg(self.actor_cfg, "use_prefix_grouper", False))
        if self._is_rollout:
            self._build_rollout(model_cfg, state, seed)
        if self.device.type == "cuda":
            torch.cuda.empty_cache()

    def _make_comm(self):
        """Peer-memory communicator of the whole job (``comm_kind`` records which collective path runs: "peer", "nccl"
        or "none"). With ``VERL_B200_REQUIRE_PEER_COMM=1`` a failed set-up raises instead of falling back to NCCL."""
        self.comm, self.comm_kind = None, "none"
        if self.world <= 1:
            return None
        self.comm_kind = "nccl" if self.device.type == "cuda" else "gloo"
        if self.device.type != "cuda" or os.environ.get("VERL_B200_DISABLE_PEER_COMM"):
            return None
        try:
            from ..parallel.peer_comm import PeerComm

            self.comm = PeerComm(dist.group.WORLD)
            self.comm_kind = "peer"
        except Exception as e:  # peer memory not available: plain NCCL collectives
            if os.environ.get("VERL_B200_REQUIRE_PEER_COMM") == "1":
                raise RuntimeError(f"peer-memory collectives are required but could not be set up: {e}") from e
            if self.dp_rank == 0:
                print(f"[verl_b200] peer-memory collectives unavailable ({type(e).__name__}: {e}); using NCCL")
        return self.comm

    def _check_rollout_parallelism(self):
        """Parallel sizes of a rollout replica that this engine cannot serve are errors, not silently ignored."""
        rc, tp = self.rollout_cfg, self.rollout_tp
        pp = int(_cfg(rc, "pipeline_model_parallel_size", 1) or 1)
        dpr = int(_cfg(rc, "data_parallel_size", 1) or 1)
        ep = int(_cfg(rc, "expert_parallel_size", 1) or 1)
        if pp != 1 or dpr != 1:
            raise ValueError("rollout.pipeline_model_parallel_size and rollout.data_parallel_size must be 1: one NVSwitch "
                             "box is served by tensor-parallel replicas (replicas = GPUs / tensor_model_parallel_size)")
        if tp < 1 or self.world % tp != 0:
            raise ValueError(f"rollout.tensor_model_parallel_size={tp} does not divide the {self.world} rank(s) of this "
                             "job; set it to a divisor (1 runs one replica per GPU)")
        if ep not in (1, tp):
            raise ValueError(f"rollout.expert_parallel_size={ep}: experts are sharded over the ranks of a replica, so it "
                             f"must be 1 or equal to tensor_model_parallel_size ({tp})")

    def _setup_rollout_tp(self):
        """Process group (and, on CUDA, peer-memory communicator) of this rank's rollout replica."""
        tp = self.rollout_tp
        mine = None
        for g in range(self.world // tp):  # collective: every rank creates every group
            ranks = list(range(g * tp, (g + 1) * tp))
            grp = dist.new_group(ranks)
            if self.dp_rank in ranks:
                mine = grp
        self.tp_group = mine
        # control group of the replica for the server mode (object broadcasts between the engine threads; gloo so
        # that a waiting follower does not occupy the GPU)
        ctrl = None
        for g in range(self.world // tp):
            ranks = list(range(g * tp, (g + 1) * tp))
            grp = dist.new_group(ranks, backend="gloo")
            if self.dp_rank in ranks:
                ctrl = grp
        self.tp_ctrl_group = ctrl
        if self.device.type == "cuda":
            from ..parallel.peer_comm import PeerComm

            self.tp_comm = self.comm if tp == self.world and self.comm is not None else PeerComm(mine)

    def _build_rollout(self, model_cfg: ModelConfig, state, seed: int):
        from ..rollout import NativeRolloutEngine

        rc = self.rollout_cfg
        tp = self.rollout_tp
        dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        if tp > 1:
            from ..parallel.reshard import shard_state_dict, tp_model_config

            self._setup_rollout_tp()
            tp_rank = self.dp_rank % tp
            self.rollout_model = CausalLM(tp_model_config(model_cfg, tp_rank, tp), dtype=dtype, device=self.device)
            if self._is_actor and not self.actor_engine.model_parallel:
                self._bind_rollout_to_flat(tp_rank, tp)
            elif self._is_actor:
                self._generic_sync = True
            else:
                if state is None:  # random init of the whole model, then this rank's slices (same seed on all ranks)
                    full = CausalLM(model_cfg, dtype=dtype, device=self.device).init_weights(seed)
                    state = dict(full.state_dict())
                    del full
                sl = shard_state_dict(model_cfg, {k: v.to(dtype) for k, v in state.items()}, tp_rank, tp)
                self.rollout_model.load_state_dict(sl, strict=False)
        elif self._is_actor and self.world == 1 and not getattr(self, "_lora", False) and not self.actor_engine.model_parallel:
            self.rollout_model = self.actor_engine.model  # same tensors: weight sync is free
        else:
            self.rollout_model = CausalLM(model_cfg, dtype=dtype, device=self.device)
            if self._is_actor and not self.actor_engine.model_parallel:
                self._bind_rollout_to_flat()
            elif self._is_actor:
                self._generic_sync = True  # a tensor-parallel trainer: weights travel as whole (HF-named) tensors
            elif state is not None:
                self.rollout_model.load_state_dict({k: v.to(dtype) for k, v in state.items()}, strict=False)
            else:
                self.rollout_model.init_weights(seed)
        max_len = rc.max_model_len or (rc.prompt_length + rc.response_length)
        kw = dict(_cfg(rc.engine_kwargs, "native", {}) or {})
        self.rollout_engine = NativeRolloutEngine(
            self.rollout_model, max_num_seqs=rc.max_num_seqs, max_model_len=max_len,
            max_num_batched_tokens=max(rc.max_num_batched_tokens, rc.prompt_length),
            gpu_memory_utilization=rc.gpu_memory_utilization, enable_prefix_caching=rc.enable_prefix_caching,
            record_routing=bool(_cfg(rc, "enable_rollout_routing_replay", False)),
            enforce_eager=rc.enforce_eager, seed=seed + 1000 * (self.dp_rank // tp),
            cudagraph_capture_sizes=rc.cudagraph_capture_sizes, quantization=_cfg(rc, "quantization", None),
            tp_group=self.tp_group, tp_comm=self.tp_comm, full_config=model_cfg, **kw)
        if getattr(self, "_generic_sync", False):
            self.rollout_engine.update_weights(self.actor_engine.get_per_tensor_param())
        if rc.free_cache_engine:
            self.rollout_engine.sleep()

    def _bind_rollout_to_flat(self, tp_rank: int = 0, tp_size: int = 1):
        """Rollout parameters become views into one destination buffer; a weight sync executes a precomputed
        copy table (trainer shards on all ranks -> this rank's rollout layout, tensor-parallel slices included) in a
        single kernel launch."""
        from ..parallel.reshard import RolloutWeights

        self._rollout_flat = RolloutWeights(self.model_config, self.actor_engine.zero, self.rollout_model, tp_rank, tp_size)
        self._sync_rollout_weights()

    @torch.no_grad()
    def _sync_rollout_weights(self):
        self._rollout_flat.sync()
        if getattr(self, "_lora", False):
            # the rollout copy now holds the frozen base weights: add the adapters' deltas (merged-weight sync)
            self.actor_engine.merge_lora_into(self.rollout_model)

    # ---------------------------------------------------------------- rollout
    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("rollout"))
    def generate_sequences(self, prompts: DataProto) -> DataProto:
        """prompts.batch: input_ids / attention_mask / position_ids (left-padded). Returns prompts + responses
        in the reference's layout (``prompts, responses, input_ids, attention_mask, position_ids,
        response_mask, rollout_log_probs``)."""
        from ..rollout import SamplingParams
        from ..rollout.postprocess import assemble_rollout_batch

        rc = self.rollout_cfg
        eng = self.rollout_engine
        t0 = time.perf_counter()
        eng.wake_up()
        stats0 = dict(eng.stats)
        meta = prompts.meta_info
        validate = meta.get("validate", False)
        do_sample = meta.get("do_sample", rc.do_sample if not validate else rc.val_kwargs.do_sample)
        temp = meta.get("temperature", rc.val_kwargs.temperature if validate else rc.temperature)
        sp = SamplingParams(temperature=float(temp) if do_sample else 0.0,
                            top_k=int(meta.get("top_k", rc.val_kwargs.top_k if validate else rc.top_k)),
                            top_p=float(meta.get("top_p", rc.val_kwargs.top_p if validate else rc.top_p)),
                            max_tokens=int(meta.get("response_length", rc.response_length)), ignore_eos=rc.ignore_eos)
        ids, mask = prompts.batch["input_ids"], prompts.batch["attention_mask"]
        prompt_lists = [row[m.bool()].tolist() for row, m in zip(ids.cpu(), mask.cpu())]
        if self.rollout_tp > 1 and os.environ.get("VERL_B200_SPMD") == "1":
            # SPMD launch: every rank drives its own share of the batch, but the ranks of a replica must serve the
            # same requests: pool the replica's prompts, generate once, keep this rank's rows
            pooled = [None] * self.rollout_tp
            dist.all_gather_object(pooled, prompt_lists, group=self.tp_group)
            lo = sum(len(p) for p in pooled[: self.dp_rank % self.rollout_tp])
            outs = eng.generate([p for part in pooled for p in part], sp)[lo : lo + len(prompt_lists)]
        else:
            mm = prompts.non_tensor_batch.get("multi_modal_inputs")
            outs = eng.generate(prompt_lists, sp, multi_modal_inputs=list(mm) if mm is not None else None)
        out = assemble_rollout_batch(ids.cpu(), mask.cpu(), outs, rc.response_length, pad_token_id=meta.get("pad_token_id", 0),
                                     with_logprobs=True)
        if getattr(self.model_config, "is_vl", False):
            # [B, 4, S]: text positions + multimodal RoPE positions of prompt and response (the actor's input layout)
            from ..utils.dataset.vision_utils import vl_position_ids

            v = self.model_config.extra.get("vision_config") or {}
            out.batch["position_ids"] = vl_position_ids(out.batch["input_ids"], out.batch["attention_mask"],
                                                        prompts.non_tensor_batch.get("multi_modal_inputs"),
                                                        self.model_config.image_token_id, int(v.get("spatial_merge_size", 2)),
                                                        video_token_id=self.model_config.extra.get("video_token_id"))
        gen_time = time.perf_counter() - t0
        out.non_tensor_batch.update(prompts.non_tensor_batch)
        n_tok = int(out.batch["response_mask"].sum())
        out.meta_info["metrics"] = {"rollout/generate_sequences_s": gen_time,
                                    "rollout/num_preempted": float(sum(o.num_preempted for o in outs)),
                                    "rollout/tokens_per_s": n_tok / max(gen_time, 1e-9)}
        for k_ in ("step_s", "decode_wait_s", "prefill_s", "decode_steps", "steps"):  # where the engine's time went
            out.meta_info["metrics"][f"rollout/engine_{k_}"] = float(eng.stats[k_] - stats0[k_])
        t_sleep = time.perf_counter()
        if rc.free_cache_engine and not meta.get("keep_cache", False):
            eng.sleep()
        # this rank's own times (the metrics above travel with the batch and get merged over ranks)
        self.last_rollout_times = {"generate_s": gen_time, "sleep_s": time.perf_counter() - t_sleep,
                                   "engine_step_s": float(eng.stats["step_s"] - stats0["step_s"])}
        return out

    # ---------------------------------------------------------------- log-probs
    def _lp_meta(self, data: DataProto, cfg, prefix="log_prob_"):
        data.meta_info.setdefault("micro_batch_size", _cfg(cfg, prefix + "micro_batch_size_per_gpu", None))
        data.meta_info.setdefault("max_token_len", _cfg(cfg, prefix + "max_token_len_per_gpu", 16384))
        data.meta_info.setdefault("use_dynamic_bsz", bool(_cfg(cfg, prefix + "use_dynamic_bsz", False)))
        data.meta_info.setdefault("temperature", _cfg(self.config.get("rollout", {}), "temperature", 1.0))

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("actor"))
    def compute_log_prob(self, data: DataProto) -> DataProto:
        assert self._is_actor
        self._lp_meta(data, self.rollout_cfg if self.rollout_cfg is not None else self.config.rollout)
        data, pooled = sp_pool(data, self.actor_engine)
        with self.actor_engine.eval_mode():
            lp, ent = self.actor.compute_log_prob(data, calculate_entropy=True)
        tensors = {"old_log_probs": lp.cpu(), "entropys": ent.cpu()}
        if self.actor.last_routed_experts is not None:  # router replay R2: the experts this pass routed every token to
            tensors["routed_experts"] = self.actor.last_routed_experts
        if self.actor.last_sum_pi_squared is not None:  # actor.calculate_sum_pi_squared (optimal token baseline)
            tensors["sum_pi_squared"] = self.actor.last_sum_pi_squared.cpu()
        out = DataProto.from_dict(tensors=tensors, meta_info={"temperature": data.meta_info["temperature"]})
        return sp_unpool(out, pooled)

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("ref"))
    def compute_ref_log_prob(self, data: DataProto) -> DataProto:
        assert self._is_ref
        self._lp_meta(data, self.ref_cfg or self.config.ref)
        data, pooled = sp_pool(data, self.ref_engine if self.ref_engine is not None else self.actor_engine)
        if self.ref_engine is None:  # LoRA: frozen base weights of the actor engine
            with self.actor_engine.eval_mode(), self.actor_engine.disable_adapter():
                lp, _ = self.actor.compute_log_prob(data, calculate_entropy=False)
            return sp_unpool(DataProto.from_dict(tensors={"ref_log_prob": lp.cpu()}), pooled)
        with self.ref_engine.eval_mode():
            lp, _ = self.ref_policy.compute_log_prob(data, calculate_entropy=False)
        return sp_unpool(DataProto.from_dict(tensors={"ref_log_prob": lp.cpu()}), pooled)

    # ------------------------------------------------------------------ update
    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("actor"))
    def update_actor(self, data: DataProto) -> DataProto:
        assert self._is_actor
        data.meta_info.setdefault("temperature", _cfg(self.config.get("rollout", {}), "temperature", 1.0))
        data, _ = sp_pool(data, self.actor_engine)
        t0 = time.perf_counter()
        with self.actor_engine.train_mode():
            metrics = self.actor.update_policy(data)
        dt = time.perf_counter() - t0
        lr = self.actor_engine._lr()
        self.actor_engine.lr_scheduler_step()
        metrics["actor/lr"] = lr
        tokens = data.meta_info.get("global_token_num")
        if tokens is not None:
            from ..utils.flops_counter import FlopsCounter

            est, promised = FlopsCounter(self.model_config).estimate_flops(tokens, dt)
            # tokens of this call's batch are processed by `sp` ranks (local counts) or by the whole job (global counts)
            denom = max(int(getattr(self.actor_engine, "mp_size", 1) or 1), 1) if data.meta_info.get("token_num_is_local") \
                else self.world
            metrics["perf/mfu/actor"] = est * self.actor_cfg.ppo_epochs / promised / denom
        return DataProto(meta_info={"metrics": metrics})

    @register(dispatch_mode=Dispatch.ONE_TO_ALL, blocking=False)
    def update_weights(self, global_steps: Optional[int] = None):
        """Push the trainer's current weights into the rollout engine."""
        t0 = time.perf_counter()
        if self._is_actor and self._is_rollout and self._rollout_flat is not None:
            self._sync_rollout_weights()
        elif self._is_actor and self._is_rollout and getattr(self, "_generic_sync", False):
            self.rollout_engine.update_weights(self.actor_engine.get_per_tensor_param())
        if self.rollout_engine is not None:
            self.rollout_engine.refresh_quantization()  # fp8 rollout: re-quantise from the fresh bf16 weights
            self.rollout_engine.clear_kv_cache()
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        return {"resync_s": time.perf_counter() - t0}

    # -------------------------------------------------------------- checkpoint
    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def save_checkpoint(self, local_path, hdfs_path=None, global_step=0, max_ckpt_to_keep=None):
        assert self._is_actor
        contents = tuple(_cfg(self.actor_cfg.checkpoint, "save_contents", ("model", "optimizer", "extra")))
        self.actor_engine.save_checkpoint(local_path, hdfs_path, global_step, max_ckpt_to_keep, save_contents=contents)
        if dist.is_initialized():
            dist.barrier()

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def load_checkpoint(self, local_path, hdfs_path=None, del_local_after_load=False):
        assert self._is_actor
        contents = tuple(_cfg(self.actor_cfg.checkpoint, "load_contents", ("model", "optimizer", "extra")))
        self.actor_engine.load_checkpoint(local_path, hdfs_path, del_local_after_load, load_contents=contents)
        if self._rollout_flat is not None:
            self._sync_rollout_weights()

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def start_profile(self, **kwargs):
        from ..utils.profiler.profile import DistProfiler

        self._profiler = DistProfiler(self.dp_rank, _cfg(self.actor_cfg or self.rollout_cfg, "profiler", None))
        self._profiler.start(**kwargs)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def stop_profile(self):
        if getattr(self, "_profiler", None) is not None:
            self._profiler.stop()


    # ------------------------------------------------------------ rollout server
    def get_async_server(self):
        """The token-in / token-out server around this worker's rollout engine (created on first use)."""
        if getattr(self, "_async_server", None) is None:
            from .rollout.async_server import NativeAsyncServer

            rc = self.rollout_cfg
            self.rollout_engine.wake_up()
            tp_group = getattr(self, "tp_ctrl_group", None) if self.rollout_tp > 1 else None
            self._async_server = NativeAsyncServer(self.rollout_engine, response_length=int(rc.response_length),
                                                   prompt_length=int(rc.prompt_length), tp_group=tp_group)
            if rc.free_cache_engine and self._async_server.tp_leader:
                import asyncio

                asyncio.run(self._async_server.sleep())  # under tensor parallelism the followers mirror it
        return self._async_server

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def start_rollout_server(self, address: str = "127.0.0.1") -> str:
        """Serve the rollout engine over HTTP from this worker process; returns ``host:port`` (the driver's agent
        loops talk to it through :class:`HttpServerHandle`)."""
        if getattr(self, "_async_server_address", None) is None:
            from .rollout.async_server import serve_in_thread

            srv = self.get_async_server()
            # a tensor-parallel replica has ONE endpoint, on its first rank; the other ranks follow it ("" here)
            self._async_server_address = serve_in_thread(srv, address) if srv.tp_leader else ""
        return self._async_server_address


class AsyncActorRolloutRefWorker(ActorRolloutRefWorker):
    """Same worker; kept as a distinct name because the reference selects it for ``rollout.mode=async``."""


class CriticWorker(_WorkerBase):
    def __init__(self, config, device_name: Optional[str] = None, **kwargs):
        super().__init__(config, device_name)
        self.critic_cfg = omega_conf_to_dataclass(config)
        self._norm_batch(self.critic_cfg, n=int(_cfg(self.critic_cfg, "rollout_n", 1)))
        self._register_dispatch_collect_info("critic", dp_rank=self.dp_rank, is_collect=True)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def init_model(self):
        model_cfg, state = resolve_model_config(self.critic_cfg.model)
        model_cfg.num_labels = 1
        if int(_cfg(self.critic_cfg.model, "lora_rank", 0) or 0) > 0 and self.dp_rank == 0:
            # adapters on a critic would leave its freshly initialised value head frozen: the critic trains in full
            print("[verl_b200] critic.model.lora_rank is ignored: LoRA applies to the actor (and SFT); the critic trains all weights")
        if state is not None:
            state = {k: v for k, v in state.items() if not k.startswith("lm_head")}
        group = dist.group.WORLD if dist.is_initialized() and self.world > 1 else None
        eng_cfg = _cfg(self.critic_cfg.model, "fsdp_config", None)
        self.engine = NativeEngine(model_cfg, eng_cfg, self.critic_cfg.optim, value_head=True, device=str(self.device),
                                   group=group, seed=int(_cfg(eng_cfg, "seed", 42)), state_dict=state,
                                   gradient_checkpointing=bool(_cfg(self.critic_cfg.model, "enable_gradient_checkpointing", True))
                                   ).initialize()
        self.engine.clip_grad_override = _role_clip(self.critic_cfg)
        self.critic = DataParallelPPOCritic(self.critic_cfg, self.engine)
        self.model_config = model_cfg

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("critic"))
    def compute_values(self, data: DataProto) -> DataProto:
        c = self.critic_cfg
        data.meta_info.setdefault("micro_batch_size", c.forward_micro_batch_size_per_gpu or c.ppo_micro_batch_size_per_gpu)
        data.meta_info.setdefault("max_token_len", c.forward_max_token_len_per_gpu)
        data.meta_info.setdefault("use_dynamic_bsz", c.use_dynamic_bsz)
        data, pooled = sp_pool(data, self.engine)
        with self.engine.eval_mode():
            values = self.critic.compute_values(data)
        return sp_unpool(DataProto.from_dict(tensors={"values": values.cpu()}), pooled)

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("critic"))
    def update_critic(self, data: DataProto) -> DataProto:
        data, _ = sp_pool(data, self.engine)
        with self.engine.train_mode():
            metrics = self.critic.update_critic(data)
        metrics["critic/lr"] = self.engine._lr()
        self.engine.lr_scheduler_step()
        return DataProto(meta_info={"metrics": metrics})

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def save_checkpoint(self, local_path, hdfs_path=None, global_step=0, max_ckpt_to_keep=None):
        self.engine.save_checkpoint(local_path, hdfs_path, global_step, max_ckpt_to_keep)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def load_checkpoint(self, local_path, hdfs_path=None, del_local_after_load=True):
        self.engine.load_checkpoint(local_path, hdfs_path, del_local_after_load)


class RewardModelWorker(_WorkerBase):
    """Discriminative reward model: a value-head transformer whose score at the last valid response token is
    the sequence reward (verl/workers/fsdp_workers.py:1626-1981)."""

    def __init__(self, config, device_name: Optional[str] = None, **kwargs):
        super().__init__(config, device_name)
        self._register_dispatch_collect_info("reward", dp_rank=self.dp_rank, is_collect=True)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def init_model(self):
        model_cfg, state = resolve_model_config(self.config.model)
        model_cfg.num_labels = 1
        if state is not None:
            state = {k: v for k, v in state.items() if not k.startswith("lm_head")}
        group = dist.group.WORLD if dist.is_initialized() and self.world > 1 else None
        self.engine = NativeEngine(model_cfg, None, None, value_head=True, device=str(self.device), group=group,
                                   trainable=False, state_dict=state).initialize()

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("reward"))
    def compute_rm_score(self, data: DataProto) -> DataProto:
        from ..models import PackedBatch

        ids, mask = data.batch["input_ids"].to(self.device), data.batch["attention_mask"].to(self.device)
        R = data.batch["responses"].shape[-1]
        micro = int(_cfg(self.config, "micro_batch_size_per_gpu", None) or len(data))
        scores = []
        with torch.no_grad():
            for s in range(0, len(data), micro):
                i, m = ids[s : s + micro], mask[s : s + micro]
                packed, _ = PackedBatch.from_padded(i, m)
                last_rows = packed.cu_seqlens[1:].long() - 1
                scores.append(self.engine.forward_values(packed, last_rows))
        score = torch.cat(scores).float().cpu()
        resp_len = data.batch["attention_mask"][:, -R:].sum(-1).clamp(min=1)
        rm = torch.zeros(len(data), R)
        rm[torch.arange(len(data)), resp_len - 1] = score
        return DataProto.from_dict(tensors={"rm_scores": rm})
