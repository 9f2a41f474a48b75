"""Typed worker configs: actor / critic / engine / optimizer / model / rollout / reward model.

Field names and defaults follow verl/workers/config/{actor,critic,engine,model,optimizer,rollout,
reward_model}.py so that YAML files and CLI overrides written for the reference keep their meaning.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from ...base_config import BaseConfig
from ...trainer.config import CheckpointConfig
from ...utils.profiler.config import ProfilerConfig

__all__ = [
    "OptimizerConfig", "FSDPOptimizerConfig", "McoreOptimizerConfig", "EngineConfig", "FSDPEngineConfig",
    "McoreEngineConfig", "McoreCriticConfig", "TrainingWorkerConfig", "PolicyLossConfig", "RouterReplayConfig", "ActorConfig",
    "FSDPActorConfig", "McoreActorConfig", "MtpConfig", "HFModelConfig", "CriticConfig", "FSDPCriticConfig",
    "FSDPCriticModelCfg", "SamplingConfig", "MultiTurnConfig", "CustomAsyncServerConfig", "AgentLoopConfig",
    "TraceConfig", "ServerConfig", "PrometheusConfig", "CheckpointEngineConfig", "RolloutConfig",
    "SandboxFusionConfig", "RewardModelConfig", "RewardManagerConfig", "ModuleConfig",
]


# --------------------------------------------------------------------------- optimizer
@dataclass
class OptimizerConfig(BaseConfig):
    _mutable_fields = {"clip_grad", "total_training_steps", "lr_warmup_steps"}
    lr: float = 1e-3
    lr_warmup_steps_ratio: float = 0.0
    total_training_steps: int = -1
    weight_decay: float = 0.01
    lr_warmup_steps: Optional[int] = -1
    betas: tuple = (0.9, 0.999)
    clip_grad: float = 1.0

    def __post_init__(self):
        assert self.lr != "???", "optimizer lr must be set"


@dataclass
class FSDPOptimizerConfig(OptimizerConfig):
    _mutable_fields = OptimizerConfig._mutable_fields | {"lr_scheduler_type"}
    optimizer: str = "AdamW"
    optimizer_impl: str = "torch.optim"
    min_lr_ratio: Optional[float] = None
    num_cycles: float = 0.5
    lr_scheduler_type: str = "constant"
    warmup_style: Optional[str] = None
    override_optimizer_config: Optional[dict] = None

    def __post_init__(self):
        if self.warmup_style is not None:
            assert self.warmup_style in ("constant", "cosine")
            object.__setattr__(self, "lr_scheduler_type", self.warmup_style)
        assert self.lr_scheduler_type in ("constant", "cosine", "wsd")
        super().__post_init__()


@dataclass
class McoreOptimizerConfig(OptimizerConfig):
    optimizer: str = "adam"
    lr_warmup_init: float = 0.0
    lr_decay_steps: Optional[int] = None
    lr_decay_style: str = "linear"
    min_lr: float = 0.0
    weight_decay_incr_style: str = "constant"
    lr_wsd_decay_style: str = "exponential"
    lr_wsd_decay_steps: Optional[int] = None
    use_checkpoint_opt_param_scheduler: bool = False
    override_optimizer_config: Optional[dict] = None


# ------------------------------------------------------------------------------ engine
@dataclass
class EngineConfig(BaseConfig):
    _mutable_fields = {"use_dynamic_bsz", "max_token_len_per_gpu", "micro_batch_size_per_gpu", "infer_max_token_len_per_gpu",
                       "infer_micro_batch_size_per_gpu", "use_fused_kernels", "use_remove_padding", "forward_only",
                       "param_offload"}
    param_offload: bool = False
    optimizer_offload: bool = False
    grad_offload: bool = False
    forward_only: bool = False
    strategy: Optional[str] = None
    dtype: str = "bfloat16"
    use_dynamic_bsz: bool = True
    max_token_len_per_gpu: Optional[int] = None
    micro_batch_size_per_gpu: Optional[int] = None
    infer_max_token_len_per_gpu: Optional[int] = None
    infer_micro_batch_size_per_gpu: Optional[int] = None
    use_fused_kernels: bool = False
    use_remove_padding: bool = True
    seed: int = 42
    full_determinism: bool = False


@dataclass
class FSDPEngineConfig(EngineConfig):
    """Sharded data-parallel engine options. ``strategy`` accepts fsdp / fsdp2 (both map to the native
    ZeRO-3 engine here). ``fsdp_size`` in ``[1, world)`` selects hybrid sharding: parameters, gradients and optimizer
    state are sharded over ``fsdp_size`` consecutive ranks and replicated over the ``world / fsdp_size`` groups;
    -1 (default) shards over the whole data-parallel group."""

    wrap_policy: dict = field(default_factory=dict)
    offload_policy: bool = False
    reshard_after_forward: bool = True
    fsdp_size: int = -1
    forward_prefetch: bool = False
    model_dtype: str = "fp32"
    use_orig_params: bool = False
    mixed_precision: Optional[dict] = None
    ulysses_sequence_parallel_size: int = 1
    # context parallelism: this many consecutive ranks share a micro-batch, each holding two zig-zag chunks of every
    # sequence (not combinable with Ulysses / tensor / pipeline parallelism)
    context_parallel_size: int = 1
    # model parallelism of the one native engine (the reference reaches these through its Megatron back end):
    # tensor-parallel ranks per model copy, pipeline stages, ranks that share the experts of an MoE model
    tensor_model_parallel_size: int = 1
    pipeline_model_parallel_size: int = 1
    expert_model_parallel_size: int = 1
    entropy_from_logits_with_chunking: bool = False
    use_torch_compile: bool = True
    entropy_checkpointing: bool = False
    # decoder layers whose activations are kept for the backward although gradient checkpointing is on:
    # an integer, or "auto" = as many as fit in the memory that is free when the micro-batch starts
    keep_activation_layers: Any = "auto"
    strategy: str = "fsdp"

    def __post_init__(self):
        assert self.strategy in ("fsdp", "fsdp2", "native"), f"strategy {self.strategy} not supported"


@dataclass
class McoreEngineConfig(EngineConfig):
    """Model-parallel sizes accepted for config compatibility; the native engine honours TP/EP/SP
    through its own parallel plan and keeps PP on NCCL p2p."""

    tensor_model_parallel_size: int = 1
    expert_model_parallel_size: int = 1
    expert_tensor_parallel_size: Optional[int] = None
    pipeline_model_parallel_size: int = 1
    virtual_pipeline_model_parallel_size: Optional[int] = None
    context_parallel_size: int = 1
    sequence_parallel: bool = True
    use_distributed_optimizer: bool = True
    use_dist_checkpointing: bool = False
    dist_checkpointing_path: Optional[str] = None
    override_ddp_config: dict = field(default_factory=dict)
    override_transformer_config: dict = field(default_factory=dict)
    use_mbridge: bool = False
    strategy: str = "megatron"


@dataclass
class TrainingWorkerConfig(BaseConfig):
    model_type: Optional[str] = None
    model_config: Any = None
    engine_config: Any = None
    optimizer_config: Any = None
    checkpoint_config: Any = None
    profiler_config: Any = None


# ------------------------------------------------------------------------------- actor
@dataclass
class PolicyLossConfig(BaseConfig):
    _mutable_fields = {"loss_mode", "rollout_correction"}
    loss_mode: str = "vanilla"
    clip_cov_ratio: float = 0.0002
    clip_cov_lb: float = 1.0
    clip_cov_ub: float = 5.0
    kl_cov_ratio: float = 0.0002
    ppo_kl_coef: float = 0.1
    rollout_correction: Optional[Any] = None


@dataclass
class RouterReplayConfig(BaseConfig):
    mode: str = "disabled"
    record_file: Optional[str] = None
    replay_file: Optional[str] = None

    def __post_init__(self):
        assert self.mode in ("disabled", "R2", "R3"), f"Invalid router_replay mode: {self.mode}"


@dataclass
class ActorConfig(BaseConfig):
    _mutable_fields = {"ppo_mini_batch_size", "ppo_micro_batch_size", "ppo_micro_batch_size_per_gpu",
                       "ppo_infer_micro_batch_size_per_gpu", "global_batch_info", "engine", "model_config"}
    strategy: str = "fsdp"
    ppo_mini_batch_size: int = 256
    ppo_micro_batch_size: Optional[int] = None
    ppo_micro_batch_size_per_gpu: Optional[int] = None
    ppo_infer_micro_batch_size_per_gpu: Optional[int] = None
    use_dynamic_bsz: bool = False
    ppo_max_token_len_per_gpu: int = 16384
    ppo_infer_max_token_len_per_gpu: int = 16384
    clip_ratio: float = 0.2
    clip_ratio_low: float = 0.2
    clip_ratio_high: float = 0.2
    tau_pos: float = 1.0
    tau_neg: float = 1.05
    freeze_vision_tower: bool = False
    policy_loss: PolicyLossConfig = field(default_factory=PolicyLossConfig)
    clip_ratio_c: float = 3.0
    loss_agg_mode: str = "token-mean"
    loss_scale_factor: Optional[int] = None
    entropy_coeff: float = 0
    calculate_entropy: bool = False
    use_kl_loss: bool = False
    use_prefix_grouper: bool = False
    use_torch_compile: bool = True
    kl_loss_coef: float = 0.001
    kl_loss_type: str = "low_var_kl"
    ppo_epochs: int = 1
    shuffle: bool = False
    data_loader_seed: int = 42
    checkpoint: CheckpointConfig = field(default_factory=CheckpointConfig)
    optim: OptimizerConfig = field(default_factory=OptimizerConfig)
    use_fused_kernels: bool = False
    use_remove_padding: bool = True
    calculate_sum_pi_squared: bool = False
    sum_pi_squared_checkpointing: bool = False
    profiler: ProfilerConfig = field(default_factory=ProfilerConfig)
    engine: Any = field(default_factory=dict)
    rollout_n: int = 1
    model_config: Any = None
    router_replay: RouterReplayConfig = field(default_factory=RouterReplayConfig)
    global_batch_info: dict = field(default_factory=dict)
    # reference-policy fields share this class in the YAML tree
    log_prob_micro_batch_size: Optional[int] = None
    log_prob_micro_batch_size_per_gpu: Optional[int] = None
    log_prob_use_dynamic_bsz: bool = False
    log_prob_max_token_len_per_gpu: int = 16384

    def __post_init__(self):
        assert self.strategy != "???"
        valid = ["token-mean", "seq-mean-token-sum", "seq-mean-token-mean", "seq-mean-token-sum-norm"]
        if self.loss_agg_mode not in valid:
            raise ValueError(f"Invalid loss_agg_mode: {self.loss_agg_mode}")

    def validate(self, n_gpus: int, train_batch_size: int, model_config: Any = None):
        """Batch-size consistency (global prompt counts in YAML; see verl/workers/config/actor.py)."""
        if not self.use_dynamic_bsz:
            if train_batch_size < self.ppo_mini_batch_size:
                raise ValueError(f"train_batch_size ({train_batch_size}) must be >= ppo_mini_batch_size ({self.ppo_mini_batch_size})")
            sp = getattr(self, "ulysses_sequence_parallel_size", 1)
            if self.ppo_micro_batch_size is not None:
                if self.ppo_mini_batch_size % self.ppo_micro_batch_size != 0:
                    raise ValueError(f"ppo_mini_batch_size ({self.ppo_mini_batch_size}) must be divisible by "
                                     f"ppo_micro_batch_size ({self.ppo_micro_batch_size})")
                if self.ppo_micro_batch_size * sp < n_gpus:
                    raise ValueError(f"ppo_micro_batch_size ({self.ppo_micro_batch_size}) * sp ({sp}) must be >= n_gpus ({n_gpus})")

    @staticmethod
    def _check_mutually_exclusive(mbs, mbs_per_gpu, name: str):
        if mbs is None and mbs_per_gpu is None:
            raise ValueError(f"[{name}] Please set at least one of '{name}.micro_batch_size' or '{name}.micro_batch_size_per_gpu'.")
        if mbs is not None and mbs_per_gpu is not None:
            raise ValueError(f"[{name}] You have set both micro_batch_size AND micro_batch_size_per_gpu; only the per-GPU form is supported.")


@dataclass
class FSDPActorConfig(ActorConfig):
    strategy: str = "fsdp"
    grad_clip: float = 1.0
    ulysses_sequence_parallel_size: int = 1
    entropy_from_logits_with_chunking: bool = False
    entropy_checkpointing: bool = False
    fsdp_config: FSDPEngineConfig = field(default_factory=FSDPEngineConfig)
    optim: FSDPOptimizerConfig = field(default_factory=lambda: FSDPOptimizerConfig(lr=1e-6))

    def __post_init__(self):
        super().__post_init__()
        object.__setattr__(self, "engine", self.fsdp_config)

    def validate(self, n_gpus: int, train_batch_size: int, model_config: Any = None):
        super().validate(n_gpus, train_batch_size, model_config)
        if self.strategy in ("fsdp", "fsdp2") and self.ulysses_sequence_parallel_size > 1 and model_config is not None:
            if not model_config.get("use_remove_padding", False):
                raise ValueError("When using sequence parallelism for actor/ref policy, you must enable `use_remove_padding`.")


@dataclass
class McoreActorConfig(ActorConfig):
    strategy: str = "megatron"
    data_loader_seed: Optional[int] = None
    load_weight: bool = True
    megatron: McoreEngineConfig = field(default_factory=McoreEngineConfig)
    optim: McoreOptimizerConfig = field(default_factory=McoreOptimizerConfig)


# ------------------------------------------------------------------------------- model
@dataclass
class MtpConfig(BaseConfig):
    enable: bool = False
    enable_train: bool = False
    enable_rollout: bool = False
    detach_encoder: bool = False
    mtp_loss_scaling_factor: float = 0.1
    speculative_algorithm: str = "EAGLE"
    speculative_num_steps: int = 3
    speculative_eagle_topk: int = 1
    speculative_num_draft_tokens: int = 4
    method: str = "mtp"
    num_speculative_tokens: int = 1


@dataclass
class HFModelConfig(BaseConfig):
    _mutable_fields = {"hf_config_path", "tokenizer_path", "hf_config", "generation_config", "tokenizer", "processor",
                       "local_path", "architectures", "local_hf_config_path", "local_tokenizer_path"}
    path: str = "???"
    hf_config_path: Optional[str] = None
    tokenizer_path: Optional[str] = None
    use_shm: bool = False
    trust_remote_code: bool = False
    custom_chat_template: Optional[str] = None
    external_lib: Optional[str] = None
    override_config: dict = field(default_factory=dict)
    enable_gradient_checkpointing: bool = True
    enable_activation_offload: bool = False
    use_remove_padding: bool = True
    lora_rank: int = 0
    lora_alpha: int = 16
    target_modules: Any = "all-linear"
    exclude_modules: Optional[Any] = None
    lora_adapter_path: Optional[str] = None
    use_liger: bool = False
    use_fused_kernels: bool = False
    fused_kernel_options: dict = field(default_factory=dict)
    tiled_mlp: dict = field(default_factory=lambda: {"enabled": False, "num_shards": 4})
    mtp: MtpConfig = field(default_factory=MtpConfig)
    hf_config: Any = None
    tokenizer: Any = None


# ------------------------------------------------------------------------------ critic
@dataclass
class CriticConfig(BaseConfig):
    _mutable_fields = {"ppo_micro_batch_size_per_gpu", "ppo_mini_batch_size", "ppo_micro_batch_size", "model_config",
                       "forward_micro_batch_size_per_gpu", "forward_micro_batch_size"}
    strategy: str = "fsdp"
    ppo_micro_batch_size_per_gpu: Optional[int] = None
    enable: Optional[bool] = None
    rollout_n: int = 1
    ppo_mini_batch_size: int = 1
    use_dynamic_bsz: bool = False
    ppo_max_token_len_per_gpu: int = 32768
    forward_max_token_len_per_gpu: int = 32768
    ppo_epochs: int = 1
    data_loader_seed: int = 42
    shuffle: bool = True
    cliprange_value: float = 0.5
    loss_agg_mode: str = "token-mean"
    ppo_micro_batch_size: Optional[int] = None
    engine: Any = field(default_factory=dict)
    optim: OptimizerConfig = field(default_factory=OptimizerConfig)
    model: Any = field(default_factory=dict)
    model_config: Any = None
    checkpoint: CheckpointConfig = field(default_factory=CheckpointConfig)
    profiler: ProfilerConfig = field(default_factory=ProfilerConfig)

    def validate(self, n_gpus: int, train_batch_size: int):
        if not self.use_dynamic_bsz:
            if train_batch_size < self.ppo_mini_batch_size:
                raise ValueError(f"train_batch_size ({train_batch_size}) must be >= critic.ppo_mini_batch_size ({self.ppo_mini_batch_size})")
            if self.ppo_micro_batch_size is not None and self.ppo_mini_batch_size % self.ppo_micro_batch_size != 0:
                raise ValueError("critic ppo_mini_batch_size must be divisible by ppo_micro_batch_size")


@dataclass
class FSDPCriticModelCfg(BaseConfig):
    path: str = "~/models/deepseek-llm-7b-chat"
    tokenizer_path: Optional[str] = None
    override_config: dict = field(default_factory=dict)
    external_lib: Optional[str] = None
    trust_remote_code: bool = False
    use_shm: bool = False
    enable_activation_offload: bool = False
    enable_gradient_checkpointing: bool = True
    use_remove_padding: bool = False
    fsdp_config: FSDPEngineConfig = field(default_factory=FSDPEngineConfig)
    lora_rank: int = 0
    lora_alpha: int = 16
    target_modules: Any = "all-linear"
    tiled_mlp: dict = field(default_factory=lambda: {"enabled": False, "num_shards": 4})


@dataclass
class FSDPCriticConfig(CriticConfig):
    _mutable_fields = CriticConfig._mutable_fields | {"forward_micro_batch_size", "forward_micro_batch_size_per_gpu"}
    strategy: str = "fsdp"
    forward_micro_batch_size: Optional[int] = None
    forward_micro_batch_size_per_gpu: Optional[int] = None
    ulysses_sequence_parallel_size: int = 1
    grad_clip: float = 1.0
    optim: FSDPOptimizerConfig = field(default_factory=lambda: FSDPOptimizerConfig(lr=1e-5))


@dataclass
class McoreCriticConfig(CriticConfig):
    """Critic section with the reference's Megatron key names; the parallel sizes of ``megatron`` are served by the one
    native engine (``utils.config.translate_megatron_overrides`` moves them to ``model.fsdp_config``)."""

    strategy: str = "megatron"
    nccl_timeout: int = 600
    megatron: McoreEngineConfig = field(default_factory=McoreEngineConfig)
    load_weight: bool = True


# ----------------------------------------------------------------------------- rollout
@dataclass
class SamplingConfig(BaseConfig):
    temperature: float = 1.0
    top_k: int = -1
    top_p: float = 1.0
    do_sample: bool = True
    n: int = 1


@dataclass
class MultiTurnConfig(BaseConfig):
    _mutable_fields = {"max_assistant_turns", "max_user_turns"}
    enable: bool = False
    max_assistant_turns: Optional[int] = None
    tool_config_path: Optional[str] = None
    max_user_turns: Optional[int] = None
    max_parallel_calls: int = 1
    max_tool_response_length: int = 256
    tool_response_truncate_side: str = "middle"
    interaction_config_path: Optional[str] = None
    use_inference_chat_template: bool = False
    tokenization_sanity_check_mode: str = "strict"
    format: str = "hermes"
    num_repeat_rollouts: Optional[int] = None


@dataclass
class CustomAsyncServerConfig(BaseConfig):
    path: Optional[str] = None
    name: Optional[str] = None


@dataclass
class AgentLoopConfig(BaseConfig):
    num_workers: int = 8
    default_agent_loop: str = "single_turn_agent"
    # route plain single-turn rollouts through the agent loops too (they are always used for multi-turn / tools)
    use_agent_loop: bool = False
    agent_loop_config_path: Optional[str] = None
    custom_async_server: CustomAsyncServerConfig = field(default_factory=CustomAsyncServerConfig)


@dataclass
class TraceConfig(BaseConfig):
    backend: Optional[str] = None
    token2text: bool = False
    max_samples_per_step_per_worker: Optional[int] = None

    def __post_init__(self):
        if self.max_samples_per_step_per_worker is not None and self.max_samples_per_step_per_worker < 0:
            raise ValueError("`max_samples_per_step_per_worker` must be a non-negative integer or null.")


@dataclass
class ServerConfig(BaseConfig):
    timeout: float = 60.0
    max_attempts: int = 3
    retry_delay: float = 2.0
    max_connections: int = 1000
    max_start_wait_time: float = 300.0


@dataclass
class PrometheusConfig(BaseConfig):
    enable: bool = False
    port: int = 9090
    file: str = "/tmp/ray/session_latest/metrics/prometheus/prometheus.yml"
    served_model_name: Optional[str] = None


@dataclass
class CheckpointEngineConfig(BaseConfig):
    """Weight-sync backend: ``naive`` (colocated generator), ``nvlink`` (single reshard kernel over
    peer memory), ``nccl`` (bucketed broadcast)."""

    backend: Optional[str] = "naive"
    update_weights_bucket_megabytes: int = 2048
    engine_kwargs: dict = field(default_factory=dict)


@dataclass
class RolloutConfig(BaseConfig):
    _mutable_fields = {"max_model_len", "load_format", "name", "mode"}
    name: Optional[str] = "native"
    mode: str = "async"
    temperature: float = 1.0
    top_k: int = -1
    top_p: float = 1.0
    do_sample: bool = True
    n: int = 1
    over_sample_rate: float = 0.0
    prompt_length: int = 512
    response_length: int = 512
    dtype: str = "bfloat16"
    gpu_memory_utilization: float = 0.5
    ignore_eos: bool = False
    enforce_eager: bool = False
    cudagraph_capture_sizes: Optional[list] = None
    free_cache_engine: bool = True
    data_parallel_size: int = 1
    expert_parallel_size: int = 1
    tensor_model_parallel_size: int = 2
    pipeline_model_parallel_size: int = 1
    max_num_batched_tokens: int = 8192
    val_kwargs: SamplingConfig = field(default_factory=lambda: SamplingConfig(temperature=0, do_sample=False))
    max_model_len: Optional[int] = None
    max_num_seqs: int = 256
    log_prob_micro_batch_size: Optional[int] = None
    log_prob_micro_batch_size_per_gpu: Optional[int] = None
    log_prob_use_dynamic_bsz: bool = False
    log_prob_max_token_len_per_gpu: int = 16384
    disable_log_stats: bool = True
    multi_stage_wake_up: bool = False
    engine_kwargs: dict = field(default_factory=dict)
    calculate_log_probs: bool = False
    agent: AgentLoopConfig = field(default_factory=AgentLoopConfig)
    trace: TraceConfig = field(default_factory=TraceConfig)
    multi_turn: MultiTurnConfig = field(default_factory=MultiTurnConfig)
    server: ServerConfig = field(default_factory=ServerConfig)
    prometheus: PrometheusConfig = field(default_factory=PrometheusConfig)
    checkpoint_engine: CheckpointEngineConfig = field(default_factory=CheckpointEngineConfig)
    enable_chunked_prefill: bool = True
    enable_prefix_caching: bool = True
    logprobs_mode: str = "processed_logprobs"
    scheduling_policy: str = "fcfs"
    load_format: str = "dummy"
    layered_summon: bool = False
    skip_rollout: bool = False
    skip_dump_dir: str = "/tmp/rollout_dump"
    skip_tokenizer_init: bool = True
    enable_rollout_routing_replay: bool = False
    profiler: Optional[ProfilerConfig] = None
    quantization: Optional[str] = None
    quantization_config_file: Optional[str] = None
    limit_images: Optional[int] = None

    def __post_init__(self):
        if self.expert_parallel_size > 1:
            assert self.expert_parallel_size == self.tensor_model_parallel_size * self.data_parallel_size, (
                "expert_parallel_size must be equal to tensor_model_parallel_size * data_parallel_size")


# ------------------------------------------------------------------------ reward model
@dataclass
class SandboxFusionConfig(BaseConfig):
    url: Optional[str] = None
    max_concurrent: int = 64
    memory_limit_mb: int = 1024


@dataclass
class RewardModelConfig(BaseConfig):
    _mutable_fields = {"max_num_seqs"}
    use_reward_loop: bool = True
    reward_manager: Optional[str] = "naive"
    enable: bool = False
    enable_resource_pool: bool = False
    n_gpus_per_node: int = 0
    nnodes: int = 0
    num_workers: int = 1
    model: Any = field(default_factory=dict)
    rollout: Any = field(default_factory=dict)
    micro_batch_size: Optional[int] = None
    micro_batch_size_per_gpu: Optional[int] = None
    max_length: Optional[int] = None
    use_dynamic_bsz: bool = False
    reward_loop_source: Optional[str] = "register"
    launch_reward_fn_async: bool = False
    sandbox_fusion: SandboxFusionConfig = field(default_factory=SandboxFusionConfig)
    profiler: ProfilerConfig = field(default_factory=ProfilerConfig)


@dataclass
class ModuleConfig(BaseConfig):
    path: Optional[str] = None
    name: Optional[str] = None


@dataclass
class RewardManagerConfig(BaseConfig):
    source: str = "register"
    name: str = "naive"
    module: Optional[ModuleConfig] = field(default_factory=ModuleConfig)
