"""``import verl`` compatibility: every ``verl.x.y`` resolves to ``verl_b200.x.y`` (the same module objects, so
``verl.protocol.DataProto is verl_b200.protocol.DataProto``). Code written against the reference's import paths
(``from verl import DataProto``, ``from verl.trainer.ppo import core_algos``, ``verl.single_controller.base``...)
runs unchanged on this framework. Reference modules whose contents have another home here (one native engine
instead of per-backend workers, registries kept in their package ``__init__``) are redirected by ``_MOVED``.
"""

import importlib
import importlib.abc
import importlib.util
import sys
import types

import verl_b200 as _impl

_PREFIX, _TARGET = "verl.", "verl_b200."

# reference module paths whose contents live in a differently named module here
_MOVED = {
    "verl.workers.fsdp_workers": "verl_b200.workers.engine_workers",
    "verl.workers.reward_manager.abstract": "verl_b200.workers.reward_manager",
    "verl.workers.reward_manager.naive": "verl_b200.workers.reward_manager",
    "verl.workers.reward_manager.batch": "verl_b200.workers.reward_manager",
    "verl.workers.reward_manager.dapo": "verl_b200.workers.reward_manager",
    "verl.workers.reward_manager.prime": "verl_b200.workers.reward_manager",
    "verl.workers.reward_manager.registry": "verl_b200.workers.reward_manager",
    "verl.workers.config.actor": "verl_b200.workers.config",
    "verl.workers.config.critic": "verl_b200.workers.config",
    "verl.workers.config.engine": "verl_b200.workers.config",
    "verl.workers.config.model": "verl_b200.workers.config",
    "verl.workers.config.optimizer": "verl_b200.workers.config",
    "verl.workers.config.rollout": "verl_b200.workers.config",
    "verl.workers.config.reward_model": "verl_b200.workers.config",
    "verl.workers.rollout.hf_rollout": "verl_b200.workers.rollout.naive_rollout",
    "verl.workers.engine.fsdp": "verl_b200.workers.engine.native",
    "verl.workers.engine.fsdp.transformer_impl": "verl_b200.workers.engine.native",
    "verl.trainer.config.algorithm": "verl_b200.trainer.config",
    "verl.trainer.config.config": "verl_b200.trainer.config",
    "verl.trainer.fsdp_sft_trainer": "verl_b200.trainer.sft_trainer",
    "verl.trainer.sft_trainer_ray": "verl_b200.trainer.sft_trainer_ray",
    "verl.utils.dataset.multiturn_sft_dataset": "verl_b200.utils.dataset.sft_dataset",
    "verl.utils.dataset.rm_dataset": "verl_b200.utils.dataset.sft_dataset",
    "verl.utils.checkpoint.fsdp_checkpoint_manager": "verl_b200.utils.checkpoint.native_checkpoint",
    "verl.utils.debug.performance": "verl_b200.utils.profiler.performance",
    "verl.utils.profiler.nvtx_profile": "verl_b200.utils.profiler.profile",
    "verl.utils.profiler.torch_profile": "verl_b200.utils.profiler.profile",
    "verl.utils.kernel.linear_cross_entropy": "verl_b200.ops.lmhead",
    "verl.utils.kernel.kernels": "verl_b200.ops.lmhead",
    "verl.utils.kernel.fp8_kernel": "verl_b200.ops.fp8",
    "verl.utils.transferqueue_utils": "verl_b200.experimental.transfer_queue.queue",
    "verl.model_merger.base_model_merger": "verl_b200.model_merger.merger",
    "verl.model_merger.fsdp_model_merger": "verl_b200.model_merger.merger",
    "verl.checkpoint_engine.nccl_checkpoint_engine": "verl_b200.checkpoint_engine.base",
    "verl.experimental.fully_async_policy.fully_async_rollouter": "verl_b200.experimental.fully_async_policy.fully_async",
    "verl.experimental.fully_async_policy.fully_async_trainer": "verl_b200.experimental.fully_async_policy.fully_async",
    "verl.experimental.fully_async_policy.fully_async_main": "verl_b200.experimental.fully_async_policy.fully_async",
    "verl.experimental.fully_async_policy.detach_utils": "verl_b200.experimental.fully_async_policy.fully_async",
    "verl.experimental.reward_loop.reward_manager.naive": "verl_b200.experimental.reward_loop.reward_manager",
    "verl.experimental.reward_loop.reward_manager.dapo": "verl_b200.experimental.reward_loop.reward_manager",
    "verl.experimental.reward_loop.reward_manager.limited": "verl_b200.experimental.reward_loop.reward_manager",
    "verl.experimental.reward_loop.reward_manager.remote": "verl_b200.experimental.reward_loop.reward_manager",
    "verl.experimental.reward_loop.reward_manager.registry": "verl_b200.experimental.reward_loop.reward_manager",
    "verl.experimental.reward_loop.reward_manager.base": "verl_b200.experimental.reward_loop.reward_manager",
    "verl.tools.mcp_search_tool": "verl_b200.tools.mcp_base_tool",
    "verl.workers.sharding_manager.fsdp_ulysses": "verl_b200.workers.sharding_manager.fsdp_ulysses",
    "verl.tools.utils.mcp_clients.McpClientManager": "verl_b200.tools.mcp_base_tool",
    "verl.utils.dataset.rl_dataset": "verl_b200.utils.dataset.rl_dataset",
    # backends of the reference whose role the one native engine / rollout engine plays here
    "verl.workers.megatron_workers": "verl_b200.workers.engine_workers",
    "verl.workers.actor.megatron_actor": "verl_b200.workers.actor.dp_actor",
    "verl.workers.critic.megatron_critic": "verl_b200.workers.critic.dp_critic",
    "verl.workers.engine.fsdp.utils": "verl_b200.workers.engine.utils",
    "verl.workers.engine.megatron": "verl_b200.workers.engine.native",
    "verl.workers.engine.megatron.transformer_impl": "verl_b200.workers.engine.native",
    "verl.workers.engine.megatron.utils": "verl_b200.workers.engine.utils",
    "verl.workers.engine.veomni": "verl_b200.workers.engine.native",
    "verl.workers.engine.veomni.transformer_impl": "verl_b200.workers.engine.native",
    "verl.workers.engine.veomni.utils": "verl_b200.workers.engine.utils",
    "verl.workers.reward_model.megatron": "verl_b200.workers.reward_model",
    "verl.workers.reward_model.megatron.reward_model": "verl_b200.workers.reward_model.base",
    "verl.workers.rollout.naive": "verl_b200.workers.rollout.naive_rollout",
    "verl.workers.rollout.naive.naive_rollout": "verl_b200.workers.rollout.naive_rollout",
    "verl.workers.rollout.vllm_rollout": "verl_b200.workers.rollout.native_rollout",
    "verl.workers.rollout.vllm_rollout.vllm_rollout": "verl_b200.workers.rollout.native_rollout",
    "verl.workers.rollout.vllm_rollout.vllm_async_server": "verl_b200.workers.rollout.async_server",
    "verl.workers.rollout.vllm_rollout.utils": "verl_b200.workers.rollout.utils",
    "verl.workers.rollout.sglang_rollout": "verl_b200.workers.rollout.native_rollout",
    "verl.workers.rollout.sglang_rollout.sglang_rollout": "verl_b200.workers.rollout.native_rollout",
    "verl.workers.rollout.sglang_rollout.async_sglang_server": "verl_b200.workers.rollout.async_server",
    "verl.workers.rollout.sglang_rollout.http_server_engine": "verl_b200.workers.rollout.async_server",
    "verl.workers.rollout.sglang_rollout.utils": "verl_b200.workers.rollout.utils",
    "verl.workers.rollout.trtllm_rollout.trtllm_rollout": "verl_b200.workers.rollout.native_rollout",
    "verl.workers.rollout.trtllm_rollout.trtllm_async_server": "verl_b200.workers.rollout.async_server",
    "verl.utils.checkpoint.megatron_checkpoint_manager": "verl_b200.utils.checkpoint.native_checkpoint",
    "verl.utils.megatron.tensor_parallel": "verl_b200.parallel.vocab_parallel",
    "verl.utils.megatron.sequence_parallel": "verl_b200.parallel.vocab_parallel",
    "verl.utils.megatron.pipeline_parallel": "verl_b200.parallel.pipeline",
    "verl.utils.megatron.memory": "verl_b200.utils.memory_buffer",
    "verl.utils.metric.utils": "verl_b200.utils.metric",
    "verl.utils.transformers_compat": "verl_b200.utils.import_utils",
    "verl.utils.vllm.utils": "verl_b200.utils.import_utils",
    "verl.utils.vllm.vllm_fp8_utils": "verl_b200.ops.fp8",
    "verl.utils.sglang.sglang_fp8_utils": "verl_b200.ops.fp8",
    "verl.utils.experimental.torch_functional": "verl_b200.ops.lmhead",
    "verl.utils.profiler.empty_annotations": "verl_b200.utils.profiler.profile",
    "verl.utils.fsdp_utils": "verl_b200.parallel.zero",
    "verl.model_merger.megatron_model_merger": "verl_b200.model_merger.merger",
    "verl.models.weight_loader_registry": "verl_b200.models.registry",
    "verl.models.mcore.registry": "verl_b200.models.registry",
    "verl.models.mcore.weight_converter": "verl_b200.models.hf_io",
    "verl.models.mcore.loader": "verl_b200.models.hf_io",
    "verl.models.mcore.saver": "verl_b200.models.hf_io",
    "verl.models.mcore.config_converter": "verl_b200.models.config",
    "verl.models.mcore.model_initializer": "verl_b200.models.registry",
    "verl.models.mcore.model_forward": "verl_b200.models.transformer",
    "verl.models.mcore.model_forward_fused": "verl_b200.ops.lmhead",
    "verl.models.mcore.qwen2_5_vl": "verl_b200.models.vision",
    "verl.models.mcore.qwen2_5_vl.model": "verl_b200.models.vision",
    "verl.models.mcore.qwen2_5_vl.vision_model": "verl_b200.models.vision",
    "verl.models.mcore.qwen2_5_vl.rope_utils": "verl_b200.models.vision",
    "verl.models.transformers.tiled_mlp": "verl_b200.models.tiled_mlp",
    "verl.models.transformers.qwen2_vl": "verl_b200.models.vision",
    "verl.models.transformers.qwen3_vl": "verl_b200.models.vision",
    "verl.models.transformers.qwen2": "verl_b200.models.transformer",
    "verl.models.transformers.llama": "verl_b200.models.transformer",
    "verl.models.transformers.apertus": "verl_b200.models.transformer",
    "verl.models.transformers.dense_common": "verl_b200.ops.lmhead",
    "verl.models.transformers.monkey_patch": "verl_b200.trainer.ppo.prefix_grouper_utils",
    "verl.models.llama.megatron.modeling_llama_megatron": "verl_b200.models.transformer",
    "verl.models.llama.megatron.layers": "verl_b200.parallel.tensor_parallel",
    "verl.models.llama.megatron.checkpoint_utils": "verl_b200.models.hf_io",
    "verl.models.qwen2.megatron.modeling_qwen2_megatron": "verl_b200.models.transformer",
    "verl.models.qwen2.megatron.layers": "verl_b200.parallel.tensor_parallel",
    "verl.models.qwen2.megatron.checkpoint_utils": "verl_b200.models.hf_io",
    "verl.single_controller.ray.base": "verl_b200.single_controller.ray",
    "verl.checkpoint_engine.nixl_checkpoint_engine": "verl_b200.checkpoint_engine.base",
    "verl.experimental.fully_async_policy.checkpoint_engine": "verl_b200.checkpoint_engine.pinned_bucket",
    "verl.experimental.fully_async_policy.base_detach_sync": "verl_b200.experimental.fully_async_policy.param_sync",
    "verl.experimental.fully_async_policy.fsdp_workers": "verl_b200.experimental.fully_async_policy.param_sync",
    "verl.experimental.fully_async_policy.megatron_worker": "verl_b200.experimental.fully_async_policy.param_sync",
    "verl.experimental.fully_async_policy.ray_trainer": "verl_b200.experimental.fully_async_policy.fully_async",
    "verl.experimental.fully_async_policy.vllm_rollout": "verl_b200.workers.rollout.async_server",
    "verl.experimental.fully_async_policy.vllm_rollout.vllm_async_server": "verl_b200.workers.rollout.async_server",
    "verl.experimental.fully_async_policy.sglang_rollout": "verl_b200.workers.rollout.async_server",
    "verl.experimental.fully_async_policy.sglang_rollout.sglang_async_server": "verl_b200.workers.rollout.async_server",
    "verl.experimental.one_step_off_policy.main_ppo": "verl_b200.experimental.one_step_off_policy.ray_trainer",
    "verl.experimental.one_step_off_policy.fsdp_workers": "verl_b200.experimental.fully_async_policy.param_sync",
    "verl.experimental.one_step_off_policy.megatron_workers": "verl_b200.experimental.fully_async_policy.param_sync",
    "verl.experimental.one_step_off_policy.distributed_utils": "verl_b200.utils.distributed",
    "verl.experimental.one_step_off_policy.agent_loop": "verl_b200.experimental.agent_loop",
    "verl.experimental.one_step_off_policy.agent_loop.agent_loop": "verl_b200.experimental.agent_loop.agent_loop",
    "verl.experimental.transfer_queue.agent_loop": "verl_b200.experimental.agent_loop.agent_loop",
    "verl.experimental.transfer_queue.main_ppo": "verl_b200.trainer.main_ppo",
    "verl.experimental.transfer_queue.ray_trainer": "verl_b200.trainer.ppo.ray_trainer",
    "verl.experimental.vla.models.openvla_oft": "verl_b200.models.openvla_oft",
    "verl.experimental.vla.models.openvla_oft.modeling_prismatic": "verl_b200.models.openvla_oft",
    "verl.experimental.vla.models.openvla_oft.configuration_prismatic": "verl_b200.models.openvla_oft",
    "verl.experimental.vla.naive_rollout_rob": "verl_b200.experimental.vla.env_loop",
    "verl.experimental.vla.rob_ray_trainer": "verl_b200.experimental.vla.env_loop",
    "verl.experimental.vla.workers.env.env_worker": "verl_b200.experimental.vla.env_loop",
    "verl.experimental.vla.workers.env.env_manager": "verl_b200.experimental.vla.env_loop",
    "verl.utils.reward_score.prime_code.utils": "verl_b200.utils.reward_score.prime_code",
    "verl.utils.reward_score.prime_code.testing_util": "verl_b200.utils.reward_score.prime_code",
    "verl.utils.reward_score.prime_math.grader": "verl_b200.utils.reward_score.prime_math",
    "verl.utils.reward_score.prime_math.math_normalize": "verl_b200.utils.reward_score.prime_math",
    "verl.utils.reward_score.sandbox_fusion.utils": "verl_b200.utils.reward_score.sandbox_fusion",
    "verl.experimental.one_step_off_policy.utils": "verl_b200.trainer.ppo.utils",
    "verl.experimental.vla.dp_rob": "verl_b200.workers.actor.dp_actor",
    "verl.experimental.vla.fsdp_workers": "verl_b200.workers.engine_workers",
    "verl.utils.rendezvous": "verl_b200.utils.rendezvous",
    "verl.utils.rendezvous.ray_backend": "verl_b200.utils.rendezvous",
    "verl.utils.checkpoint.checkpoint_handler": "verl_b200.utils.checkpoint.checkpoint_handler",
}


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target: str, as_package: bool = False):
        self.target, self.as_package = target, as_package

    def create_module(self, spec):
        if self.target is None:  # a reference package that exists here only through its redirected sub-modules
            view = types.ModuleType(spec.name)
            view.__path__ = []
            return view
        real = importlib.import_module(self.target)
        if self.as_package and not hasattr(real, "__path__"):
            # a plain module here that the reference splits into sub-modules: a package-shaped view of its names
            view = types.ModuleType(spec.name, real.__doc__)
            view.__dict__.update({k: v for k, v in real.__dict__.items() if not k.startswith("__")})
            view.__path__ = []
            return view
        return real

    def exec_module(self, module):  # already executed under its real name
        pass


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_PREFIX):
            return None
        real = _MOVED.get(fullname) or _TARGET + fullname[len(_PREFIX):]
        has_moved_children = any(k.startswith(fullname + ".") for k in _MOVED)
        try:
            found = importlib.util.find_spec(real) is not None
        except (ImportError, ValueError):
            found = False
        if not found:
            if has_moved_children:
                return importlib.util.spec_from_loader(fullname, _AliasLoader(None, True), is_package=True)
            return None
        is_pkg = hasattr(importlib.import_module(real), "__path__") or has_moved_children
        return importlib.util.spec_from_loader(fullname, _AliasLoader(real, has_moved_children), is_package=is_pkg)


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())

# names the reference exports at the top level
DataProto = _impl.DataProto
__version__ = getattr(_impl, "__version__", "0.0.0")


def __getattr__(name):
    return getattr(_impl, name)
