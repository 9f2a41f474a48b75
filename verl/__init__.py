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
    "verl.trainer.sft_trainer_ray": "verl_b200.trainer.sft_trainer",
    "verl.utils.dataset.multiturn_sft_dataset": "verl_b200.utils.dataset.sft_dataset",
    "verl.utils.dataset.rm_dataset": "verl_b200.utils.dataset.sft_dataset",
    "verl.utils.checkpoint.fsdp_checkpoint_manager": "verl_b200.utils.checkpoint.native_checkpoint",
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
