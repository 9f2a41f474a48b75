"""``TrainingWorker``: a coarse-grained train / infer service around one engine, driven by a single controller
with TensorDict batches (verl/workers/engine_workers.py:53-322).

    worker.set_loss_fn(partial(sft_loss_on_batch, config))
    out = worker.train_mini_batch(batch)      # mini-batch loop for several epochs, one optimizer step per mini-batch
    out = worker.train_batch(batch)           # one optimizer step on the whole batch (micro-batched inside the engine)
    out = worker.infer_batch(batch)           # forward only: log-probs / entropy / values (+ loss when a loss fn is set)

Batches are in the no-padding layout (``input_ids`` jagged nested); the engine is chosen through the registry from
``config.engine_config.strategy`` (one native engine serves "fsdp", "fsdp2" and "native").
"""

from __future__ import annotations

import time
from contextlib import nullcontext
from typing import Optional

import torch
import torch.distributed as dist

from ..single_controller.base import Dispatch, Worker, register
from ..single_controller.base.decorator import make_nd_compute_dataproto_dispatch_fn
from ..utils import tensordict_utils as tu
from ..utils.flops_counter import FlopsCounter
from ..utils.py_functional import append_to_dict
from .engine.base import EngineRegistry
from .engine.native import _cfg

__all__ = ["TrainingWorker"]


class TrainingWorker(Worker):
    def __init__(self, config, device_name: Optional[str] = None):
        super().__init__()
        from .engine_workers import _init_dist, resolve_model_config

        self.config = config
        self.engine_config = _cfg(config, "engine_config", None)
        self.optimizer_config = _cfg(config, "optimizer_config", None)
        self.checkpoint_config = _cfg(config, "checkpoint_config", None)
        self.device_name = device_name or ("cuda" if torch.cuda.is_available() else "cpu")
        _init_dist(self.device_name)
        mc = _cfg(config, "model_config", None)
        state = None
        if not hasattr(mc, "num_hidden_layers"):  # an HF-style model section (path / override_config)
            mc, state = resolve_model_config(mc)
        self.model_config = mc
        model_type = _cfg(config, "model_type", None) or "language_model"
        backend = _cfg(self.engine_config, "strategy", "fsdp") or "fsdp"
        group = dist.group.WORLD if dist.is_initialized() and dist.get_world_size() > 1 else None
        device = f"cuda:{torch.cuda.current_device()}" if self.device_name == "cuda" else "cpu"
        cls = EngineRegistry.get_engine_cls(model_type, backend, self.device_name)
        self.engine = cls(mc, self.engine_config, self.optimizer_config, device=device, group=group, state_dict=state,
                          trainable=not bool(_cfg(self.engine_config, "forward_only", False)),
                          seed=int(_cfg(self.engine_config, "seed", 42) or 42))
        self._initialized = False
        rank = dist.get_rank() if dist.is_initialized() else 0
        sp = int(_cfg(self.engine_config, "ulysses_sequence_parallel_size", 1) or 1)
        self._register_dispatch_collect_info("train", dp_rank=rank // sp, is_collect=rank % sp == 0)
        self.flops_counter = FlopsCounter(mc)
        self.loss_fn = None

    # ------------------------------------------------------------------------------ control
    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def to(self, device, model=True, optimizer=True, grad=True):
        assert device in ("cpu", "device")
        self.engine.to(device=self.device_name if device == "device" else "cpu", model=model, optimizer=optimizer, grad=grad)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def set_loss_fn(self, loss_fn):
        self.loss_fn = loss_fn

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def reset(self):
        """Build (or rebuild) the engine's state: sharded weights, optimizer, schedules."""
        self.engine.initialize()
        self._initialized = True

    def _ensure(self):
        if not self._initialized:
            self.reset()

    # ------------------------------------------------------------------------------ results
    def _postprocess(self, output: dict, *, global_token_num, delta_time: float, forward_only: bool):
        metrics = dict(output.pop("metrics", {}))
        loss = torch.tensor([float(sum(output.pop("loss", []) or [0.0]))], dtype=torch.float64)
        grp = self.engine.get_data_parallel_group()
        if dist.is_initialized() and dist.get_world_size() > 1:
            dev = torch.device(self.engine.device)
            loss = loss.to(dev)
            # a rank's loss is its samples' part of the global mean: add the parts up (ranks of a tensor- / sequence-
            # parallel group report the same part)
            dist.all_reduce(loss, group=grp)
            loss = loss / max(int(getattr(self.engine, "_mp_inner", 1)), 1)
        grad_norm, lr = metrics.pop("grad_norm", None), metrics.pop("lr", None)
        final = {}
        if dist.is_initialized() and dist.get_world_size() > 1:
            gathered = [None] * dist.get_world_size(grp)
            dist.all_gather_object(gathered, metrics, group=grp)
            for m in gathered:
                for k, v in m.items():
                    final.setdefault(k, []).extend(v if isinstance(v, list) else [v])
        else:
            final = {k: (v if isinstance(v, list) else [v]) for k, v in metrics.items()}
        final["loss"] = float(loss.item())
        if grad_norm is not None:
            final["grad_norm"] = grad_norm
        if lr is not None:
            final["lr"] = lr
        if global_token_num is not None:
            est, promised = self.flops_counter.estimate_flops(list(global_token_num), max(delta_time, 1e-9))
            world = dist.get_world_size() if dist.is_initialized() else 1
            final["mfu"] = est / promised / world / (3.0 if forward_only else 1.0)
        model_output = {k: v.cpu() for k, v in (output.pop("model_output", {}) or {}).items()}
        return tu.get_tensordict(tensor_dict=model_output, non_tensor_dict={"metrics": final})

    def _defaults(self, data, infer: bool):
        pre = "infer_" if infer else ""
        for key, src in (("use_dynamic_bsz", "use_dynamic_bsz"), ("max_token_len_per_gpu", pre + "max_token_len_per_gpu"),
                         ("micro_batch_size_per_gpu", pre + "micro_batch_size_per_gpu")):
            if key not in data.keys():
                val = _cfg(self.engine_config, src, None)
                if val is not None:
                    tu.assign_non_tensor(data, **{key: val})

    # ------------------------------------------------------------------------------ training
    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("train"), blocking=False)
    def train_mini_batch(self, data):
        """Split this rank's batch into mini-batches (``mini_batch_size`` global samples, or ``num_mini_batch``
        pieces), run ``epochs`` passes with one optimizer step per mini-batch. Returns the per-step metrics."""
        self._ensure()
        tu.maybe_fix_3d_position_ids(data)
        per_dp = data.batch_size[0]
        mini = tu.pop(data, "mini_batch_size", None)
        num_mini = tu.pop(data, "num_mini_batch", None)
        epochs = int(tu.pop(data, "epochs", 1) or 1)
        seed = int(tu.pop(data, "seed", 42) or 42)
        dl_kwargs = tu.pop(data, "dataloader_kwargs", {}) or {}
        assert mini is not None or num_mini is not None, "pass mini_batch_size (global) or num_mini_batch"
        dp = self.engine.get_data_parallel_size()
        if mini is None:
            assert per_dp % num_mini == 0, f"Got batch_size_per_dp={per_dp} and num_mini_batch={num_mini}"
            per_gpu = per_dp // num_mini
        else:
            assert mini % dp == 0, f"Got mini_batch_size={mini} and data-parallel size {dp}"
            per_gpu = mini // dp
        loader = tu.make_iterator(data, mini_batch_size=per_gpu, epochs=epochs, seed=seed + self.engine.get_data_parallel_rank(),
                                  dataloader_kwargs=dl_kwargs)
        total = per_dp // per_gpu * epochs
        metrics: dict = {}
        for i, mb in enumerate(loader):
            tokens = mb["input_ids"].offsets().diff().tolist()
            if dist.is_initialized() and dist.get_world_size() > 1:
                parts = [None] * dist.get_world_size(self.engine.get_data_parallel_group())
                dist.all_gather_object(parts, tokens, group=self.engine.get_data_parallel_group())
                tokens = [t for p in parts for t in p]
            tu.assign_non_tensor(mb, global_token_num=tokens, update_lr_scheduler=i == total - 1)
            out = self._train_batch(mb)
            append_to_dict(metrics, tu.get(out, "metrics"))
        return tu.get_tensordict(tensor_dict={}, non_tensor_dict={"metrics": metrics})

    def _train_batch(self, data):
        assert self.loss_fn is not None, "loss function can't be None when calling train_batch"
        assert not bool(_cfg(self.engine_config, "forward_only", False)), "the engine was built forward-only"
        self._defaults(data, infer=False)
        tokens = tu.get(data, "global_token_num", None)
        t0 = time.perf_counter()
        with self.engine.train_mode():
            out = self.engine.train_batch(data, loss_function=self.loss_fn)
        dt = time.perf_counter() - t0
        if tu.get(data, "update_lr_scheduler", False):
            self.engine.lr_scheduler_step()
            out["metrics"]["lr"] = self.engine._lr()
        out.pop("model_output", None)
        return self._postprocess(out, global_token_num=tokens, delta_time=dt, forward_only=False)

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("train"), blocking=False)
    def train_batch(self, data):
        self._ensure()
        return self._train_batch(data)

    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("train"), blocking=False)
    def infer_batch(self, data):
        self._ensure()
        tokens = tu.get(data, "global_token_num", None)
        compute_loss = bool(tu.get(data, "compute_loss", True))
        no_adapter = bool(tu.pop(data, "no_lora_adapter", False))
        self._defaults(data, infer=True)
        loss_fn = self.loss_fn if compute_loss else None
        t0 = time.perf_counter()
        with self.engine.eval_mode():
            ctx = self.engine.disable_adapter() if no_adapter and hasattr(self.engine, "disable_adapter") else nullcontext()
            with ctx:
                out = self.engine.infer_batch(data, loss_function=loss_fn)
        return self._postprocess(out, global_token_num=tokens, delta_time=time.perf_counter() - t0, forward_only=True)

    # ------------------------------------------------------------------------------ checkpoints
    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def save_checkpoint(self, local_path, hdfs_path=None, global_step=0, max_ckpt_to_keep=None):
        self._ensure()
        return self.engine.save_checkpoint(local_path, hdfs_path, global_step, max_ckpt_to_keep)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def load_checkpoint(self, local_path, hdfs_path=None, del_local_after_load=False):
        self._ensure()
        return self.engine.load_checkpoint(local_path, hdfs_path, del_local_after_load)
