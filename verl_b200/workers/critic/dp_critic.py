"""PPO critic on the native engine (value head = Linear(hidden, 1) on the final norm).

Semantics of ``DataParallelPPOCritic`` (verl/workers/critic/dp_critic.py:53-263): values are read at the
positions that predict response tokens (``[:, -R-1:-1]`` of the padded layout), multiplied by the response
mask; the clipped value loss and the metrics ``critic/vf_loss, vf_clipfrac, vpred_mean, grad_norm``.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ...protocol import DataProto
from ...trainer.ppo import core_algos
from ...utils.py_functional import append_to_dict
from ...utils.seqlen_balancing import prepare_dynamic_batch, restore_dynamic_batch
from ...utils.torch_functional import masked_mean
from ..engine.native import NativeEngine, _cfg
from .base import BasePPOCritic

__all__ = ["DataParallelPPOCritic"]


class DataParallelPPOCritic(BasePPOCritic):
    def __init__(self, config, engine: NativeEngine):
        self.config, self.engine, self.device = config, engine, engine.device

    def _forward_micro_batch(self, micro: DataProto) -> torch.Tensor:
        b = micro.batch
        input_ids, mask = b["input_ids"].to(self.device), b["attention_mask"].to(self.device)
        pos = b["position_ids"].to(self.device) if "position_ids" in b else None
        if pos is not None and pos.dim() == 3:
            pos = pos[:, 0]
        R = b["responses"].shape[-1]
        packed, rows, _labels, bj = NativeEngine.response_rows(input_ids, mask, R, pos)
        v = self.engine.forward_values(packed, rows)
        out = torch.zeros(input_ids.shape[0], R, dtype=torch.float32, device=self.device)
        return out.index_put((bj[:, 0], bj[:, 1]), v)

    def _micro_batches(self, data, max_token_len, micro_bsz, use_dyn):
        if use_dyn:
            return prepare_dynamic_batch(data, max_token_len=max_token_len,
                                         dp_group=self.engine.group if self.engine.world > 1 else None)
        return data.split(micro_bsz or len(data)), None

    @torch.no_grad()
    def compute_values(self, data: DataProto) -> torch.Tensor:
        use_dyn = data.meta_info.get("use_dynamic_bsz", False)
        keys = [k for k in ("responses", "input_ids", "response_mask", "attention_mask", "position_ids") if k in data.batch.keys()]
        sel = data.select(batch_keys=keys)
        micros, idx = self._micro_batches(sel, data.meta_info.get("max_token_len"), data.meta_info.get("micro_batch_size"), use_dyn)
        values = torch.cat([self._forward_micro_batch(mb) for mb in micros], dim=0)
        if use_dyn:
            values = restore_dynamic_batch(values, idx)
        if "response_mask" in data.batch.keys():
            values = values * data.batch["response_mask"].to(values.device)
        return values

    def update_critic(self, data: DataProto) -> dict:
        cfg = self.config
        keys = [k for k in ("input_ids", "responses", "response_mask", "attention_mask", "position_ids", "values", "returns")
                if k in data.batch.keys()]
        data = data.select(batch_keys=keys)
        mini_bsz = min(int(cfg.ppo_mini_batch_size), len(data))
        mini_batches = data.split(mini_bsz)
        metrics: dict = {}
        eng = self.engine
        self._epochs_done = getattr(self, "_epochs_done", 0)
        for _ in range(cfg.ppo_epochs):
            if bool(_cfg(cfg, "shuffle", False)):  # critic.shuffle / critic.data_loader_seed, as in the actor
                g = torch.Generator().manual_seed(int(_cfg(cfg, "data_loader_seed", 42) or 42) + self._epochs_done)
                mini_batches = data.select_idxs(torch.randperm(len(data), generator=g)).split(mini_bsz)
            self._epochs_done += 1
            for mini in mini_batches:
                n_tok = torch.tensor([float(mini.batch["response_mask"].sum())], dtype=torch.float64, device=self.device)
                if eng.world > 1:
                    dist.all_reduce(n_tok, group=eng.group)
                    n_tok = n_tok / max(int(getattr(eng, "mp_size", 1) or 1), 1)  # an SP group shares its samples
                n_tok = max(n_tok.item(), 1.0)
                micros, _ = self._micro_batches(mini, int(cfg.ppo_max_token_len_per_gpu), cfg.ppo_micro_batch_size_per_gpu,
                                                bool(cfg.use_dynamic_bsz))
                eng.optimizer_zero_grad()
                for mb in micros:
                    b = mb.batch
                    mask = b["response_mask"].to(self.device).float()
                    vpreds = self._forward_micro_batch(mb)
                    old_v, ret = b["values"].to(self.device), b["returns"].to(self.device)
                    vclip = torch.max(torch.min(vpreds, old_v + cfg.cliprange_value), old_v - cfg.cliprange_value)
                    l1, l2 = (vpreds - ret) ** 2, (vclip - ret) ** 2
                    vf_loss = 0.5 * core_algos.agg_loss(torch.max(l1, l2), mask, cfg.loss_agg_mode, batch_num_tokens=n_tok)
                    vf_loss.backward()
                    append_to_dict(metrics, {
                        "critic/vf_loss": vf_loss.detach().item() * n_tok / max(mask.sum().item(), 1.0),
                        "critic/vf_clipfrac": masked_mean(torch.gt(l2, l1).float(), mask).item(),
                        "critic/vpred_mean": masked_mean(vpreds.detach(), mask).item()})
                append_to_dict(metrics, {"critic/grad_norm": float(eng.optimizer_step())})
        return metrics
