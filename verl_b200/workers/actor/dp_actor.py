"""PPO actor on the native engine: ``compute_log_prob`` and ``update_policy``.

Semantics follow ``DataParallelPPOActor`` (verl/workers/actor/dp_actor.py:113-669): mini-batch /
micro-batch loops, dynamic batching by token budget, on-policy shortcut, policy-loss registry, KL and
entropy terms, one optimizer step per mini-batch, metric names ``actor/*``.

Loss normalisation is global: every micro-batch loss is divided by the token (or sequence) count of
the whole mini-batch summed over data-parallel ranks, and gradients are *summed* across ranks by the
engine's reduce-scatter, so the optimiser sees the gradient of the global mean regardless of how
tokens are spread over ranks and micro-batches.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ... import ops
from ...protocol import DataProto
from ...trainer.ppo import core_algos
from ...trainer.ppo.core_algos import agg_loss, get_policy_loss_fn, kl_penalty
from ...utils.py_functional import append_to_dict
from ...utils.seqlen_balancing import prepare_dynamic_batch, restore_dynamic_batch
from ..engine.native import NativeEngine, _cfg
from .base import BasePPOActor

__all__ = ["DataParallelPPOActor"]


class DataParallelPPOActor(BasePPOActor):
    def __init__(self, config, engine: NativeEngine):
        self.config = config
        self.engine = engine
        self.device = engine.device
        self.use_fused_loss = self.device.type == "cuda"
        # forward-only passes evaluate every distinct prompt of a micro-batch once (trainer/ppo/prefix_grouper_utils.py)
        self.use_prefix_grouper = bool(_cfg(config, "use_prefix_grouper", False))
        self.last_prefix_saving = 0.0
        # router replay for mixture-of-experts models (verl/utils/megatron/router_replay_patch.py): "R2" records the
        # experts every token was routed to during compute_log_prob and routes the same way in the update, so the old
        # and the new log-probs of a token come from the same experts; "R3" takes the record from the rollout
        # (``routed_experts`` in the batch) and replays it in compute_log_prob and in the update
        self.router_replay = str(_cfg(_cfg(config, "router_replay", None), "mode", "disabled") or "disabled")
        self.last_routed_experts = None
        self.record_routing = True  # a reference policy built on this class switches it off: nothing reads its record
        # optimal-token-baseline estimators: compute_log_prob also returns sum_v pi(v)^2 per response token
        self.calculate_sum_pi_squared = bool(_cfg(config, "calculate_sum_pi_squared", False))
        self._want_spp, self._spp, self.last_sum_pi_squared = False, [], None
        if self.router_replay != "disabled":
            if not getattr(engine.model_config, "is_moe", False):
                raise ValueError("actor.router_replay needs a mixture-of-experts model")
            if getattr(engine, "sp_size", 1) > 1 or getattr(engine, "cp_size", 1) > 1 or getattr(engine, "pp_size", 1) > 1:
                raise NotImplementedError("actor.router_replay with sequence, context or pipeline parallelism")
            self.use_prefix_grouper = False  # the record is laid out by the plain packing of a micro-batch

    # ------------------------------------------------------------------ forward
    def _forward_micro_batch(self, micro: DataProto, temperature: float, calculate_entropy: bool):
        """Returns (log_probs [b,R], entropy [b,R]) for the response part of a micro-batch."""
        b = micro.batch
        input_ids = b["input_ids"].to(self.device)
        mask = b["attention_mask"].to(self.device)
        pos = b["position_ids"].to(self.device) if "position_ids" in b else None
        vl = bool(getattr(self.engine.model_config, "is_vl", False))
        if pos is not None and pos.dim() == 3:
            # mrope layouts carry [b, 3, S] or [b, 4, S] (row 0 = text positions, rows 1..3 = temporal / height / width)
            pos = pos[:, -3:] if vl else pos[:, 0]
        R = b["responses"].shape[-1]
        e = self.engine
        if (self.use_prefix_grouper and not torch.is_grad_enabled() and not vl
                and getattr(e, "sp_size", 1) <= 1 and getattr(e, "cp_size", 1) <= 1 and getattr(e, "pp_size", 1) <= 1):
            # forward-only evaluation: every distinct prompt of the micro-batch is evaluated once, its n responses
            # attend to its keys (update_policy keeps the plain layout: the backward kernels have no such form)
            from ...trainer.ppo.prefix_grouper_utils import shared_prefix_batch

            packed, rows, labels, bj, saving = shared_prefix_batch(input_ids, mask, R)
            self.last_prefix_saving = saving
        else:
            packed, rows, labels, bj = NativeEngine.response_rows(input_ids, mask, R, pos)
        mm = micro.non_tensor_batch.get("multi_modal_inputs") if vl else None
        if mm is not None:
            from ...utils.model import extract_multi_modal_inputs

            inputs = extract_multi_modal_inputs(list(mm))
            if inputs.get("pixel_values") is not None:
                packed.pixel_values = inputs["pixel_values"].to(self.device)
                packed.image_grid_thw = inputs["image_grid_thw"].to(self.device)
            if inputs.get("pixel_values_videos") is not None:
                packed.pixel_values_videos = inputs["pixel_values_videos"].to(self.device)
                packed.video_grid_thw = inputs["video_grid_thw"].to(self.device)
        replay = record = False
        if self.router_replay != "disabled":
            flat = torch.nonzero(mask.reshape(-1).bool(), as_tuple=True)[0]  # packed token t sits at (b, s) = flat[t]
            moe = [layer.mlp for layer in self.engine.model.layers]
            if "routed_experts" in b.keys():
                # [b, S, layers, top-k] -> per layer the [T, top-k] ids of the packed tokens; stays set through the
                # backward (recomputed layers must route the same way) until update_policy clears it
                rec = b["routed_experts"].to(self.device).reshape(-1, *b["routed_experts"].shape[2:])[flat].long()
                for li, m in enumerate(moe):
                    m.replay_routing = rec[:, li].contiguous()
                replay = True
            elif self.router_replay == "R2" and self.record_routing and not torch.is_grad_enabled():
                record = True
        want_spp = self._want_spp and not torch.is_grad_enabled()
        if want_spp:
            lp, ent, spp = self.engine.forward_logprob(packed, rows, labels, temperature, sum_pi_squared=True)
        else:
            lp, ent = self.engine.forward_logprob(packed, rows, labels, temperature)
        B = input_ids.shape[0]
        if want_spp:
            self._spp.append(torch.zeros(B, R, dtype=torch.float32, device=self.device).index_put((bj[:, 0], bj[:, 1]), spp))
        if record:
            S = input_ids.shape[1]
            rec = torch.stack([m.last_routing for m in moe], dim=1)  # [T, layers, top-k]
            full = torch.zeros(B * S, *rec.shape[1:], dtype=torch.int16, device=self.device)
            full[flat] = rec.to(torch.int16)
            self._recorded.append(full.view(B, S, *rec.shape[1:]).cpu())
        if replay and not torch.is_grad_enabled():
            self._clear_replay()
        log_probs = torch.zeros(B, R, dtype=torch.float32, device=self.device)
        entropy = torch.zeros(B, R, dtype=torch.float32, device=self.device)
        log_probs = log_probs.index_put((bj[:, 0], bj[:, 1]), lp)
        if calculate_entropy:
            entropy = entropy.index_put((bj[:, 0], bj[:, 1]), ent)
        return log_probs, (entropy if calculate_entropy else None)

    def _clear_replay(self):
        for layer in self.engine.model.layers:
            if hasattr(layer.mlp, "replay_routing"):
                layer.mlp.replay_routing = None

    def _micro_batches_by_group(self, data: DataProto, max_token_len: int):
        """Token-budget micro-batches for the shared-prefix layout: the samples of one prompt stay together (a group
        counts its prompt once), groups are spread over the micro-batches largest first onto the least loaded one, and
        every rank makes the same number of micro-batches. Returns None when there are fewer groups than micro-batches."""
        b = data.batch
        R = b["responses"].shape[-1]
        ids, mask = b["input_ids"], b["attention_mask"]
        P = ids.shape[1] - R
        groups: dict = {}
        for i in range(ids.shape[0]):
            groups.setdefault(ids[i, :P][mask[i, :P].bool()].cpu().numpy().tobytes(), []).append(i)
        rows = list(groups.values())
        cost = [int(mask[r[0], :P].sum()) + int(mask[r, P:].sum()) for r in rows]
        k = max(1, -(-sum(cost) // max(int(max_token_len), 1)))
        if self.engine.world > 1:
            t = torch.tensor([k, -len(rows)], dtype=torch.int64, device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.engine.group)
            k, min_groups = int(t[0]), -int(t[1])
        else:
            min_groups = len(rows)
        if min_groups < k:
            return None
        bins: list[list[int]] = [[] for _ in range(k)]
        load = [0] * k
        for g in sorted(range(len(rows)), key=lambda g: -cost[g]):
            j = min(range(k), key=lambda j: load[j])
            bins[j] += rows[g]
            load[j] += cost[g]
        out = []
        for idx in bins:
            sel = torch.tensor(idx, dtype=torch.long)
            nt = {key: v[idx] for key, v in data.non_tensor_batch.items()}
            out.append(DataProto(batch=b[sel], non_tensor_batch=nt, meta_info=data.meta_info))
        return out, bins

    def _micro_batches(self, data: DataProto, max_token_len: Optional[int], micro_bsz: Optional[int], use_dyn: bool):
        if use_dyn and self.use_prefix_grouper and not torch.is_grad_enabled() and max_token_len:
            grouped = self._micro_batches_by_group(data, int(max_token_len))
            if grouped is not None:
                return grouped
        if use_dyn:
            return prepare_dynamic_batch(data, max_token_len=max_token_len, dp_group=self.engine.group
                                         if self.engine.world > 1 else None)
        return data.split(micro_bsz or len(data)), None

    # -------------------------------------------------------------- log-prob only
    @torch.no_grad()
    def compute_log_prob(self, data: DataProto, calculate_entropy: bool = False):
        """data.batch: responses, input_ids, attention_mask, position_ids; meta: temperature,
        micro_batch_size | (max_token_len, use_dynamic_bsz). Returns (log_probs [B,R], entropys | None)."""
        temperature = data.meta_info["temperature"]
        use_dyn = data.meta_info.get("use_dynamic_bsz", False)
        keys = ["responses", "input_ids", "attention_mask", "position_ids"]
        if self.router_replay == "R3":
            keys.append("routed_experts")  # recorded by the rollout
        sel = data.select(batch_keys=[k for k in keys if k in data.batch.keys()])
        micros, idx = self._micro_batches(sel, data.meta_info.get("max_token_len"),
                                          data.meta_info.get("micro_batch_size"), use_dyn)
        lps, ents = [], []
        self._recorded, self.last_routed_experts = [], None
        self._want_spp, self._spp, self.last_sum_pi_squared = self.calculate_sum_pi_squared and self.record_routing, [], None
        if self._want_spp and self.use_prefix_grouper:
            raise NotImplementedError("calculate_sum_pi_squared with use_prefix_grouper")
        for mb in micros:
            lp, ent = self._forward_micro_batch(mb, temperature, calculate_entropy)
            lps.append(lp)
            if calculate_entropy:
                ents.append(ent)
        log_probs = torch.cat(lps, dim=0)
        entropys = torch.cat(ents, dim=0) if calculate_entropy else None
        if use_dyn:
            log_probs = restore_dynamic_batch(log_probs, idx)
            if calculate_entropy:
                entropys = restore_dynamic_batch(entropys, idx)
        if self._spp:
            spp = torch.cat(self._spp, dim=0)
            self.last_sum_pi_squared = restore_dynamic_batch(spp, idx) if use_dyn else spp
        self._want_spp, self._spp = False, []
        if self._recorded:
            rec = torch.cat(self._recorded, dim=0)
            self.last_routed_experts = restore_dynamic_batch(rec, idx) if use_dyn else rec
            self._recorded = []
        return log_probs, entropys

    # -------------------------------------------------------------------- update
    def _global_counts(self, mini: DataProto):
        mask = mini.batch["response_mask"]
        t = torch.tensor([float(mask.sum()), float((mask.sum(-1) > 0).sum())], dtype=torch.float64, device=self.device)
        if self.engine.world > 1:
            dist.all_reduce(t, group=self.engine.group)
            # the ranks of a sequence- / tensor-parallel group hold the same samples: count each sample once
            t = t / max(int(getattr(self.engine, "mp_size", 1) or 1), 1)
        return max(t[0].item(), 1.0), max(t[1].item(), 1.0)

    def update_policy(self, data: DataProto) -> dict:
        cfg = self.config
        temperature = data.meta_info["temperature"]
        keys = ["responses", "response_mask", "input_ids", "attention_mask", "position_ids", "old_log_probs", "advantages"]
        for opt_key in ("ref_log_prob", "rollout_is_weights", "rollout_log_probs"):
            if opt_key in data.batch.keys():
                keys.append(opt_key)
        if self.router_replay != "disabled":
            assert "routed_experts" in data.batch.keys(), \
                "actor.router_replay: the batch has no routed_experts (R2: from compute_log_prob, R3: from the rollout)"
            keys.append("routed_experts")
        keys = [k for k in keys if k in data.batch.keys()]
        data = data.select(batch_keys=keys)
        mini_bsz = min(int(cfg.ppo_mini_batch_size), len(data))
        mini_batches = data.split(mini_bsz)
        shuffle = bool(_cfg(cfg, "shuffle", False))
        self._epochs_done = getattr(self, "_epochs_done", 0)
        on_policy = len(mini_batches) == 1 and cfg.ppo_epochs == 1
        loss_mode = _cfg(cfg.policy_loss, "loss_mode", "vanilla")
        entropy_coeff = float(cfg.entropy_coeff)
        calc_entropy = entropy_coeff != 0 or bool(_cfg(cfg, "calculate_entropy", False))
        use_kl = bool(cfg.use_kl_loss)
        metrics: dict = {}
        engine = self.engine
        for _ in range(cfg.ppo_epochs):
            if shuffle:
                # actor.shuffle: a fresh order of this rank's samples every epoch, reproducible from
                # actor.data_loader_seed (the same on every rank: ranks of a model-parallel group hold the same samples)
                g = torch.Generator().manual_seed(int(_cfg(cfg, "data_loader_seed", 42) or 42) + self._epochs_done)
                mini_batches = data.select_idxs(torch.randperm(len(data), generator=g)).split(mini_bsz)
            self._epochs_done += 1
            for mini in mini_batches:
                n_tok, n_seq = self._global_counts(mini)
                micros, _ = self._micro_batches(mini, int(cfg.ppo_max_token_len_per_gpu),
                                                cfg.ppo_micro_batch_size_per_gpu, bool(cfg.use_dynamic_bsz))
                engine.optimizer_zero_grad()
                acc = {"actor/pg_loss": 0.0, "actor/kl_loss": 0.0}
                for mb in micros:
                    b = mb.batch
                    mask = b["response_mask"].to(self.device).float()
                    adv = b["advantages"].to(self.device)
                    log_prob, entropy = self._forward_micro_batch(mb, temperature, calc_entropy)
                    old = log_prob.detach() if on_policy else b["old_log_probs"].to(self.device)
                    ref = b["ref_log_prob"].to(self.device) if use_kl else None
                    isw = b["rollout_is_weights"].to(self.device) if "rollout_is_weights" in b else None
                    # the fused kernel differentiates every KL estimator itself; the "+" variants (estimator's value,
                    # gradient of k2: core_algos.kl_penalty) take the composed path
                    kl_plus = use_kl and str(cfg.kl_loss_type).endswith("+")
                    fused_ok = (self.use_fused_loss and loss_mode == "vanilla" and cfg.loss_agg_mode == "token-mean"
                                and not kl_plus)
                    if fused_ok:
                        loss, sums = ops.ppo_loss_fused(
                            log_prob, old, adv, mask, entropy=entropy, ref_logp=ref, is_weight=isw,
                            clip_low=_cfg(cfg, "clip_ratio_low", cfg.clip_ratio), clip_high=_cfg(cfg, "clip_ratio_high", cfg.clip_ratio),
                            clip_c=_cfg(cfg, "clip_ratio_c", 3.0), kl_coef=float(cfg.kl_loss_coef) if use_kl else 0.0,
                            kl_type=cfg.kl_loss_type, entropy_coeff=entropy_coeff, denom=n_tok)
                        loss.backward()
                        s = sums.tolist()
                        n_local = max(s[6], 1.0)
                        acc["actor/pg_loss"] += s[0] / n_tok
                        if use_kl:
                            acc["actor/kl_loss"] += s[4] / n_tok
                        mb_metrics = {"actor/pg_clipfrac": s[1] / n_local, "actor/ppo_kl": s[2] / n_local,
                                      "actor/pg_clipfrac_lower": s[3] / n_local}
                        if calc_entropy:
                            mb_metrics["actor/entropy"] = s[5] / n_local
                    else:
                        info = {"dp_size": 1, "batch_num_tokens": n_tok, "global_batch_size": n_seq,
                                "loss_scale_factor": _cfg(cfg, "loss_scale_factor", None)}
                        object.__setattr__(cfg, "global_batch_info", info) if not isinstance(cfg, dict) else cfg.update(
                            global_batch_info=info)
                        fn = get_policy_loss_fn(loss_mode)
                        pg_loss, mb_metrics = fn(old_log_prob=old, log_prob=log_prob, advantages=adv, response_mask=mask,
                                                 loss_agg_mode=cfg.loss_agg_mode, config=cfg, rollout_is_weights=isw)
                        loss = pg_loss
                        acc["actor/pg_loss"] += pg_loss.detach().item()
                        if calc_entropy:
                            ent_agg = agg_loss(entropy, mask, cfg.loss_agg_mode, **info)
                            mb_metrics["actor/entropy"] = (entropy.detach() * mask).sum().item() / max(mask.sum().item(), 1.0)
                            if entropy_coeff != 0:
                                loss = loss - entropy_coeff * ent_agg
                        if use_kl:
                            kld = kl_penalty(log_prob, ref, cfg.kl_loss_type)
                            kl_loss = agg_loss(kld, mask, cfg.loss_agg_mode, **info)
                            loss = loss + float(cfg.kl_loss_coef) * kl_loss
                            acc["actor/kl_loss"] += kl_loss.detach().item()
                            mb_metrics["actor/kl_coef"] = float(cfg.kl_loss_coef)
                        loss.backward()
                    if self.router_replay != "disabled":
                        self._clear_replay()
                    append_to_dict(metrics, mb_metrics)
                grad_norm = engine.optimizer_step()
                mini_metrics = {"actor/grad_norm": float(grad_norm), "actor/pg_loss": acc["actor/pg_loss"]}
                if use_kl:
                    mini_metrics["actor/kl_loss"] = acc["actor/kl_loss"]
                append_to_dict(metrics, mini_metrics)
        return metrics
