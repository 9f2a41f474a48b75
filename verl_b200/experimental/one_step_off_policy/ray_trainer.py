"""One-step-off-policy trainer: the rollout of step t+1 runs while step t trains.

Role of verl/experimental/one_step_off_policy/ray_trainer.py:57 (``OneStepOffRayTrainer``) and
``fsdp_workers.py:68-117`` (``sync_rollout_weights``): generation for the next batch is launched before the
current batch is trained on, so its samples come from the weights of one update ago; the weights are pushed to
the rollout engine after every update, between two generations.

The generation runs on a worker thread with its own CUDA stream; on a box where rollout and training own
different GPUs (two resource pools) the two phases overlap fully, on shared GPUs they interleave. The policy
loss should be told about the staleness through the rollout-correction options (``algorithm.rollout_correction``),
exactly as in the reference.
"""

from __future__ import annotations

import concurrent.futures as cf
from typing import Optional

import torch

from ...trainer.ppo.ray_trainer import RayPPOTrainer, _wait_all, marked_timer
from ...utils.tracking import Tracking


class OneStepOffRayTrainer(RayPPOTrainer):
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._gen_pool = cf.ThreadPoolExecutor(max_workers=1, thread_name_prefix="rollout")
        self._gen_stream = None

    def _generate_async(self, batch_dict: dict) -> cf.Future:
        def run():
            timing, metrics = {}, {}
            if torch.cuda.is_available() and self.device_name == "cuda":
                if self._gen_stream is None:
                    self._gen_stream = torch.cuda.Stream()
                with torch.cuda.stream(self._gen_stream):
                    batch = self._rollout_and_reward(batch_dict, timing, metrics)
                self._gen_stream.synchronize()
            else:
                batch = self._rollout_and_reward(batch_dict, timing, metrics)
            return batch, timing, metrics

        return self._gen_pool.submit(run)

    def fit(self):
        cfg = self.config
        logger = Tracking(cfg.trainer.project_name, cfg.trainer.experiment_name, list(cfg.trainer.logger),
                          config=None) if self.rank == 0 else None
        self.global_steps = 0
        self._load_checkpoint()
        _wait_all(self.actor_rollout_wg.update_weights(self.global_steps))
        last: dict = {}
        it = iter(self._epoch_iterator())
        try:
            pending: Optional[cf.Future] = self._generate_async(next(it))
        except StopIteration:
            return last
        while pending is not None:
            batch, timing_raw, metrics = pending.result()
            # launch the next rollout now: it samples from the weights that are in the rollout engine at this moment,
            # i.e. the weights before the update below (one step off)
            try:
                nxt = next(it)
                pending = self._generate_async(nxt) if self.global_steps + 1 < self.total_training_steps else None
            except StopIteration:
                pending = None
            self.global_steps += 1
            with marked_timer("step", timing_raw):
                self._train_on_batch(batch, timing_raw, metrics)
            metrics = self._finish_step(timing_raw, metrics)
            metrics["training/staleness"] = 1.0 if self.global_steps > 1 else 0.0
            is_last = self.global_steps >= self.total_training_steps or pending is None
            if self.val_reward_fn is not None and cfg.trainer.test_freq > 0 and (is_last or self.global_steps % cfg.trainer.test_freq == 0):
                metrics.update(self._validate())
            if cfg.trainer.save_freq > 0 and (is_last or self.global_steps % cfg.trainer.save_freq == 0):
                self._save_checkpoint()
            if logger is not None:
                logger.log(metrics, step=self.global_steps)
            last = metrics
            if is_last:
                break
        if pending is not None:
            pending.cancel()
        self._gen_pool.shutdown(wait=True)
        return last

    def _epoch_iterator(self):
        for _ in range(int(self.config.trainer.total_epochs)):
            for batch_dict in self.train_dataloader:
                yield batch_dict
