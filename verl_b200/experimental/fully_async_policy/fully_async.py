"""Fully asynchronous RL: a rollouter streams samples into a queue, a trainer consumes them.

Role of verl/experimental/fully_async_policy/ (``FullyAsyncRollouter :45``, ``FullyAsyncTrainer :42``,
``MetricsAggregator`` in ``detach_utils.py:197``): generation never waits for training. The rollouter keeps
producing prompt groups with whatever weights the rollout engine currently holds and tags them with the
parameter version; the trainer takes ``required_samples`` groups per step, trains, and every
``trigger_parameter_sync_step`` steps hands the new weights to the synchroniser, which pauses the rollouter for
the copy. Staleness is bounded by the queue (``max_staleness`` versions; stale groups are dropped) and by
back-pressure (the rollouter stops when ``max_queue_size`` groups are waiting).
"""

from __future__ import annotations

import threading
import time
from collections import defaultdict
from typing import Optional

import numpy as np

from ...protocol import DataProto
from ...trainer.ppo.ray_trainer import RayPPOTrainer, _wait_all
from .message_queue import MessageQueue
from .param_sync import ParameterSynchronizer


class MetricsAggregator:
    """Combine the metric dicts of several trainer steps between two logging points: times and counts add up,
    everything else is averaged, ``*/max`` and ``*/min`` keep their extremum."""

    def __init__(self):
        self._vals: dict[str, list[float]] = defaultdict(list)

    def add_step_metrics(self, metrics: dict) -> None:
        for k, v in metrics.items():
            if isinstance(v, (int, float, np.floating, np.integer)):
                self._vals[k].append(float(v))

    @staticmethod
    def _rule(key: str) -> str:
        if key.startswith("timing_s/") or key.endswith("/count") or key.endswith("_count") or "total" in key.rsplit("/", 1)[-1]:
            return "sum"
        if key.endswith("/max") or key.endswith("_max"):
            return "max"
        if key.endswith("/min") or key.endswith("_min"):
            return "min"
        if key.endswith("global_step") or key.endswith("param_version"):
            return "last"
        return "mean"

    def get_aggregated_metrics(self) -> dict:
        out = {}
        for k, v in self._vals.items():
            r = self._rule(k)
            out[k] = {"sum": sum, "max": max, "min": min, "last": lambda x: x[-1], "mean": lambda x: sum(x) / len(x)}[r](v)
        return out

    def reset(self) -> None:
        self._vals.clear()


class FullyAsyncRollouter:
    """Producer thread: prompt batches -> rollout + reward -> one queue entry per prompt group."""

    def __init__(self, trainer: RayPPOTrainer, message_queue: MessageQueue, max_queue_size: Optional[int] = None,
                 total_rollout_steps: Optional[int] = None):
        self.trainer, self.mq = trainer, message_queue
        self.n = int(trainer.config.actor_rollout_ref.rollout.n)
        self.max_queue_size = int(max_queue_size or message_queue.max_queue_size)
        self.total_rollout_steps = total_rollout_steps
        self.param_version = 0
        self._run = threading.Event()
        self._run.set()
        self._idle = threading.Event()
        self._idle.set()
        self._stop = False
        self._thread: Optional[threading.Thread] = None
        self.produced_groups = 0
        self.error: Optional[BaseException] = None

    # -------------------------------------------------------------- control
    def start(self):
        self._thread = threading.Thread(target=self._loop, name="fully-async-rollouter", daemon=True)
        self._thread.start()

    def pause(self):
        """Stop taking new prompt batches and wait for the batch in flight (partial rollouts of an aborted batch would
        be re-queued here; the in-process engine finishes a batch in bounded time, so it is drained instead)."""
        self._run.clear()
        self._idle.wait()

    def resume(self):
        self._run.set()

    def update_param_version(self, v: int):
        self.param_version = int(v)

    def stop(self):
        self._stop = True
        self._run.set()
        self.mq.close()
        if self._thread is not None:
            self._thread.join(timeout=60)

    # ----------------------------------------------------------------- loop
    def _loop(self):
        try:
            steps = 0
            while not self._stop:
                for batch_dict in self.trainer.train_dataloader:
                    if self._stop or (self.total_rollout_steps is not None and steps >= self.total_rollout_steps):
                        return
                    self._run.wait()
                    if not self.mq.wait_below(self.max_queue_size, timeout=None):
                        return
                    self._idle.clear()
                    try:
                        version = self.param_version
                        batch = self.trainer._rollout_and_reward(batch_dict, {}, {})
                        for g in range(len(batch) // self.n):
                            self.mq.put_sample(batch[g * self.n : (g + 1) * self.n], version)
                            self.produced_groups += 1
                    finally:
                        self._idle.set()
                    steps += 1
                if self.total_rollout_steps is None:
                    return
        except BaseException as e:  # surface producer failures to the consumer
            self.error = e
            self.mq.close()


class StreamingRollouter(FullyAsyncRollouter):
    """Producer with partial rollouts: every prompt group runs as its own task through the fully-async agent-loop
    manager. ``pause()`` (a parameter update) aborts the generations in flight; the groups keep their partial
    outputs and continue after ``resume()`` under the new weights, so a weight sync never waits for the longest
    sample. A group's queue entry carries the oldest parameter version that produced any of its tokens.
    (verl/experimental/fully_async_policy/fully_async_rollouter.py: ``partial_rollout=True``.)"""

    def __init__(self, trainer: RayPPOTrainer, message_queue: MessageQueue, manager, max_queue_size: Optional[int] = None,
                 total_rollout_steps: Optional[int] = None, max_concurrent_groups: int = 64):
        super().__init__(trainer, message_queue, max_queue_size, total_rollout_steps)
        self.manager = manager
        self.max_concurrent_groups = int(max_concurrent_groups)
        self._loop_obj = None
        self._ready = threading.Event()
        self.cancelled_generations = 0

    def pause(self):
        self._run.clear()
        if self._thread is None:  # not started yet: nothing in flight
            return
        self._ready.wait(60)
        if self._loop_obj is not None and self._thread is not None and self._thread.is_alive():
            import asyncio

            asyncio.run_coroutine_threadsafe(self.manager.cancel(), self._loop_obj).result(timeout=600)

    def resume(self):
        if self._loop_obj is not None and self._thread is not None and self._thread.is_alive():
            import asyncio

            asyncio.run_coroutine_threadsafe(self.manager.resume(), self._loop_obj).result(timeout=600)
        self._run.set()

    def _loop(self):
        import asyncio

        try:
            asyncio.run(self._main())
        except BaseException as e:
            self.error = e
            self.mq.close()
        finally:
            self._ready.set()

    async def _main(self):
        import asyncio
        import uuid

        self._loop_obj = asyncio.get_running_loop()
        self._ready.set()
        tr, n = self.trainer, self.n
        sem = asyncio.Semaphore(self.max_concurrent_groups)
        tasks: set = set()
        steps = 0

        async def drive(group: DataProto):
            try:
                gen = tr._get_gen_batch(group)
                gen.meta_info.update({"pad_token_id": getattr(tr.tokenizer, "pad_token_id", 0) or 0,
                                      "eos_token_id": getattr(tr.tokenizer, "eos_token_id", None)})
                gen = gen.repeat(repeat_times=n, interleave=True)
                outs, cancelled = await self.manager.generate_single_sample_async(gen, None, self.param_version)
                while cancelled and not self._stop:
                    self.cancelled_generations += sum(bool(o.extra_fields.get("is_cancel")) for o in outs)
                    await self.manager.wait_resumed()
                    outs, cancelled = await self.manager.generate_single_sample_async(gen, outs, self.param_version)
                if self._stop:
                    return
                version = min(int(o.extra_fields.get("param_version_start", self.param_version)) for o in outs)
                gen_out = self.manager.postprocess(outs)
                gen_out.meta_info.pop("metrics", None)
                batch = tr._attach_rollout_and_reward(group.repeat(repeat_times=n, interleave=True), gen_out, {})
                await asyncio.get_running_loop().run_in_executor(None, self.mq.put_sample, batch, version)
                self.produced_groups += 1
            finally:
                sem.release()

        await asyncio.gather(*[h.wake_up() for h in self.manager.server_handles])  # the engines stay awake
        finished = False
        while not self._stop and not finished:
            for batch_dict in tr.train_dataloader:
                if self._stop or (self.total_rollout_steps is not None and steps >= self.total_rollout_steps):
                    finished = True
                    break
                batch = tr._local(DataProto.from_single_dict(batch_dict))
                batch.non_tensor_batch["uid"] = np.array([str(uuid.uuid4()) for _ in range(len(batch))], dtype=object)
                for g in range(len(batch)):
                    while not self._stop:  # back-pressure: room in the queue first, then a free slot
                        if await asyncio.get_running_loop().run_in_executor(
                                None, lambda: self.mq.wait_below(self.max_queue_size, timeout=0.5)):
                            break
                    if self._stop:
                        break
                    await sem.acquire()
                    t = asyncio.ensure_future(drive(batch[g : g + 1]))
                    tasks.add(t)
                    t.add_done_callback(tasks.discard)
                steps += 1
            if self.total_rollout_steps is None:
                finished = True  # one pass over the data
        if tasks:
            done, _ = await asyncio.wait(tasks)
            for t in done:
                if t.exception() is not None:
                    raise t.exception()


class FullyAsyncTrainer:
    """Consumer: ``required_samples`` prompt groups per training step, parameter sync every k steps."""

    def __init__(self, trainer: RayPPOTrainer, message_queue: MessageQueue, synchronizer: ParameterSynchronizer,
                 required_samples: int, trigger_parameter_sync_step: int = 1):
        self.trainer, self.mq, self.sync = trainer, message_queue, synchronizer
        self.required_samples = int(required_samples)
        self.trigger = max(1, int(trigger_parameter_sync_step))
        self.agg = MetricsAggregator()
        self.local_step = 0

    def fit_step(self, timeout: Optional[float] = None) -> Optional[dict]:
        samples = self.mq.get_samples(self.required_samples, timeout=timeout)
        if samples is None:
            return None
        tr = self.trainer
        batch = DataProto.concat([s.data for s in samples])
        versions = [s.param_version for s in samples]
        timing_raw, metrics = {}, {}
        tr.global_steps += 1
        t0 = time.perf_counter()
        tr._train_on_batch(batch, timing_raw, metrics)
        timing_raw["step"] = time.perf_counter() - t0
        metrics = tr._finish_step(timing_raw, metrics)
        cur = self.sync.get_current_param_version()
        metrics.update({"fully_async/staleness_mean": float(np.mean([cur - v for v in versions])),
                        "fully_async/staleness_max": float(max(cur - v for v in versions)),
                        "fully_async/queue_size": float(self.mq.get_queue_size()),
                        "fully_async/param_version": float(cur)})
        self.local_step += 1
        if self.local_step % self.trigger == 0:
            metrics.update(self.sync.sync_weights(cur + 1))
        self.agg.add_step_metrics(metrics)
        return metrics


def _push_weights(trainer: RayPPOTrainer):
    def sync(version: int):
        res = _wait_all(trainer.actor_rollout_wg.update_weights(version))
        return res if isinstance(res, dict) else {}

    return sync


def run_fully_async(trainer: RayPPOTrainer, total_train_steps: int, required_samples: Optional[int] = None,
                    max_queue_size: Optional[int] = None, max_staleness: Optional[int] = 3,
                    trigger_parameter_sync_step: int = 1, step_timeout: Optional[float] = 600.0,
                    partial_rollout: bool = False, max_concurrent_groups: int = 64) -> list[dict]:
    """Wire queue, rollouter, synchroniser and trainer around an initialised ``RayPPOTrainer`` and run
    ``total_train_steps`` trainer steps. Returns the per-step metrics. ``partial_rollout``: prompt groups stream
    through the agent-loop manager and generations cut by a parameter update are resumed (:class:`StreamingRollouter`)
    instead of whole batches being drained before every update."""
    groups_per_batch = int(trainer.config.data.train_batch_size) // max(1, trainer.spmd_world)
    required = int(required_samples or groups_per_batch)
    mq = MessageQueue(max_queue_size or 4 * required, max_staleness)
    if partial_rollout:
        from .agent_loop import FullyAsyncAgentLoopManager

        if not getattr(trainer, "async_rollout_mode", False):
            trainer._init_async_rollout_manager()
        manager = FullyAsyncAgentLoopManager(trainer.config, server_handles=trainer._rollout_server_handles,
                                             tokenizer=trainer.tokenizer, processor=trainer.processor)
        rollouter = StreamingRollouter(trainer, mq, manager, max_queue_size=max_queue_size or 4 * required,
                                       max_concurrent_groups=max_concurrent_groups)
        trainer.fully_async_rollouter = rollouter
    else:
        rollouter = FullyAsyncRollouter(trainer, mq, max_queue_size=max_queue_size or 4 * required)
    sync = ParameterSynchronizer(_push_weights(trainer), mq, rollouter)
    consumer = FullyAsyncTrainer(trainer, mq, sync, required, trigger_parameter_sync_step)
    sync.sync_weights(0)
    rollouter.start()
    out = []
    try:
        for _ in range(total_train_steps):
            m = consumer.fit_step(timeout=step_timeout)
            if m is None:
                if rollouter.error is not None:
                    raise rollouter.error
                break
            out.append(m)
    finally:
        rollouter.stop()
    return out
