"""Trainer-side adapter to the native rollout engine (role of ``ServerAdapter`` in
verl/workers/rollout/vllm_rollout/vllm_rollout.py:62-232).

The reference ships weights to a separate vLLM process through CUDA-IPC buckets and a ZMQ handshake. Here the
engine lives in the trainer's process on the same GPU, so ``update_weights`` writes straight into the engine's
parameters (or does nothing when they alias the trainer's tensors)."""

from __future__ import annotations

from typing import Generator, Optional

import torch

from ...rollout import NativeRolloutEngine
from .base import BaseRollout


class ServerAdapter(BaseRollout):
    def __init__(self, config, model_config, device_mesh=None, engine: Optional[NativeRolloutEngine] = None):
        super().__init__(config, model_config, device_mesh)
        self.engine = engine

    def attach(self, engine: NativeRolloutEngine):
        self.engine = engine

    async def resume(self, tags: list[str]):
        self.engine.wake_up(tags)

    async def release(self):
        self.engine.sleep()

    async def update_weights(self, weights: Generator[tuple[str, torch.Tensor], None, None], peft_config=None,
                             base_sync_done: bool = False, **kwargs):
        self.engine.update_weights(weights)

    def generate_sequences(self, prompts):
        """Batch generation on the attached engine: ``prompts.batch`` holds left-padded ``input_ids`` /
        ``attention_mask``; ``meta_info`` may carry ``do_sample``, ``temperature``, ``top_k``, ``top_p``,
        ``response_length``, ``pad_token_id``; ``non_tensor_batch["multi_modal_inputs"]`` images. Returns the
        reference's rollout layout (``prompts, responses, input_ids, attention_mask, position_ids, response_mask,
        rollout_log_probs``). The hybrid worker's ``generate_sequences`` adds replica pooling and timing on top."""
        from ...rollout import SamplingParams
        from ...rollout.postprocess import assemble_rollout_batch

        assert self.engine is not None, "attach() an engine first"
        rc, meta = self.config, prompts.meta_info
        g = (lambda k, d: rc.get(k, d)) if hasattr(rc, "get") else (lambda k, d: getattr(rc, k, d))
        do_sample = meta.get("do_sample", g("do_sample", True))
        sp = SamplingParams(temperature=float(meta.get("temperature", g("temperature", 1.0))) if do_sample else 0.0,
                            top_k=int(meta.get("top_k", g("top_k", -1))), top_p=float(meta.get("top_p", g("top_p", 1.0))),
                            max_tokens=int(meta.get("response_length", g("response_length", 512))),
                            ignore_eos=bool(g("ignore_eos", False)))
        ids, mask = prompts.batch["input_ids"].cpu(), prompts.batch["attention_mask"].cpu()
        plists = [row[m.bool()].tolist() for row, m in zip(ids, mask)]
        mm = prompts.non_tensor_batch.get("multi_modal_inputs")
        self.engine.wake_up()
        outs = self.engine.generate(plists, sp, multi_modal_inputs=list(mm) if mm is not None else None)
        out = assemble_rollout_batch(ids, mask, outs, sp.max_tokens, pad_token_id=meta.get("pad_token_id", 0), with_logprobs=True)
        out.non_tensor_batch.update(prompts.non_tensor_batch)
        return out
