"""Reference rollouts without paging: a plain token-by-token sampling loop (``NaiveRollout``,
verl/workers/rollout/naive/naive_rollout.py) and its HF-generate-style variant (``HFRollout``,
verl/workers/rollout/hf_rollout.py). They recompute the full context every step — useful as oracles for the
paged engine and on machines without the native library."""

from __future__ import annotations

import torch

from ...models import PackedBatch
from ...protocol import DataProto
from ...utils.torch_functional import get_response_mask
from .base import BaseRollout


class NaiveRollout(BaseRollout):
    def __init__(self, module, config, model_config=None, device_mesh=None):
        super().__init__(config, model_config, device_mesh)
        self.module = module

    async def resume(self, tags):
        pass

    async def release(self):
        pass

    async def update_weights(self, weights, **kwargs):
        own = dict(self.module.named_parameters())
        from ...models.hf_io import hf_to_native_state_dict

        for k, v in hf_to_native_state_dict(self.module.cfg, dict(weights)).items():
            if k in own:
                own[k].data.copy_(v.to(own[k].dtype))

    @torch.no_grad()
    def generate_sequences(self, prompts: DataProto) -> DataProto:
        g = self.config.get if hasattr(self.config, "get") else (lambda k, d=None: getattr(self.config, k, d))
        ids, mask = prompts.batch["input_ids"], prompts.batch["attention_mask"]
        eos = prompts.meta_info.get("eos_token_id", self.module.cfg.eos_token_id)
        R = int(g("response_length", 16))
        temp = float(prompts.meta_info.get("temperature", g("temperature", 1.0)))
        do_sample = bool(prompts.meta_info.get("do_sample", g("do_sample", True)))
        top_k = int(g("top_k", -1) or -1)
        B, P = ids.shape
        done = torch.zeros(B, dtype=torch.bool)
        logps = []
        for _ in range(R):
            batch, idx = PackedBatch.from_padded(ids, mask)
            logits = self.module(batch)
            last = batch.cu_seqlens[1:].long() - 1
            lg = logits[last].float() / max(temp, 1e-6)
            if top_k > 0:
                kth = torch.topk(lg, min(top_k, lg.size(-1)))[0][:, -1, None]
                lg = lg.masked_fill(lg < kth, float("-inf"))
            lp = torch.log_softmax(lg, -1)
            nxt = torch.multinomial(lp.exp(), 1)[:, 0] if do_sample else lp.argmax(-1)
            logps.append(lp.gather(1, nxt[:, None])[:, 0])
            nxt = torch.where(done, torch.full_like(nxt, eos), nxt)
            ids = torch.cat([ids, nxt[:, None]], 1)
            mask = torch.cat([mask, (~done).long()[:, None]], 1)
            done |= nxt == eos
            if done.all():
                break
        resp = ids[:, P:]
        pad = R - resp.shape[1]
        if pad > 0:
            resp = torch.nn.functional.pad(resp, (0, pad), value=eos)
            ids = torch.cat([ids[:, :P], resp], 1)
            mask = torch.nn.functional.pad(mask, (0, pad), value=0)
        rmask = get_response_mask(resp, eos, dtype=mask.dtype)
        mask = torch.cat([mask[:, :P], rmask], 1)
        lps = torch.zeros(B, R)
        if logps:
            lps[:, : len(logps)] = torch.stack(logps, 1)
        pos = (mask.cumsum(-1) - 1).clamp(min=0)
        return DataProto.from_dict({"prompts": ids[:, :P], "responses": resp, "input_ids": ids, "attention_mask": mask,
                                    "position_ids": pos, "response_mask": rmask, "rollout_log_probs": lps * rmask})


class HFRollout(NaiveRollout):
    """HF ``generate``-style rollout on the training module itself (verl/workers/rollout/hf_rollout.py:39-176): the
    batch is processed in chunks of ``micro_batch_size``; greedy decoding when ``do_sample`` is off, the ``val_kwargs``
    sampling parameters for validation batches, the rollout's ``temperature / top_k / top_p`` otherwise (``top_k <= 0``
    = off, as the inference servers count it); ``num_return_sequences`` repeats the prompts. Padding after the end of
    a response uses ``pad_token_id``."""

    def generate_sequences(self, prompts: DataProto) -> DataProto:
        g = self.config.get if hasattr(self.config, "get") else (lambda k, d=None: getattr(self.config, k, d))
        n = int(prompts.meta_info.get("num_return_sequences", 1))
        if n > 1:
            prompts = prompts.repeat(n, interleave=True)
        B = len(prompts)
        micro = int(g("micro_batch_size", None) or B)
        chunks = prompts.chunk(max(B // micro, 1)) if B >= micro and B % max(B // micro, 1) == 0 else [prompts]
        return DataProto.concat([self._generate_minibatch(c) for c in chunks])

    @torch.no_grad()
    def _generate_minibatch(self, prompts: DataProto) -> DataProto:
        g = self.config.get if hasattr(self.config, "get") else (lambda k, d=None: getattr(self.config, k, d))
        meta = prompts.meta_info
        do_sample = bool(meta.get("do_sample", g("do_sample", True)))
        validate = bool(meta.get("validate", False))
        vk = g("val_kwargs", None)
        vget = (vk.get if hasattr(vk, "get") else (lambda k, d=None: getattr(vk, k, d))) if vk is not None else (lambda k, d=None: d)
        if not do_sample:
            temp, top_k, top_p = 0.0, 0, 1.0
        elif validate:
            temp, top_k, top_p = float(vget("temperature", 1.0)), max(0, int(vget("top_k", 0) or 0)), float(vget("top_p", 1.0))
        else:
            temp = float(meta.get("temperature", g("temperature", 1.0)))
            top_k = max(0, int(meta.get("top_k", g("top_k", 0)) or 0))
            top_p = float(meta.get("top_p", g("top_p", 1.0)))
        R = int(meta.get("response_length", g("response_length", 16)))
        eos = meta.get("eos_token_id", self.module.cfg.eos_token_id)
        pad = meta.get("pad_token_id", eos if eos is not None else 0)
        ids, mask = prompts.batch["input_ids"], prompts.batch["attention_mask"]
        B, P = ids.shape
        was_training = self.module.training
        self.module.eval()
        done = torch.zeros(B, dtype=torch.bool, device=ids.device)
        logps = []
        for _ in range(R):
            batch, _ = PackedBatch.from_padded(ids, mask)
            logits = self.module(batch)
            lg = logits[batch.cu_seqlens[1:].long() - 1].float()
            if temp > 0:
                lg = lg / temp
                if top_k > 0:
                    kth = torch.topk(lg, min(top_k, lg.size(-1)))[0][:, -1, None]
                    lg = lg.masked_fill(lg < kth, float("-inf"))
                if top_p < 1.0:
                    sp, si = torch.sort(torch.softmax(lg, -1), descending=True)
                    drop = sp.cumsum(-1) - sp > top_p  # keep the smallest prefix whose mass reaches top_p
                    lg = lg.masked_fill(torch.zeros_like(drop).scatter(1, si, drop), float("-inf"))
            lp = torch.log_softmax(lg, -1)
            nxt = torch.multinomial(lp.exp(), 1)[:, 0] if temp > 0 else lp.argmax(-1)
            logps.append(lp.gather(1, nxt[:, None])[:, 0])
            nxt = torch.where(done, torch.full_like(nxt, pad), nxt)
            ids = torch.cat([ids, nxt[:, None]], 1)
            mask = torch.cat([mask, (~done).to(mask.dtype)[:, None]], 1)
            if eos is not None:
                done |= nxt == eos
            if done.all():
                break
        self.module.train(was_training)
        resp = ids[:, P:]
        short = R - resp.shape[1]
        if short > 0:
            resp = torch.nn.functional.pad(resp, (0, short), value=pad)
            ids = torch.cat([ids[:, :P], resp], 1)
            mask = torch.nn.functional.pad(mask, (0, short), value=0)
        rmask = mask[:, P:]
        lps = torch.zeros(B, R, device=ids.device)
        if logps:
            lps[:, : len(logps)] = torch.stack(logps, 1)
        pos = (mask.cumsum(-1) - 1).clamp(min=0)
        return DataProto.from_dict({"prompts": ids[:, :P], "responses": resp, "input_ids": ids, "attention_mask": mask,
                                    "position_ids": pos, "response_mask": rmask, "rollout_log_probs": lps * rmask},
                                   meta_info={k: v for k, v in meta.items() if k in ("eos_token_id", "pad_token_id")})
