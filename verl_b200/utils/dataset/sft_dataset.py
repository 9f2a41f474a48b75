"""Supervised fine-tuning datasets.

``SFTDataset`` (verl/utils/dataset/sft_dataset.py): single-turn rows with a prompt and a response column
(optionally nested through ``prompt_dict_keys`` / ``response_dict_keys``); the prompt goes through the chat
template with a generation prompt, the response gets EOS appended, the loss mask covers the response tokens
(shifted so that position ``i`` predicts token ``i + 1``).

``MultiTurnSFTDataset`` (verl/utils/dataset/multiturn_sft_dataset.py): rows with a ``messages`` list; every
message is tokenised incrementally with the chat template and only assistant turns carry loss.

``RMDataset`` (verl/utils/dataset/rm_dataset.py): (prompt, chosen, rejected) triples for reward-model training.

Items are dicts of 1-D tensors. ``pad_mode = "right"`` pads / truncates to ``max_length``;
``pad_mode = "no_padding"`` returns the ragged sequence (the engine packs sequences, so nothing is padded).
Synthetic token data (``synthetic:<num>:<min_len>:<max_len>:<vocab>:<seed>``) needs no files.
"""

from __future__ import annotations

from typing import Optional

import numpy as np
import torch
from torch.utils.data import Dataset

from .rl_dataset import _read_rows


def _get(cfg, key, default=None):
    if cfg is None:
        return default
    if isinstance(cfg, dict):
        return cfg.get(key, default)
    v = getattr(cfg, key, default)
    return default if v is None else v


def _nested(row, key, dict_keys):
    v = row[key]
    for k in dict_keys or []:
        v = v[k]
    return v


def _finish(ids: list[int], loss: list[int], max_length: int, truncation: str, pad_mode: str, pad_id: int) -> dict:
    n = len(ids)
    if n > max_length:
        if truncation == "error":
            raise ValueError(f"sequence length {n} is larger than max_length {max_length}")
        if truncation == "left":
            ids, loss = ids[-max_length:], loss[-max_length:]
        else:  # right
            ids, loss = ids[:max_length], loss[:max_length]
        n = max_length
    input_ids = torch.tensor(ids, dtype=torch.long)
    loss_mask = torch.tensor(loss, dtype=torch.long)
    attn = torch.ones(n, dtype=torch.long)
    if pad_mode == "right" and n < max_length:
        pad = max_length - n
        input_ids = torch.cat([input_ids, torch.full((pad,), pad_id, dtype=torch.long)])
        loss_mask = torch.cat([loss_mask, torch.zeros(pad, dtype=torch.long)])
        attn = torch.cat([attn, torch.zeros(pad, dtype=torch.long)])
    pos = (torch.cumsum(attn, 0) - 1).clamp(min=0)
    return {"input_ids": input_ids, "attention_mask": attn, "position_ids": pos, "loss_mask": loss_mask}


class _SyntheticRows:
    """``synthetic:<num>:<min_len>:<max_len>:<vocab>:<seed>``: random token sequences, first third = prompt."""

    def __init__(self, spec: str):
        p = spec.split(":")
        self.num, self.lo, self.hi, self.vocab = int(p[1]), int(p[2]), int(p[3]), int(p[4])
        self.seed = int(p[5]) if len(p) > 5 else 0

    def __len__(self):
        return self.num

    def row(self, i: int):
        g = np.random.default_rng(self.seed * 1_000_003 + i)
        n = int(g.integers(self.lo, self.hi + 1))
        ids = g.integers(3, self.vocab, size=n).tolist()
        k = max(1, n // 3)
        return ids, [0] * k + [1] * (n - k)


class SFTDataset(Dataset):
    def __init__(self, parquet_files, tokenizer, config=None, max_samples: int = -1):
        self.tokenizer = tokenizer
        self.prompt_key = _get(config, "prompt_key", "prompt")
        self.response_key = _get(config, "response_key", "response")
        self.prompt_dict_keys = _get(config, "prompt_dict_keys", None)
        self.response_dict_keys = _get(config, "response_dict_keys", None)
        self.max_length = int(_get(config, "max_length", 1024))
        self.truncation = _get(config, "truncation", "error")
        self.pad_mode = _get(config, "pad_mode", "right")
        self.chat_kwargs = dict(_get(config, "apply_chat_template_kwargs", {}) or {})
        files = parquet_files if isinstance(parquet_files, (list, tuple)) else [parquet_files]
        self.synthetic: Optional[_SyntheticRows] = None
        self.rows: list[dict] = []
        if len(files) == 1 and str(files[0]).startswith("synthetic:"):
            self.synthetic = _SyntheticRows(str(files[0]))
        else:
            for f in files:
                self.rows.extend(_read_rows(f))
            if max_samples and max_samples > 0:
                self.rows = self.rows[:max_samples]

    def __len__(self):
        return len(self.synthetic) if self.synthetic is not None else len(self.rows)

    def _pad_id(self) -> int:
        pid = getattr(self.tokenizer, "pad_token_id", None)
        return 0 if pid is None else int(pid)

    def __getitem__(self, i: int) -> dict:
        if self.synthetic is not None:
            ids, loss = self.synthetic.row(i)
            return _finish(ids, _shift(loss), self.max_length, "right", self.pad_mode, self._pad_id())
        row = self.rows[i]
        prompt = _nested(row, self.prompt_key, self.prompt_dict_keys)
        response = _nested(row, self.response_key, self.response_dict_keys)
        chat = prompt if isinstance(prompt, list) else [{"role": "user", "content": str(prompt)}]
        p_ids = list(self.tokenizer.apply_chat_template(chat, add_generation_prompt=True, tokenize=True, **self.chat_kwargs))
        eos = getattr(self.tokenizer, "eos_token", None) or ""
        r_ids = list(self.tokenizer.encode(str(response) + eos, add_special_tokens=False))
        ids = p_ids + r_ids
        loss = [0] * len(p_ids) + [1] * len(r_ids)
        return _finish(ids, _shift(loss), self.max_length, self.truncation, self.pad_mode, self._pad_id())


def _shift(token_is_target: list[int]) -> list[int]:
    """Loss mask aligned with predictions: position i carries loss if token i + 1 is a target
    (verl/utils/dataset/sft_dataset.py: the mask of the last prompt token is 1, of the last response token 0)."""
    return token_is_target[1:] + [0]


class MultiTurnSFTDataset(Dataset):
    def __init__(self, parquet_files, tokenizer, config=None, max_samples: int = -1):
        self.tokenizer = tokenizer
        self.messages_key = _get(config, "messages_key", "messages")
        self.tools_key = _get(config, "tools_key", "tools")
        self.enable_thinking_key = _get(config, "enable_thinking_key", "enable_thinking")
        self.max_length = int(_get(config, "max_length", 1024))
        self.truncation = _get(config, "truncation", "error")
        self.pad_mode = _get(config, "pad_mode", "no_padding")
        self.chat_kwargs = dict(_get(config, "apply_chat_template_kwargs", {}) or {})
        self.ignore_mismatch = bool(_get(config, "ignore_input_ids_mismatch", False))
        files = parquet_files if isinstance(parquet_files, (list, tuple)) else [parquet_files]
        self.synthetic: Optional[_SyntheticRows] = None
        self.rows: list[dict] = []
        if len(files) == 1 and str(files[0]).startswith("synthetic:"):
            self.synthetic = _SyntheticRows(str(files[0]))
        else:
            for f in files:
                self.rows.extend(_read_rows(f))
            if max_samples and max_samples > 0:
                self.rows = self.rows[:max_samples]

    def __len__(self):
        return len(self.synthetic) if self.synthetic is not None else len(self.rows)

    def _tokenize(self, messages, tools, upto: int, gen_prompt: bool) -> list[int]:
        kw = dict(self.chat_kwargs)
        if tools:
            kw["tools"] = tools
        return list(self.tokenizer.apply_chat_template(messages[:upto], add_generation_prompt=gen_prompt, tokenize=True, **kw))

    def __getitem__(self, i: int) -> dict:
        pad_id = getattr(self.tokenizer, "pad_token_id", None) or 0
        if self.synthetic is not None:
            ids, loss = self.synthetic.row(i)
            return _finish(ids, _shift(loss), self.max_length, "right", self.pad_mode, pad_id)
        row = self.rows[i]
        messages = list(row[self.messages_key])
        tools = row.get(self.tools_key)
        ids: list[int] = []
        target: list[int] = []
        for k, msg in enumerate(messages):
            if msg["role"] == "assistant":
                # tokens up to the generation prompt belong to the context, the rest is the model's turn
                head = self._tokenize(messages, tools, k, True)
                full = self._tokenize(messages, tools, k + 1, False)
                if full[: len(ids)] != ids and not self.ignore_mismatch:
                    raise ValueError("chat template is not prefix-stable across turns (set ignore_input_ids_mismatch)")
                head = head if full[: len(head)] == head else full[: len(ids)]
                target += [0] * (len(head) - len(ids)) + [1] * (len(full) - len(head))
                ids = full
            elif k == len(messages) - 1 or messages[k + 1]["role"] != "assistant":
                full = self._tokenize(messages, tools, k + 1, False)
                target += [0] * (len(full) - len(ids))
                ids = full
        if not ids:
            ids = self._tokenize(messages, tools, len(messages), False)
            target = [0] * len(ids)
        return _finish(ids, _shift(target), self.max_length, self.truncation, self.pad_mode, pad_id)


class RMDataset(Dataset):
    """(prompt, chosen, rejected) -> input_ids [2, L], attention_mask [2, L] (chosen first)."""

    def __init__(self, parquet_files, tokenizer, prompt_key="prompt", chosen_key="chosen", rejected_key="rejected",
                 max_length: int = 1024, add_eos: bool = True, max_samples: int = -1):
        self.tokenizer, self.max_length, self.add_eos = tokenizer, max_length, add_eos
        self.keys = (prompt_key, chosen_key, rejected_key)
        files = parquet_files if isinstance(parquet_files, (list, tuple)) else [parquet_files]
        self.rows = []
        for f in files:
            self.rows.extend(_read_rows(f))
        if max_samples and max_samples > 0:
            self.rows = self.rows[:max_samples]

    def __len__(self):
        return len(self.rows)

    def _pad(self, ids: list[int]):
        ids = ids[: self.max_length]
        n = len(ids)
        pad_id = getattr(self.tokenizer, "pad_token_id", None) or 0
        t = torch.full((self.max_length,), pad_id, dtype=torch.long)
        t[:n] = torch.tensor(ids, dtype=torch.long)
        m = torch.zeros(self.max_length, dtype=torch.long)
        m[:n] = 1
        return t, m

    def __getitem__(self, i: int) -> dict:
        row = self.rows[i]
        pk, ck, rk = self.keys
        enc = lambda s: list(self.tokenizer.encode(str(s), add_special_tokens=False))  # noqa: E731
        p = enc(row[pk])
        eos = [self.tokenizer.eos_token_id] if self.add_eos and getattr(self.tokenizer, "eos_token_id", None) is not None else []
        c, cm = self._pad(p + enc(row[ck]) + eos)
        r, rm = self._pad(p + enc(row[rk]) + eos)
        return {"input_ids": torch.stack([c, r]), "attention_mask": torch.stack([cm, rm])}


def sft_collate_fn(items: list[dict]) -> dict:
    """Right-padded batches stack; ragged (``no_padding``) batches are padded to the longest item here, the
    trainer packs them again by attention mask."""
    n = max(int(it["input_ids"].numel()) for it in items)
    out = {}
    for k in items[0]:
        rows = []
        for it in items:
            t = it[k]
            if t.numel() < n:
                t = torch.cat([t, torch.zeros(n - t.numel(), dtype=t.dtype)])
            rows.append(t)
        out[k] = torch.stack(rows)
    return out
