"""Prompt datasets for RL (verl/utils/dataset/rl_dataset.py:39-362): parquet / json(l) rows with a chat
``prompt``, ``data_source``, ``reward_model{ground_truth,style}`` and ``extra_info``; items carry
``raw_prompt`` plus tokenised, left-padded ``input_ids / attention_mask / position_ids``. Also a synthetic
token-prompt dataset for benchmarks without any files.
"""

from __future__ import annotations

import copy
import json
import os
from collections import defaultdict
from typing import Optional

import numpy as np
import torch
from torch.utils.data import Dataset

from .. import torch_functional as F_


def collate_fn(data_list: list[dict]) -> dict:
    """Stack tensors; everything else becomes an object array (one entry per sample)."""
    tensors, others = defaultdict(list), defaultdict(list)
    for d in data_list:
        for k, v in d.items():
            (tensors if isinstance(v, torch.Tensor) else others)[k].append(v)
    out = {k: torch.stack(v, dim=0) for k, v in tensors.items()}
    for k, v in others.items():
        arr = np.empty(len(v), dtype=object)
        arr[:] = v
        out[k] = arr
    return out


def _read_rows(path: str) -> list[dict]:
    path = os.path.expanduser(path)
    if path.endswith(".parquet"):
        import pyarrow.parquet as pq

        return pq.read_table(path).to_pylist()
    if path.endswith(".jsonl"):
        with open(path) as f:
            return [json.loads(line) for line in f if line.strip()]
    if path.endswith(".json"):
        with open(path) as f:
            return json.load(f)
    raise ValueError(f"unsupported data file {path}")


class RLHFDataset(Dataset):
    def __init__(self, data_files, tokenizer, config, processor=None, max_samples: int = -1):
        if not isinstance(data_files, (list, tuple)):
            data_files = [data_files]
        self.data_files = list(copy.deepcopy(data_files))
        self.tokenizer, self.processor, self.config = tokenizer, processor, config
        g = config.get
        self.prompt_key = g("prompt_key", "prompt")
        self.max_prompt_length = g("max_prompt_length", 1024)
        self.return_raw_chat = g("return_raw_chat", True)
        self.return_full_prompt = g("return_full_prompt", False)
        self.truncation = g("truncation", "error")
        self.filter_overlong_prompts = g("filter_overlong_prompts", False)
        self.apply_chat_template_kwargs = dict(g("apply_chat_template_kwargs", {}) or {})
        self.need_tools_kwargs = g("need_tools_kwargs", False)
        self.shuffle, self.seed = g("shuffle", False), g("seed", None)
        self.rows: list[dict] = []
        for f in self.data_files:
            self.rows.extend(_read_rows(f))
        if max_samples is not None and 0 < max_samples < len(self.rows):
            if self.shuffle:
                rng = np.random.default_rng(self.seed)
                keep = rng.choice(len(self.rows), size=max_samples, replace=False)
                self.rows = [self.rows[i] for i in keep.tolist()]
            else:
                self.rows = self.rows[:max_samples]
        if self.filter_overlong_prompts:
            self.rows = [r for r in self.rows if len(self._tokenize(r[self.prompt_key])) <= self.max_prompt_length]
        print(f"dataset len: {len(self.rows)}")

    def _tokenize(self, messages) -> list[int]:
        if isinstance(messages, str):
            return self.tokenizer.encode(messages, add_special_tokens=False)
        if isinstance(messages, np.ndarray):
            messages = messages.tolist()
        if len(messages) and isinstance(messages[0], (int, np.integer)):
            return [int(t) for t in messages]
        return list(self.tokenizer.apply_chat_template(messages, add_generation_prompt=True, tokenize=True,
                                                       **self.apply_chat_template_kwargs))

    def __len__(self):
        return len(self.rows)

    def split(self, num_splits: int) -> list["RLHFDataset"]:
        """``num_splits`` datasets over consecutive, near-equal parts of the rows (the first ``len % num_splits`` parts
        hold one row more); they share the tokenizer, the processor and the configuration (the per-rollouter shares
        of the fully asynchronous pipeline; verl/utils/dataset/rl_dataset.py:398-447)."""
        if not isinstance(num_splits, int) or num_splits <= 0:
            raise ValueError(f"num_splits must be a positive integer, got {num_splits}")
        base, extra = divmod(len(self.rows), num_splits)
        out, lo = [], 0
        for i in range(num_splits):
            hi = lo + base + (1 if i < extra else 0)
            part = copy.copy(self)
            part.rows = self.rows[lo:hi]
            out.append(part)
            lo = hi
        return out

    def maybe_filter_out_long_prompts(self, rows: Optional[list] = None) -> list:
        """The rows whose tokenised prompt fits ``max_prompt_length`` (all rows when ``filter_overlong_prompts`` is off)."""
        rows = self.rows if rows is None else rows
        if not self.filter_overlong_prompts:
            return rows
        return [r for r in rows if len(self._tokenize(r[self.prompt_key])) <= self.max_prompt_length]

    def __getitem__(self, item):
        row = dict(self.rows[item])
        messages = row.pop(self.prompt_key)
        toks = self._tokenize(messages)
        images = row.pop(self.config.get("image_key", "images"), None)
        videos = row.pop(self.config.get("video_key", "videos"), None)
        pos3 = None
        has_img, has_vid = images is not None and len(images) > 0, videos is not None and len(videos) > 0
        if (has_img or has_vid) and self.processor is not None:
            # vision-language prompt: placeholders expanded to one token per merged patch, pixels and grids travel
            # with the row, rows 1..3 of position_ids carry the multimodal RoPE positions
            toks, mm, pos3 = self.processor(toks, list(images) if has_img else None, list(videos) if has_vid else None)
            row["multi_modal_inputs"] = mm
        ids = torch.tensor([toks], dtype=torch.long)
        mask = torch.ones_like(ids)
        pad = getattr(self.tokenizer, "pad_token_id", 0) or 0
        ids, mask = F_.postprocess_data(ids, mask, self.max_prompt_length, pad, left_pad=True, truncation=self.truncation)
        row["input_ids"], row["attention_mask"] = ids[0], mask[0]
        row["position_ids"] = F_.compute_position_id_with_mask(mask)[0]
        if pos3 is not None:
            row["position_ids"] = _with_mrope_rows(row["position_ids"], mask[0], pos3)
        row["raw_prompt_ids"] = ids[0][mask[0].bool()].tolist()
        if self.return_raw_chat:
            row["raw_prompt"] = messages
        extra = row.get("extra_info") or {}
        row["index"] = extra.get("index", item) if isinstance(extra, dict) else item
        row["tools_kwargs"] = extra.get("tools_kwargs", {}) if isinstance(extra, dict) else {}
        row["interaction_kwargs"] = extra.get("interaction_kwargs", {}) if isinstance(extra, dict) else {}
        row.setdefault("data_source", "unknown")
        return row

    def resume_dataset_state(self):
        pass

    def __getstate__(self):
        return self.__dict__.copy()


def _with_mrope_rows(text_pos: torch.Tensor, mask: torch.Tensor, pos3: torch.Tensor) -> torch.Tensor:
    """[S] text positions + [3, L] multimodal positions of the L unpadded tokens -> [4, S]."""
    out = torch.zeros(4, text_pos.numel(), dtype=torch.long)
    out[0] = text_pos
    out[1:, mask.bool()] = pos3[:, -int(mask.sum()):]  # left truncation keeps the tail
    return out


class SyntheticPromptDataset(Dataset):
    """Uniform-random token prompts: lengths in [min_len, max_len], ids in [id_lo, id_hi), fixed seed.
    Rows look like RLHFDataset rows so the same trainer, reward manager and collate function apply."""

    def __init__(self, num_prompts: int, min_len: int, max_len: int, id_lo: int, id_hi: int, max_prompt_length: int,
                 seed: int = 0, data_source: str = "synthetic/even_fraction", pad_token_id: int = 0, ground_truth=None,
                 processor=None, image_size: int = 0, video_frames: int = 0):
        """``processor`` + ``image_size`` > 0: every prompt starts with one random RGB image of that size (vision-
        language models); the text length is then in addition to the image placeholders. ``video_frames`` > 0: a random
        video of that many frames of the same size instead of the image."""
        g = torch.Generator().manual_seed(seed)
        self.items = []
        for i in range(num_prompts):
            n = int(torch.randint(min_len, max_len + 1, (1,), generator=g))
            toks = torch.randint(id_lo, id_hi, (n,), generator=g)
            extra_row, pos3 = {}, None
            if processor is not None and image_size > 0:
                if video_frames > 0:
                    vid = torch.randint(0, 256, (video_frames, image_size, image_size, 3), generator=g, dtype=torch.uint8).numpy()
                    tl, mm, pos3 = processor(toks.tolist(), None, [vid])
                else:
                    img = torch.randint(0, 256, (image_size, image_size, 3), generator=g, dtype=torch.uint8).numpy()
                    tl, mm, pos3 = processor(toks.tolist(), [img])
                toks = torch.tensor(tl, dtype=torch.long)
                n = toks.numel()
                assert n <= max_prompt_length, f"prompt of {n} tokens (with image placeholders) exceeds max_prompt_length"
                extra_row["multi_modal_inputs"] = mm
            ids = torch.full((max_prompt_length,), pad_token_id, dtype=torch.long)
            mask = torch.zeros(max_prompt_length, dtype=torch.long)
            ids[-n:], mask[-n:] = toks, 1
            pos = F_.compute_position_id_with_mask(mask)
            if pos3 is not None:
                pos = _with_mrope_rows(pos, mask, pos3)
            self.items.append({"input_ids": ids, "attention_mask": mask,
                               "position_ids": pos, "data_source": data_source,
                               "reward_model": {"ground_truth": ground_truth, "style": "rule"}, "extra_info": {"index": i},
                               "index": i, "raw_prompt_ids": toks.tolist(), **extra_row})

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        return dict(self.items[i])


def get_dataset_class(data_config):
    """``data.custom_cls`` (``path`` + ``name``: a ``torch.utils.data.Dataset`` subclass, or any class with ``__len__`` and
    ``__getitem__``, from a user's file) or :class:`RLHFDataset`."""
    from ..py_functional import load_extern_object

    cc = data_config.get("custom_cls") if hasattr(data_config, "get") else getattr(data_config, "custom_cls", None)
    path = (cc.get("path") if hasattr(cc, "get") else getattr(cc, "path", None)) if cc else None
    if not path:
        return RLHFDataset
    cls = load_extern_object(path, cc.get("name") if hasattr(cc, "get") else cc.name)
    if not (isinstance(cls, type) and hasattr(cls, "__len__") and hasattr(cls, "__getitem__")):
        raise TypeError(f"The custom dataset class '{getattr(cls, '__name__', cls)}' from '{path}' must be a dataset class "
                        "(__len__ and __getitem__)")
    return cls
