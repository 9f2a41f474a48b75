"""Tokenizer helpers (verl/utils/tokenizer.py): HF tokenizers with pad-token fix-ups, plus a dependency-free
integer tokenizer for synthetic-token benchmarks and tests."""

from __future__ import annotations

import warnings


def set_pad_token_id(tokenizer):
    if tokenizer.pad_token_id is None:
        tokenizer.pad_token_id = tokenizer.eos_token_id
        warnings.warn(f"tokenizer.pad_token_id is None. Now set to {tokenizer.eos_token_id}", stacklevel=1)
    if tokenizer.pad_token is None:
        tokenizer.pad_token = tokenizer.eos_token


def hf_tokenizer(name_or_path, correct_pad_token=True, correct_gemma2=True, **kwargs):
    from transformers import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(name_or_path, **kwargs)
    if correct_pad_token:
        set_pad_token_id(tok)
    return tok


def hf_processor(name_or_path, **kwargs):
    from transformers import AutoProcessor

    try:
        proc = AutoProcessor.from_pretrained(name_or_path, **kwargs)
    except Exception:
        return None
    if proc is not None and "Processor" not in proc.__class__.__name__:
        return None
    return proc


class IntTokenizer:
    """Token ids <-> space-separated integers. Used where prompts are synthetic id sequences."""

    def __init__(self, vocab_size: int, eos_token_id: int = 2, pad_token_id: int = 0):
        self.vocab_size, self.eos_token_id, self.pad_token_id = vocab_size, eos_token_id, pad_token_id
        self.eos_token, self.pad_token = str(eos_token_id), str(pad_token_id)
        self.chat_template = None

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        return [int(t) % self.vocab_size for t in text.split()]

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        ids = [int(t) for t in ids]
        if skip_special_tokens:
            ids = [t for t in ids if t not in (self.eos_token_id, self.pad_token_id)]
        return " ".join(str(t) for t in ids)

    def batch_decode(self, batch, skip_special_tokens: bool = True) -> list[str]:
        return [self.decode(x, skip_special_tokens) for x in batch]

    def apply_chat_template(self, messages, add_generation_prompt=True, tokenize=True, **kwargs):
        text = " ".join(str(m["content"]) for m in messages)
        return self.encode(text) if tokenize else text

    def __call__(self, text, return_tensors=None, add_special_tokens=False, **kwargs):
        import torch

        ids = self.encode(text)
        if return_tensors == "pt":
            t = torch.tensor([ids])
            return {"input_ids": t, "attention_mask": torch.ones_like(t)}
        return {"input_ids": ids, "attention_mask": [1] * len(ids)}
