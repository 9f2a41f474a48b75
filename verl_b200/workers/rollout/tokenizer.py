"""Tokenizer interface a rollout engine needs (verl/workers/rollout/tokenizer.py:26-163): the subset of the HF
tokenizer API that inference engines call, so that non-HF tokenizers can be plugged in, plus an adapter that exposes
any object with ``encode`` / ``decode`` (e.g. :class:`verl_b200.utils.tokenizer.IntTokenizer`) through it."""

from __future__ import annotations

from abc import ABC, abstractmethod


class HybridEngineBaseTokenizer(ABC):
    @property
    @abstractmethod
    def vocab_size(self) -> int: ...

    @property
    @abstractmethod
    def pad_token_id(self) -> int: ...

    @property
    @abstractmethod
    def eos_token_id(self) -> int: ...

    @property
    @abstractmethod
    def all_special_ids(self) -> list[int]: ...

    @property
    @abstractmethod
    def all_special_tokens(self) -> list[str]: ...

    @abstractmethod
    def encode(self, text: str) -> list[int]: ...

    @abstractmethod
    def decode(self, token_ids, skip_special_tokens: bool = False, clean_up_tokenization_spaces=None, **kwargs) -> str: ...

    @abstractmethod
    def convert_ids_to_tokens(self, ids, skip_special_tokens: bool = False): ...

    @abstractmethod
    def get_added_vocab(self) -> dict[str, int]: ...

    @abstractmethod
    def convert_tokens_to_string(self, tokens: list[str]) -> str: ...

    @property
    def is_fast(self) -> bool:
        return False


class TokenizerAdapter(HybridEngineBaseTokenizer):
    """Wraps an HF tokenizer or a minimal ``encode`` / ``decode`` object."""

    def __init__(self, tokenizer):
        self.tok = tokenizer

    @property
    def vocab_size(self) -> int:
        return int(getattr(self.tok, "vocab_size", 0) or len(self.tok))

    @property
    def pad_token_id(self) -> int:
        return self.tok.pad_token_id

    @property
    def eos_token_id(self) -> int:
        return self.tok.eos_token_id

    @property
    def all_special_ids(self) -> list[int]:
        ids = getattr(self.tok, "all_special_ids", None)
        return list(ids) if ids is not None else [i for i in {self.pad_token_id, self.eos_token_id} if i is not None]

    @property
    def all_special_tokens(self) -> list[str]:
        toks = getattr(self.tok, "all_special_tokens", None)
        return list(toks) if toks is not None else [str(i) for i in self.all_special_ids]

    def encode(self, text: str) -> list[int]:
        return list(self.tok.encode(text))

    def decode(self, token_ids, skip_special_tokens: bool = False, clean_up_tokenization_spaces=None, **kwargs) -> str:
        return self.tok.decode(token_ids, skip_special_tokens=skip_special_tokens)

    def convert_ids_to_tokens(self, ids, skip_special_tokens: bool = False):
        f = getattr(self.tok, "convert_ids_to_tokens", None)
        if f is not None:
            return f(ids, skip_special_tokens=skip_special_tokens)
        special = set(self.all_special_ids) if skip_special_tokens else set()
        if isinstance(ids, int):
            return str(ids)
        return [str(i) for i in ids if i not in special]

    def get_added_vocab(self) -> dict[str, int]:
        f = getattr(self.tok, "get_added_vocab", None)
        return dict(f()) if f is not None else {}

    def convert_tokens_to_string(self, tokens: list[str]) -> str:
        f = getattr(self.tok, "convert_tokens_to_string", None)
        return f(tokens) if f is not None else " ".join(tokens)

    @property
    def is_fast(self) -> bool:
        return bool(getattr(self.tok, "is_fast", False))
