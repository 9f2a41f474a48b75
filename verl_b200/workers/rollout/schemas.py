"""Multi-turn rollout request state (verl/workers/rollout/schemas.py:37-690).

``AsyncRolloutRequest`` carries one conversation through a multi-turn rollout: the message list, and the token /
attention-mask / loss-mask / position-id streams that grow turn by turn. Each new message is tokenised
*incrementally*: the chat template is rendered on a fixed base conversation plus the new message, and the tokens
after the base conversation are appended, so earlier tokens (which the model sampled and whose log-probs are already
recorded) are never re-tokenised. Assistant tokens get ``loss_mask = 1``; user, tool and template tokens get 0.
``finalize`` splits the streams into prompt / response parts, truncates them to the configured lengths and can check
that the incremental tokenisation agrees with one full rendering of the final conversation.
"""

from __future__ import annotations

import difflib
import logging
from enum import Enum
from typing import Any, Optional

import torch
from pydantic import BaseModel, ConfigDict

from ...tools.schemas import OpenAIFunctionToolCall, OpenAIFunctionToolSchema, ToolResponse

logger = logging.getLogger(__name__)

BASE_CHAT_HISTORY = [{"role": "system", "content": "You are a helpful assistant."},
                     {"role": "user", "content": "I am a user."}]


class FinishReasonTypeEnum(str, Enum):
    LENGTH = "length"
    STOP = "stop"
    TOOL_CALL = "tool_calls"

    @classmethod
    def from_str(cls, value: str) -> "FinishReasonTypeEnum":
        for m in cls:
            if value in (m.value, m.name.lower(), "tool_call" if m is cls.TOOL_CALL else m.value):
                return m
        raise ValueError(f"Unsupported finish reason type: {value}")


class Message(BaseModel):
    role: str
    content: str | dict[str, Any] | list[dict[str, Any]]
    tool_calls: Optional[list[OpenAIFunctionToolCall]] = None


class AsyncRolloutRequestStateEnum(str, Enum):
    PENDING = "pending"
    RUNNING = "running"
    COMPLETED = "completed"
    FAILED = "failed"
    TOOL_CALLING = "tool_calling"
    INTERACTING = "interacting"


class TokenizationSanityCheckModeEnum(str, Enum):
    DISABLE = "disable"
    STRICT = "strict"
    IGNORE_STRIPPABLE = "ignore_strippable"


def _ids(tokenizer, messages, tools=None, add_generation_prompt=False) -> list[int]:
    kw = {"tools": tools} if tools else {}
    out = tokenizer.apply_chat_template(messages, add_generation_prompt=add_generation_prompt, tokenize=True, **kw)
    if isinstance(out, dict):
        out = out["input_ids"]
    if isinstance(out, torch.Tensor):
        out = out.flatten().tolist()
    return [int(t) for t in out]


class AsyncRolloutRequest(BaseModel):
    model_config = ConfigDict(arbitrary_types_allowed=True)

    batch_data_id: int = 0
    rollout_offset: int = 0
    request_id: str
    state: AsyncRolloutRequestStateEnum = AsyncRolloutRequestStateEnum.PENDING
    messages: list[Message]
    tool_schemas: Optional[list[OpenAIFunctionToolSchema]] = None
    tools_kwargs: dict[str, Any] = {}
    interaction_kwargs: dict[str, Any] = {}
    multi_modal_data: Optional[dict[str, Any]] = None
    reward_scores: dict[str, Any] = {}
    max_prompt_len: int = 1024
    max_response_len: int = 8192
    max_model_len: int = 32768
    metrics: dict[str, list[Any]] = {}
    use_inference_chat_template: bool = False
    tokenization_sanity_check_mode: TokenizationSanityCheckModeEnum = TokenizationSanityCheckModeEnum.STRICT

    # token streams: built by ``create`` and the add_* methods
    input_ids: Optional[torch.Tensor] = None
    attention_mask: Optional[torch.Tensor] = None
    loss_mask: Optional[torch.Tensor] = None
    position_ids: Optional[torch.Tensor] = None
    prompt_ids: Optional[torch.Tensor] = None
    response_ids: Optional[torch.Tensor] = None
    prompt_attention_mask: Optional[torch.Tensor] = None
    response_attention_mask: Optional[torch.Tensor] = None
    prompt_position_ids: Optional[torch.Tensor] = None
    response_position_ids: Optional[torch.Tensor] = None
    prompt_loss_mask: Optional[torch.Tensor] = None
    response_loss_mask: Optional[torch.Tensor] = None
    rollout_log_probs: Optional[torch.Tensor] = None
    generation_prompt_ids: Optional[torch.Tensor] = None
    base_conv_wo_gen_prompt_end_pos: int = 0
    base_conv_with_gen_prompt_end_pos: int = 0
    prompt_len: int = 0

    # ---------------------------------------------------------------- construction
    @classmethod
    def create(cls, processing_class, messages: list[dict | Message], **fields) -> "AsyncRolloutRequest":
        """Tokenise the initial conversation (without generation prompt) and measure the base conversation."""
        msgs = [m if isinstance(m, Message) else Message(**m) for m in messages]
        req = cls(messages=msgs, **fields)
        tools = req._tools()
        ids = _ids(processing_class, [m.model_dump(exclude_none=True) for m in msgs], tools)
        wo = _ids(processing_class, BASE_CHAT_HISTORY, tools, add_generation_prompt=False)
        with_gen = _ids(processing_class, BASE_CHAT_HISTORY, tools, add_generation_prompt=True)
        req.base_conv_wo_gen_prompt_end_pos = len(wo)
        req.base_conv_with_gen_prompt_end_pos = len(with_gen)
        req.generation_prompt_ids = torch.tensor(with_gen[len(wo):], dtype=torch.long)
        req.input_ids = torch.tensor(ids, dtype=torch.long)
        req.attention_mask = torch.ones(len(ids), dtype=torch.long)
        req.loss_mask = torch.zeros(len(ids), dtype=torch.long)
        req.position_ids = torch.arange(len(ids), dtype=torch.long)
        req.prompt_len = len(ids)
        return req

    def _tools(self):
        return [t.model_dump() for t in self.tool_schemas] if self.tool_schemas else None

    def _append(self, new_ids, loss: bool) -> None:
        new = torch.as_tensor(new_ids, dtype=torch.long).flatten()
        n = new.numel()
        if n == 0:
            return
        start = int(self.position_ids[-1]) + 1 if self.position_ids.numel() else 0
        self.input_ids = torch.cat([self.input_ids, new])
        self.attention_mask = torch.cat([self.attention_mask, torch.ones(n, dtype=torch.long)])
        self.loss_mask = torch.cat([self.loss_mask, torch.full((n,), int(loss), dtype=torch.long)])
        self.position_ids = torch.cat([self.position_ids, torch.arange(start, start + n, dtype=torch.long)])

    def _ends_with_generation_prompt(self) -> bool:
        g = self.generation_prompt_ids
        return g is not None and g.numel() > 0 and self.input_ids.numel() >= g.numel() and bool(
            (self.input_ids[-g.numel():] == g).all())

    # ---------------------------------------------------------------- turn updates
    def get_generation_prompt_ids(self, processing_class) -> list[int]:
        """Token ids to hand to the engine for the next assistant turn (appends the generation prompt once)."""
        if not self._ends_with_generation_prompt():
            self._append(self.generation_prompt_ids, loss=False)
        if self.use_inference_chat_template:
            return _ids(processing_class, [m.model_dump(exclude_none=True) for m in self.messages], self._tools(), True)
        return self.input_ids.tolist()

    def add_user_message(self, processing_class, content: str) -> None:
        self.messages.append(Message(role="user", content=content))
        self._remove_generation_prompt_ids_if_present()
        ids = _ids(processing_class, [*BASE_CHAT_HISTORY, self.messages[-1].model_dump(exclude_none=True)], self._tools())
        self._append(ids[self.base_conv_wo_gen_prompt_end_pos:], loss=False)

    def add_assistant_message(self, processing_class, content: str, content_ids=None,
                              tool_calls: Optional[list[OpenAIFunctionToolCall]] = None) -> None:
        """``content_ids``: the ids the engine sampled (preferred: they are what the log-probs belong to)."""
        self.messages.append(Message(role="assistant", content=content, tool_calls=tool_calls))
        if content_ids is None:
            ids = _ids(processing_class, [*BASE_CHAT_HISTORY, self.messages[-1].model_dump(exclude_none=True)], self._tools())
            content_ids = ids[self.base_conv_with_gen_prompt_end_pos:]
            if not self._ends_with_generation_prompt():
                self._append(self.generation_prompt_ids, loss=False)
        self._append(content_ids, loss=True)

    def add_tool_response_messages(self, processing_class, contents: list[ToolResponse | str]) -> None:
        contents = [c if isinstance(c, ToolResponse) else ToolResponse(text=str(c)) for c in contents]
        contents = [c for c in contents if not c.is_empty()]
        if not contents:
            return
        for c in contents:
            if c.is_text_only():
                self.messages.append(Message(role="tool", content=c.text))
            else:
                parts = [{"type": "image"} for _ in (c.image or [])] + [{"type": "video"} for _ in (c.video or [])]
                if c.text:
                    parts.append({"type": "text", "text": c.text})
                self.messages.append(Message(role="tool", content=parts))
                if self.multi_modal_data is None:
                    self.multi_modal_data = {}
                self.multi_modal_data.setdefault("image", []).extend(c.image or [])
                self.multi_modal_data.setdefault("video", []).extend(c.video or [])
        self._remove_generation_prompt_ids_if_present()
        new = [m.model_dump(exclude_none=True) for m in self.messages[-len(contents):]]
        ids = _ids(processing_class, [*BASE_CHAT_HISTORY, *new], self._tools())
        self._append(ids[self.base_conv_wo_gen_prompt_end_pos:], loss=False)

    def update_metrics(self, metrics: Any, tool_id: str) -> None:
        self.metrics.setdefault(tool_id, []).append(metrics)

    def _remove_generation_prompt_ids_if_present(self) -> None:
        if self._ends_with_generation_prompt() and self.input_ids.numel() > self.prompt_len:
            n = self.generation_prompt_ids.numel()
            for name in ("input_ids", "attention_mask", "loss_mask", "position_ids"):
                setattr(self, name, getattr(self, name)[:-n])

    # ---------------------------------------------------------------- finish
    def _sanity_check(self, processing_class) -> None:
        mode = self.tokenization_sanity_check_mode
        if mode == TokenizationSanityCheckModeEnum.DISABLE:
            return
        full = _ids(processing_class, [m.model_dump(exclude_none=True) for m in self.messages], self._tools())
        mine = self.input_ids.tolist()
        if full == mine:
            return
        diffs = [(tag, full[i1:i2], mine[j1:j2]) for tag, i1, i2, j1, j2 in
                 difflib.SequenceMatcher(None, full, mine, autojunk=False).get_opcodes() if tag != "equal"]
        if mode == TokenizationSanityCheckModeEnum.IGNORE_STRIPPABLE and hasattr(processing_class, "decode"):
            if all(not processing_class.decode(a).strip() and not processing_class.decode(b).strip() for _, a, b in diffs):
                return
        logger.warning("incremental tokenisation of request %s differs from a full rendering in %d place(s); the "
                       "model saw the incremental stream. First difference: %s", self.request_id, len(diffs), diffs[:1])

    def finalize(self, processing_class, reward_scores: dict[str, Any],
                 finish_reason_type: FinishReasonTypeEnum = FinishReasonTypeEnum.STOP) -> None:
        self.state = AsyncRolloutRequestStateEnum.COMPLETED
        self.reward_scores = reward_scores
        self._remove_generation_prompt_ids_if_present()
        self._sanity_check(processing_class)
        if finish_reason_type not in (FinishReasonTypeEnum.STOP, FinishReasonTypeEnum.LENGTH):
            raise ValueError(f"Unsupported finalize finish reason type: {finish_reason_type}")
        self.truncate_output_ids(processing_class)

    def truncate_output_ids(self, processing_class=None) -> None:
        p = self.prompt_len
        cut = min(self.input_ids.numel(), self.max_model_len, p + self.max_response_len)
        for name in ("input_ids", "attention_mask", "loss_mask", "position_ids"):
            full = getattr(self, name)[:cut]
            setattr(self, name, full)
            lo = max(0, p - self.max_prompt_len)  # prompts keep their tail, as left truncation does
            setattr(self, {"input_ids": "prompt_ids"}.get(name, "prompt_" + name), full[lo:p])
            setattr(self, {"input_ids": "response_ids"}.get(name, "response_" + name), full[p:])
