"""Tool-call parsers for model output (verl/experimental/agent_loop/tool_parser.py:76-162): Hermes
``<tool_call>{json}</tool_call>`` blocks and the GPT-OSS channel format."""

from __future__ import annotations

import json
import re
from abc import ABC, abstractmethod
from dataclasses import dataclass


@dataclass
class FunctionCall:
    name: str
    arguments: str  # JSON text


class ToolParser(ABC):
    _registry: dict[str, type["ToolParser"]] = {}

    def __init__(self, tokenizer):
        self.tokenizer = tokenizer

    @abstractmethod
    async def extract_tool_calls(self, responses_ids: list[int]) -> tuple[str, list[FunctionCall]]:
        """Return (text with the tool-call markup removed, parsed calls)."""

    @classmethod
    def register(cls, name: str):
        def deco(sub):
            cls._registry[name] = sub
            return sub

        return deco

    @classmethod
    def get_tool_parser(cls, name: str, tokenizer) -> "ToolParser":
        if name not in cls._registry:
            raise ValueError(f"Unknown tool parser: {name}")
        return cls._registry[name](tokenizer)


@ToolParser.register("hermes")
class HermesToolParser(ToolParser):
    _pat = re.compile(r"<tool_call>(.*?)</tool_call>", re.DOTALL)

    async def extract_tool_calls(self, responses_ids):
        text = self.tokenizer.decode(responses_ids)
        if "<tool_call>" not in text or "</tool_call>" not in text:
            return text, []
        calls = []
        for m in self._pat.findall(text):
            try:
                obj = json.loads(m)
                calls.append(FunctionCall(name=obj["name"], arguments=json.dumps(obj.get("arguments", {}), ensure_ascii=False)))
            except Exception:
                continue  # malformed JSON is ignored; the model sees no tool response for it
        return self._pat.sub("", text), calls


@ToolParser.register("gpt-oss")
class GptOssToolParser(ToolParser):
    _pat = re.compile(r"<\|start\|>assistant<\|channel\|>commentary to=functions\.(\w+).*?<\|message\|>(.*?)<\|call\|>", re.DOTALL)
    _cot = re.compile(r"<\|start\|>assistant<\|channel\|>analysis<\|message\|>.*?<\|end\|>", re.DOTALL)

    async def extract_tool_calls(self, responses_ids):
        text = self.tokenizer.decode(responses_ids, skip_special_tokens=False)
        text = text.replace(getattr(self.tokenizer, "pad_token", None) or "\x00", "")
        text = self._cot.sub("", text)
        calls = []
        for name, args in self._pat.findall(text):
            try:
                json.loads(args)
                calls.append(FunctionCall(name=name, arguments=args))
            except Exception:
                continue
        return self._pat.sub("", text), calls
