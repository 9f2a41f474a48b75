"""Agent-loop helpers (verl/experimental/agent_loop/utils.py:19-109)."""

from __future__ import annotations

import os
from typing import Any


def _inside(path: str, root: str) -> bool:
    return path == root or path.startswith(root + os.sep)


def resolve_config_path(config_path: str) -> str:
    """Absolute paths pass; relative ones are tried against the working directory, then the project root, then the
    package directory (worker processes may start in another directory than the driver)."""
    if os.path.isabs(config_path):
        return config_path
    import verl_b200

    pkg = os.path.abspath(os.path.dirname(verl_b200.__file__))
    for root in (os.path.abspath(os.getcwd()), os.path.dirname(pkg), pkg):
        cand = os.path.abspath(os.path.join(root, config_path))
        if _inside(cand, root) and os.path.exists(cand):
            return cand
    raise FileNotFoundError(f"Agent loop configuration file not found: {config_path}. Tried current directory and "
                            "the project root.")


def format_gpt_oss_tool_response_manually(tool_response: str, tool_call_name: str) -> str:
    """gpt-oss chat templates cannot render a tool message without the call that caused it; this is the same text."""
    return f"<|start|>functions.{tool_call_name} to=assistant<|channel|>commentary<|message|>{tool_response}<|end|>"


def add_generation_prompt_for_gpt_oss(message_content: str) -> str:
    return message_content + "<|start|>assistant"


def build_gpt_oss_tool_response_text(messages: list[dict[str, Any]], tool_call_names: list[str]) -> str:
    text = "".join(format_gpt_oss_tool_response_manually(m["content"], n) for m, n in zip(messages, tool_call_names))
    return add_generation_prompt_for_gpt_oss(text)
