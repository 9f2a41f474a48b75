"""Chat-template probes (verl/utils/chat_template.py:9-47): find the tokens a template puts in front of the first
turn (system prompt) and the generation prompt, by differencing renderings of one and two empty user turns."""

from __future__ import annotations


def _render(tokenizer, n_turns: int, add_generation_prompt: bool, **kw) -> list[int]:
    ids = tokenizer.apply_chat_template([{"role": "user", "content": ""}] * n_turns,
                                        add_generation_prompt=add_generation_prompt, tokenize=True, **kw)
    return list(ids["input_ids"] if isinstance(ids, dict) else ids)


def initialize_system_prompt(tokenizer, **apply_chat_template_kwargs) -> list[int]:
    one = _render(tokenizer, 1, False, **apply_chat_template_kwargs)
    two = _render(tokenizer, 2, False, **apply_chat_template_kwargs)
    turn = len(two) - len(one)
    return one[: len(one) - turn] if turn > 0 else []


def extract_system_prompt_and_generation(tokenizer):
    one = _render(tokenizer, 1, False)
    system = initialize_system_prompt(tokenizer)
    with_gen = _render(tokenizer, 1, True)
    return system, with_gen[len(one):]
