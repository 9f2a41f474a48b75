"""Single-turn agent loop: one prompt, one completion (verl/experimental/agent_loop/single_turn_agent_loop.py)."""

from __future__ import annotations

import time
from typing import Any
from uuid import uuid4

from .agent_loop import AgentLoopBase, AgentLoopMetrics, AgentLoopOutput, register


@register("single_turn_agent")
class SingleTurnAgentLoop(AgentLoopBase):
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        rc = self.config.actor_rollout_ref.rollout
        self.prompt_length, self.response_length = int(rc.prompt_length), int(rc.response_length)

    async def run(self, sampling_params: dict[str, Any], **kwargs) -> AgentLoopOutput:
        mm = kwargs.get("multi_modal_inputs")
        if isinstance(mm, dict) and mm and kwargs.get("raw_prompt_ids") is not None:
            # vision-language sample: the dataset's ids already hold one placeholder token per merged patch of the
            # sample's images / videos; re-tokenising the chat messages would lose that expansion
            prompt_ids = [int(t) for t in kwargs["raw_prompt_ids"]]
        else:
            prompt_ids = await self.apply_chat_template(kwargs["raw_prompt"])
        t0 = time.perf_counter()
        # the output is cut to response_length below: do not let the server spend the unused prompt budget on it
        sampling_params = dict(sampling_params)
        sampling_params["max_tokens"] = min(int(sampling_params.get("max_tokens", self.response_length)), self.response_length)
        # vision-language samples: the dataset's patches and grids go with the request (the prompt ids already hold one
        # placeholder token per merged patch)
        out = await self.server_manager.generate(uuid4().hex, prompt_ids=prompt_ids, sampling_params=sampling_params,
                                                 image_data=mm if isinstance(mm, dict) and mm else None)
        dt = time.perf_counter() - t0
        ids = out.token_ids[: self.response_length]
        return AgentLoopOutput(prompt_ids=prompt_ids, response_ids=ids, response_mask=[1] * len(ids),
                               response_logprobs=out.log_probs[: self.response_length] if out.log_probs else None,
                               routed_experts=out.routed_experts, num_turns=2,
                               multi_modal_data={"multi_modal_inputs": mm} if isinstance(mm, dict) and mm else None,
                               metrics=AgentLoopMetrics(generate_sequences=dt, num_preempted=out.num_preempted))
