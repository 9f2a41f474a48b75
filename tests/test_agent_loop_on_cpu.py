"""Async server, abort semantics and agent loops (single turn + tool calling) against the native engine on CPU."""
import asyncio
import json

import numpy as np
import pytest
import torch

from verl_b200 import DataProto
from verl_b200.experimental.agent_loop import AgentLoopManager, AsyncLLMServerManager
from verl_b200.experimental.agent_loop.tool_parser import HermesToolParser
from verl_b200.models import build_model, preset
from verl_b200.rollout import NativeRolloutEngine
from verl_b200.utils.config import compose
from verl_b200.utils.tokenizer import IntTokenizer
from verl_b200.workers.rollout.async_server import NativeAsyncServer


@pytest.fixture(scope="module")
def server():
    torch.manual_seed(0)
    m = build_model(preset("tiny-qwen2"), dtype=torch.float32)
    eng = NativeRolloutEngine(m, max_num_seqs=8, max_model_len=160, max_num_batched_tokens=128, num_blocks=96)
    s = NativeAsyncServer(eng, response_length=32, prompt_length=64)
    yield s
    s.shutdown()


def _cfg(extra=()):
    return compose("ppo_trainer", ["actor_rollout_ref.model.path=preset:tiny-qwen2", "data.max_prompt_length=64",
                                   "data.max_response_length=32", "actor_rollout_ref.rollout.agent.num_workers=2"] + list(extra))


def test_generate_and_abort(server):
    async def go():
        fut = [server.generate(list(range(10, 30)), {"temperature": 0.0, "max_tokens": 8}) for _ in range(3)]
        outs = await asyncio.gather(*fut)
        assert all(len(o.token_ids) == 8 and o.stop_reason in ("length", "completed") for o in outs)
        assert outs[0].token_ids == outs[1].token_ids  # greedy
        long = asyncio.ensure_future(server.generate(list(range(10, 40)), {"temperature": 1.0, "max_tokens": 100}, request_id="victim"))
        await asyncio.sleep(0.05)
        res = await server.abort_all_requests()
        out = await long
        assert out.stop_reason == "aborted" and len(out.token_ids) < 100 and "victim" in res["request_ids"]

    asyncio.run(go())


def test_load_balancer_is_sticky_and_least_loaded():
    class H:
        def __init__(self, i):
            self.i, self.calls = i, 0

        async def generate(self, **kw):
            self.calls += 1
            return self.i

    hs = [H(i) for i in range(3)]
    mgr = AsyncLLMServerManager(None, hs)

    async def go():
        first = await mgr.generate("conv", prompt_ids=[1], sampling_params={})
        again = await mgr.generate("conv", prompt_ids=[1, 2], sampling_params={})
        assert first == again
        for k in range(6):
            await mgr.generate(f"r{k}", prompt_ids=[1], sampling_params={})
        # 7 distinct conversations over 3 servers: assignments differ by at most one (the sticky call adds one more)
        assert sum(h.calls for h in hs) == 8 and min(h.calls for h in hs) >= 2

    asyncio.run(go())


def test_single_turn_agent_loop_batch(server):
    cfg = _cfg()
    tok = IntTokenizer(2048)
    mgr = AgentLoopManager(cfg, server_handles=[server], tokenizer=tok)
    prompts = np.empty(5, dtype=object)
    prompts[:] = [list(range(20, 20 + n)) for n in (12, 30, 7, 18, 25)]
    batch = DataProto.from_dict(tensors={"dummy": torch.zeros(5)}, non_tensors={"raw_prompt": prompts})
    out = mgr.generate_sequences(batch)
    assert out.batch["prompts"].shape == (5, 64) and out.batch["responses"].shape == (5, 32)
    assert out.batch["input_ids"].shape == (5, 96)
    assert (out.batch["attention_mask"][:, :64].sum(-1) == torch.tensor([12, 30, 7, 18, 25])).all()
    assert (out.batch["prompts"][1, -30:] == torch.arange(20, 50)).all()
    assert "rollout_log_probs" in out.batch.keys() and "agent_loop/generate_sequences/mean" in out.meta_info["timing"]
    assert (out.non_tensor_batch["__num_turns__"] == 2).all()


class _Tok(IntTokenizer):
    """Integer tokenizer whose decode can be made to contain a tool call."""

    def decode(self, ids, skip_special_tokens=True):
        ids = [int(t) for t in ids]
        if getattr(self, "emit_call", 0) > 0 and ids:
            self.emit_call -= 1
            return '<tool_call>{"name": "echo", "arguments": {"text": "hi"}}</tool_call>'
        return super().decode(ids, skip_special_tokens)


def test_tool_agent_loop_masks_tool_tokens(server, tmp_path):
    tools_yaml = tmp_path / "tools.yaml"
    tools_yaml.write_text(json.dumps({"tools": [{
        "class_name": "tests_tool_helpers.EchoTool", "config": {"type": "native"},
        "tool_schema": {"type": "function", "function": {"name": "echo", "description": "echo",
                                                         "parameters": {"type": "object", "properties": {"text": {"type": "string"}}, "required": ["text"]}}}}]}))
    import sys
    import types

    from verl_b200.tools import BaseTool, ToolResponse

    mod = types.ModuleType("tests_tool_helpers")

    class EchoTool(BaseTool):
        async def execute(self, instance_id, parameters, **kw):
            return ToolResponse(text="7 8 9"), 0.5, {}

    mod.EchoTool = EchoTool
    sys.modules["tests_tool_helpers"] = mod
    cfg = _cfg([f"actor_rollout_ref.rollout.multi_turn.tool_config_path={tools_yaml}",
                "actor_rollout_ref.rollout.multi_turn.max_assistant_turns=3",
                "actor_rollout_ref.rollout.agent.default_agent_loop=tool_agent", "actor_rollout_ref.rollout.agent.num_workers=1"])
    tok = _Tok(2048)
    tok.emit_call = 1
    mgr = AgentLoopManager(cfg, server_handles=[server], tokenizer=tok)
    prompts = np.empty(1, dtype=object)
    prompts[:] = [[{"role": "user", "content": "30 31 32 33"}]]
    batch = DataProto.from_dict(tensors={"dummy": torch.zeros(1)}, non_tensors={"raw_prompt": prompts})
    # make the first assistant turn one token long: greedy decoding, and that token is declared EOS
    first = asyncio.run(server.generate([30, 31, 32, 33], {"temperature": 0.0, "max_tokens": 1})).token_ids[0]
    old_eos, server.engine.eos = server.engine.eos, first
    batch.meta_info["validate"] = True
    try:
        out = mgr.generate_sequences(batch)
    finally:
        server.engine.eos = old_eos
    rm, am = out.batch["response_mask"][0], out.batch["attention_mask"][0, 64:]
    assert am.sum() > rm.sum() > 0  # some response tokens are tool tokens (mask 0)
    assert int(out.non_tensor_batch["__num_turns__"][0]) >= 3
    assert out.non_tensor_batch["tool_rewards"][0] == [0.5]


def test_hermes_parser():
    class T:
        def decode(self, ids, **kw):
            return 'think <tool_call>{"name": "f", "arguments": {"a": 1}}</tool_call> and <tool_call>not json</tool_call>'

    text, calls = asyncio.run(HermesToolParser(T()).extract_tool_calls([1]))
    assert len(calls) == 1 and calls[0].name == "f" and json.loads(calls[0].arguments) == {"a": 1}
    assert "<tool_call>" not in text


def test_partial_single_turn_loop_resumes_cancelled_sample(server):
    """A sample cut by abort_all_requests comes back cancelled; running it again continues where it stopped."""
    from verl_b200.experimental.fully_async_policy.agent_loop import PartialSingleTurnAgentLoop

    cfg = _cfg()

    async def go():
        loop = PartialSingleTurnAgentLoop(cfg, AsyncLLMServerManager(cfg, [server]), IntTokenizer(2048))
        sp = {"temperature": 0.0, "max_tokens": 32, "ignore_eos": True}
        prompt = list(range(30, 50))
        full = await loop.run(sp, raw_prompt=prompt, param_version=1)
        assert not full.extra_fields["is_cancel"]
        task = asyncio.ensure_future(loop.run(sp, raw_prompt=prompt, param_version=1))
        while not server._pending:
            await asyncio.sleep(0.001)
        await asyncio.sleep(0.02)
        await server.abort_all_requests(reset_prefix_cache=False)
        part = await task
        if not part.extra_fields["is_cancel"]:  # the engine finished before the abort landed: nothing to resume
            assert part.response_ids == full.response_ids
            return
        assert len(part.response_ids) < len(full.response_ids)
        resumed = await loop.run(sp, raw_prompt=prompt, output=part, param_version=2)
        assert not resumed.extra_fields["is_cancel"]
        assert resumed.extra_fields["param_version_start"] == 1 and resumed.extra_fields["param_version_end"] == 2
        assert resumed.prompt_ids == prompt and resumed.response_ids == full.response_ids  # greedy: same continuation
        assert len(resumed.response_logprobs) == len(resumed.response_ids)
        assert (await loop.run(sp, raw_prompt=prompt, output=resumed)) is resumed

    asyncio.run(go())


def test_partial_tool_agent_loop_resumes_inside_a_turn(tmp_path):
    """An assistant turn cut by an abort continues in the next run; the tool call spanning both generations is
    parsed from the whole turn, the tool's tokens are masked, and the loop then finishes normally."""
    import sys
    import types

    from verl_b200.experimental.fully_async_policy.agent_loop import PartialToolAgentLoop
    from verl_b200.tools import BaseTool, ToolResponse

    mod = types.ModuleType("tests_tool_helpers2")

    class EchoTool(BaseTool):
        async def execute(self, instance_id, parameters, **kw):
            return ToolResponse(text="7 8 9"), 0.25, {}

    mod.EchoTool = EchoTool
    sys.modules["tests_tool_helpers2"] = mod
    tools_yaml = tmp_path / "tools.yaml"
    tools_yaml.write_text(json.dumps({"tools": [{
        "class_name": "tests_tool_helpers2.EchoTool", "config": {"type": "native"},
        "tool_schema": {"type": "function", "function": {"name": "echo", "description": "echo",
                                                         "parameters": {"type": "object", "properties": {"text": {"type": "string"}}, "required": ["text"]}}}}]}))
    cfg = _cfg([f"actor_rollout_ref.rollout.multi_turn.tool_config_path={tools_yaml}",
                "actor_rollout_ref.rollout.multi_turn.max_assistant_turns=4"])

    class Tok(IntTokenizer):
        def decode(self, ids, skip_special_tokens=True):
            ids = [int(t) for t in ids]
            if ids == [101, 102, 103]:  # only the complete turn spells the call
                return '<tool_call>{"name": "echo", "arguments": {"text": "hi"}}</tool_call>'
            return super().decode(ids, skip_special_tokens)

    class FakeServers:
        def __init__(self):
            self.script = [([101, 102], [-0.1, -0.2], True), ([103], [-0.3], False), ([104], [-0.4], False)]
            self.prompts = []

        async def generate_for_partial(self, request_id, *, prompt_ids, sampling_params, **kw):
            self.prompts.append(list(prompt_ids))
            return self.script.pop(0)

    async def go():
        servers = FakeServers()
        loop = PartialToolAgentLoop(cfg, servers, Tok(2048))
        sp = {"temperature": 0.0}
        part = await loop.run(sp, raw_prompt=[{"role": "user", "content": "30 31"}], param_version=3)
        assert part.extra_fields["is_cancel"] and part.response_ids == [101, 102] and part.response_mask == [1, 1]
        done = await loop.run(sp, raw_prompt=None, output=part, param_version=4)
        assert not done.extra_fields["is_cancel"]
        assert done.extra_fields["param_version_start"] == 3 and done.extra_fields["param_version_end"] == 4
        # second generation continued the cut turn from prompt + partial response
        assert servers.prompts[1] == servers.prompts[0] + [101, 102]
        ids, mask = done.response_ids, done.response_mask
        assert ids[:3] == [101, 102, 103] and ids[-1] == 104 and mask[:3] == [1, 1, 1] and mask[-1] == 1
        tool = ids[3:-1]
        assert 7 in tool and 8 in tool and 9 in tool and set(mask[3:-1]) == {0}
        assert done.extra_fields["tool_rewards"] == [0.25] and len(done.response_logprobs) == len(ids)
        assert done.num_turns == 4  # user, assistant (in two pieces), tool, assistant
        assert (await loop.run(sp, raw_prompt=None, output=done)) is done

    asyncio.run(go())


def test_fully_async_manager_cancels_and_resumes_groups(server):
    """Prompt groups driven through the fully-async manager: a cancel in mid-generation leaves cancelled outputs,
    the groups continue after resume, and (greedy) end with the same tokens as an undisturbed run."""
    from verl_b200.experimental.fully_async_policy.agent_loop import FullyAsyncAgentLoopManager

    cfg = _cfg(["actor_rollout_ref.rollout.agent.num_workers=2"])
    tok = IntTokenizer(2048)
    mgr = FullyAsyncAgentLoopManager(cfg, server_handles=[server], tokenizer=tok)

    def group(seed, n=2):
        p = np.empty(n, dtype=object)
        p[:] = [list(range(40 + seed, 60 + seed))] * n
        d = DataProto.from_dict(tensors={"dummy": torch.zeros(n)}, non_tensors={"raw_prompt": p})
        d.meta_info["validate"] = True  # greedy
        return d

    groups = [group(s) for s in range(3)]

    async def drive(g, version_box, log):
        outs, cancelled = await mgr.generate_single_sample_async(g, None, version_box[0])
        while cancelled:
            log.append(sum(o.extra_fields["is_cancel"] for o in outs))
            await mgr.wait_resumed()
            outs, cancelled = await mgr.generate_single_sample_async(g, outs, version_box[0])
        return mgr.postprocess(outs), outs

    async def go():
        ref = [await drive(g, [0], []) for g in groups]  # undisturbed
        version, log = [0], []
        tasks = [asyncio.ensure_future(drive(g, version, log)) for g in groups]
        while not server._pending:
            await asyncio.sleep(0.001)
        await asyncio.sleep(0.02)
        await mgr.cancel()
        version[0] = 1  # "weights updated"
        await asyncio.sleep(0.01)
        pending_after_cancel = sum(not t.done() for t in tasks)  # cancelled groups wait for resume
        await mgr.resume()
        done = await asyncio.gather(*tasks)
        assert pending_after_cancel >= (1 if log else 0)
        return ref, done, log

    ref, done, log = asyncio.run(go())
    for (rb, _), (db, douts) in zip(ref, done):
        assert torch.equal(rb.batch["responses"], db.batch["responses"])
        assert torch.equal(rb.batch["response_mask"], db.batch["response_mask"])
        assert db.batch["responses"].shape == (2, 32) and "agent_data" not in db.non_tensor_batch
    if log:  # the cancel landed while requests were in flight: those samples span two parameter versions
        spans = [(o.extra_fields["param_version_start"], o.extra_fields["param_version_end"]) for _, outs in done for o in outs]
        assert (0, 1) in spans
