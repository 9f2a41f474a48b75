"""Tools, interactions, scorers, request schema, samplers, tiled MLP, registry and small helpers (CPU)."""

import asyncio

import numpy as np
import pytest
import torch

from verl_b200.tools.schemas import OpenAIFunctionToolSchema, ToolResponse

_SCHEMA = OpenAIFunctionToolSchema.model_validate({
    "type": "function",
    "function": {"name": "t", "description": "d", "parameters": {"type": "object", "properties": {}, "required": []}}})


def test_geo3k_and_zoom_tools():
    from verl_b200.tools.geo3k_tool import Geo3kTool
    from verl_b200.tools.image_zoom_in_tool import ImageZoomInTool

    async def run():
        g = Geo3kTool({}, _SCHEMA)
        iid, _ = await g.create(ground_truth="12")
        resp, step, _ = await g.execute(iid, {"answer": "12"})
        assert "reward=1.0" in resp.text and step == 0.0
        _, step2, _ = await g.execute(iid, {"answer": "13"})
        assert step2 == -0.05
        await g.release(iid)

        z = ImageZoomInTool({}, _SCHEMA)
        img = np.zeros((100, 200, 3), dtype=np.uint8)
        iid, _ = await z.create(image=img)
        r, _, meta = await z.execute(iid, {"bbox_2d": [10, 10, 110, 60], "label": "x"})
        assert meta["success"] and r.image[0].shape == (50, 100, 3)
        r, pen, meta = await z.execute(iid, {"bbox_2d": [50, 50, 40, 40]})
        assert not meta["success"] and pen < 0
        r, _, meta = await z.execute(iid, {"bbox_2d": [50, 50, 52, 52]})  # tiny box grows to the minimum size
        assert meta["success"] and min(r.image[0].shape[:2]) >= 28

    asyncio.run(run())


def test_mcp_tool_with_injected_client():
    from verl_b200.tools import mcp_base_tool as m

    async def run():
        calls = []

        async def fake(name, params, timeout):
            calls.append((name, params))
            return {"hits": [1, 2]}

        await m.ClientManager.initialize(rate_limit=100, call_tool=fake)
        tool = m.MCPBaseTool({"timeout": 1}, _SCHEMA)
        iid, _ = await tool.create()
        r, _, meta = await tool.execute(iid, {"q": "x"})
        assert meta["status"] == "success" and "hits" in r.text and calls == [("t", {"q": "x"})]

        async def boom(name, params, timeout):
            raise RuntimeError("down")

        await m.ClientManager.initialize(rate_limit=100, call_tool=boom)
        r, _, meta = await tool.execute(iid, {"q": "x"})
        assert meta["status"] == "error" and "down" in r.text

    asyncio.run(run())


def test_weather_interaction():
    from verl_b200.interactions.weather_interaction import WeatherInteraction

    async def run():
        w = WeatherInteraction({})
        iid = await w.start_interaction()
        done, _, s, _ = await w.generate_response(iid, [{"role": "assistant", "content": "hello"}])
        assert not done and s == 0.0
        done, _, s, _ = await w.generate_response(iid, [{"role": "assistant", "content": "The temperature is 20°C"}])
        assert done and s == 1.0
        await w.finalize_interaction(iid)

    asyncio.run(run())


def test_prime_and_batch_scorers():
    from verl_b200.utils.reward_score import default_compute_score, math_batch, math_verify, prime_code, prime_math

    assert prime_math.compute_score("thus \\boxed{\\frac{1}{2}}", "\\frac{1}{2}")[0]
    assert not prime_math.compute_score("the answer is 7", "8")[0]
    assert prime_math.compute_score("we get 0.5", "1/2")[0]
    code = "```python\nn=int(input())\nprint(n*n)\n```"
    assert prime_code.compute_score(code, {"inputs": ["2", "3"], "outputs": ["4", "9"]})[0] == 1.0
    s, info = prime_code.compute_score(code, {"inputs": ["2", "3"], "outputs": ["4", "8"]}, continuous=True)
    assert s == 0.5 and info["passed"] == 1
    assert prime_code.compute_score("while True: pass", {"inputs": [""], "outputs": [""]}, timeout=0.5)[0] == 0.0
    assert prime_code.compute_score("def f(x):\n    return x+1", {"functional": "assert f(1) == 2"})[0] == 1.0
    assert math_batch.compute_score_batched(["a", "a"], ["\\boxed{3}", "\\boxed{4}"], ["3", "3"]) == [1.0, 0.0]
    assert math_verify.compute_score("so \\boxed{3}", "3") == 1.0
    assert default_compute_score("prime_math", "\\boxed{5}", "5") == 1.0


def test_async_rollout_request_incremental_tokenisation():
    from verl_b200.utils.tokenizer import IntTokenizer
    from verl_b200.workers.rollout.schemas import (AsyncRolloutRequest, AsyncRolloutRequestStateEnum,
                                                   FinishReasonTypeEnum)

    class Tok(IntTokenizer):
        """<role-marker> content ... per message; generation prompt = assistant marker."""

        MARK = {"system": 900, "user": 901, "assistant": 902, "tool": 903}

        def apply_chat_template(self, messages, add_generation_prompt=True, tokenize=True, **kw):
            ids = []
            for m in messages:
                c = m["content"] if isinstance(m["content"], str) else "7"
                ids += [self.MARK[m["role"]]] + self.encode(c if c[:1].isdigit() else "5 5")
            if add_generation_prompt:
                ids.append(902)
            return ids

    tok = Tok(1000)
    req = AsyncRolloutRequest.create(tok, [{"role": "user", "content": "1 2 3"}], request_id="r0", max_prompt_len=8,
                                     max_response_len=6)
    assert req.input_ids.tolist() == [901, 1, 2, 3] and req.generation_prompt_ids.tolist() == [902]
    assert req.get_generation_prompt_ids(tok) == [901, 1, 2, 3, 902]
    assert req.get_generation_prompt_ids(tok) == [901, 1, 2, 3, 902]  # not appended twice
    req.add_assistant_message(tok, "10 11", content_ids=[10, 11])
    req.add_tool_response_messages(tok, [ToolResponse(text="20")])
    req.get_generation_prompt_ids(tok)
    req.add_assistant_message(tok, "12")  # tokenised from text
    req.add_user_message(tok, "30 31")
    assert req.input_ids.tolist() == [901, 1, 2, 3, 902, 10, 11, 903, 20, 902, 12, 901, 30, 31]
    assert req.loss_mask.tolist() == [0, 0, 0, 0, 0, 1, 1, 0, 0, 0, 1, 0, 0, 0]
    assert req.position_ids.tolist() == list(range(14))
    req.finalize(tok, {"score": 1.0}, FinishReasonTypeEnum.STOP)
    assert req.state == AsyncRolloutRequestStateEnum.COMPLETED
    assert req.prompt_ids.tolist() == [901, 1, 2, 3]
    assert req.response_ids.tolist() == [902, 10, 11, 903, 20, 902] and req.response_loss_mask.tolist() == [0, 1, 1, 0, 0, 0]
    assert FinishReasonTypeEnum.from_str("tool_call") == FinishReasonTypeEnum.TOOL_CALL
    with pytest.raises(ValueError):
        FinishReasonTypeEnum.from_str("nope")


def test_curriculum_sampler_prefers_informative_prompts():
    from verl_b200.experimental.dataset import AbstractCurriculumSampler, DifficultyCurriculumSampler
    from verl_b200.protocol import DataProto

    s = DifficultyCurriculumSampler(list(range(4)), {"seed": 3, "sampler": {"floor": 0.01, "momentum": 0.0}})
    assert isinstance(s, AbstractCurriculumSampler) and len(s) == 4
    scores = torch.zeros(4, 3)
    scores[0, -1], scores[1, -1] = 1.0, 1.0  # prompts 0,1 always solved; 2,3 never solved
    batch = DataProto.from_dict({"token_level_scores": scores}, non_tensors={"index": np.arange(4)})
    s.update(batch)
    assert np.allclose(s.p, [1, 1, 0, 0])
    s.p[3] = 0.5
    draws = [i for _ in range(50) for i in s]
    assert draws.count(3) > 0.8 * len(draws)


def test_tiled_mlp_matches_plain():
    from verl_b200.models.tiled_mlp import TiledMLP

    torch.manual_seed(0)
    mlp = torch.nn.Sequential(torch.nn.Linear(8, 32), torch.nn.SiLU(), torch.nn.Linear(32, 8)).double()
    x = torch.randn(11, 8, dtype=torch.double, requires_grad=True)
    y = mlp(x)
    y.square().sum().backward()
    ref = [x.grad.clone()] + [p.grad.clone() for p in mlp.parameters()]
    x.grad = None
    mlp.zero_grad()
    y2 = TiledMLP(mlp, 3)(x)
    assert torch.allclose(y, y2)
    y2.square().sum().backward()
    got = [x.grad] + [p.grad for p in mlp.parameters()]
    for a, b in zip(ref, got):
        assert torch.allclose(a, b)


def test_registry_and_model_helpers(tmp_path):
    from verl_b200.models.registry import ModelRegistry
    from verl_b200.utils import model as mu
    from verl_b200.utils.chat_template import extract_system_prompt_and_generation

    assert "Qwen2ForCausalLM" in ModelRegistry.get_supported_archs()
    assert ModelRegistry.load_model_cls("NopeForCausalLM") is None
    assert callable(ModelRegistry.load_model_cls("Qwen3MoeForCausalLM", value=True))
    mask = torch.tensor([[0, 0, 1, 1, 1]])
    assert mu.compute_position_id_with_mask(mask).tolist() == [[0, 0, 0, 1, 2]]
    m = mu.create_random_mask(torch.zeros(4, 20, dtype=torch.long), 0.5, 0.2, 0.1)
    assert m.shape == (4, 20) and (m.sum(-1) >= 2).all() and (m.sum(-1) <= 10).all()
    t, cu, mx = mu.pad_packed_inputs(torch.arange(10), torch.tensor([0, 4, 10]), 6, 8)
    assert t.shape[0] == 16 and cu.tolist() == [0, 4, 10, 16] and mx == 6
    n, scale = mu.get_model_size(torch.nn.Linear(100, 100))
    assert scale == "K" and abs(n - 10.1) < 1e-6
    (tmp_path / "adapter_config.json").write_text('{"r": 16}')
    assert mu.get_lora_rank_from_adapter(tmp_path) == 16
    assert mu.check_target_modules({"target_modules": ["q_proj"]}, "layers.0.attn.q_proj")
    assert not mu.check_target_modules({"target_modules": "x.*"}, "layers.0.attn.q_proj")

    class Tok:
        def apply_chat_template(self, messages, add_generation_prompt=False, tokenize=True, **kw):
            ids = [1, 1]  # system prompt
            for _ in messages:
                ids += [5, 6]
            return ids + ([9] if add_generation_prompt else [])

    assert extract_system_prompt_and_generation(Tok()) == ([1, 1], [9])


def test_run_unvicorn_serves():
    import urllib.request

    from fastapi import FastAPI

    from verl_b200.workers.rollout.utils import ensure_async_iterator, get_max_position_embeddings, run_unvicorn

    app = FastAPI()

    @app.get("/ping")
    def ping():
        return {"ok": True}

    async def run():
        port, task = await run_unvicorn(app, {"a": 1}, "127.0.0.1")
        loop = asyncio.get_running_loop()
        body = await loop.run_in_executor(None, lambda: urllib.request.urlopen(f"http://127.0.0.1:{port}/ping", timeout=5).read())
        task.server.should_exit = True
        await task
        return body, [x async for x in ensure_async_iterator([1, 2])]

    body, items = asyncio.run(run())
    assert b"true" in body and items == [1, 2]

    class C:
        max_position_embeddings = None

        class text_config:
            max_position_embeddings = 77

    assert get_max_position_embeddings(C) == 77


def test_model_with_tiled_mlp_matches_plain():
    from verl_b200.models.config import preset
    from verl_b200.models.tiled_mlp import apply_tiled_mlp
    from verl_b200.models.transformer import PackedBatch, build_model
    from verl_b200.workers.engine.native import NativeEngine

    cfg = preset("tiny-qwen2")
    ids = torch.randint(3, cfg.vocab_size, (2, 12))
    pb, _ = PackedBatch.from_padded(ids, torch.ones_like(ids))
    grads, names = [], []
    for shards in (0, 3):
        m = build_model(cfg, dtype=torch.float32, seed=1)
        if shards:
            assert apply_tiled_mlp(m, shards) == cfg.num_hidden_layers
        m.forward_hidden(pb).float().square().mean().backward()
        grads.append(m.layers[0].mlp.down_proj.weight.grad.clone())
        names.append(sorted(n for n, _ in m.named_parameters()))
    assert names[0] == names[1] and torch.allclose(grads[0], grads[1], atol=1e-6)
    eng = NativeEngine(cfg, None, None, device="cpu", seed=1, trainable=False, tiled_mlp_shards=3).initialize()
    assert eng.model.layers[0].mlp.tile_shards == 3


def test_tensordict_utils_roundtrip():
    from verl_b200.utils import tensordict_utils as tu

    nested = torch.nested.as_nested_tensor([torch.arange(2), torch.arange(3), torch.arange(1), torch.arange(4)], layout=torch.jagged)
    td = tu.get_tensordict({"x": torch.arange(8).view(4, 2), "ids": nested, "turns": [[], [0.5], [1], [2, 3]]}, {"temp": 0.7})
    assert td.batch_size[0] == 4 and tu.get(td, "temp") == 0.7 and tu.get(td, "turns")[1] == [0.5]
    sel = tu.index_select_tensor_dict(td, [3, 0])
    assert sel["x"].tolist() == [[6, 7], [0, 1]] and [r.tolist() for r in sel["ids"].unbind(0)] == [[0, 1, 2, 3], [0, 1]]
    assert tu.get(sel, "turns") == [[2, 3], []] and tu.get(sel, "temp") == 0.7
    chunks = tu.chunk_tensordict(td, 2)
    tu.assert_tensordict_eq(tu.concat_tensordict(chunks), td)
    padded, pad = tu.pad_to_divisor(td, 3)
    assert pad == 2 and padded.batch_size[0] == 6
    tu.assert_tensordict_eq(tu.unpad(padded, pad), td)
    tu.assign_non_tensor(td, tags=["a", "b", "c", "d"], step=3)
    assert tu.get(td, "tags")[2] == "c" and tu.pop(td, "step") == 3 and "step" not in td
    other = tu.get_tensordict({"x": torch.arange(8).view(4, 2), "y": torch.ones(4)})
    tu.union_tensor_dict(td, other)
    assert "y" in td
    with pytest.raises(AssertionError):
        tu.union_tensor_dict(td, tu.get_tensordict({"x": torch.zeros(4, 2, dtype=torch.long)}))
    sub = tu.pop_keys(td, ["x", "y"])
    assert set(sub.keys()) == {"x", "y"} and "x" not in td
    batches = list(tu.make_iterator(other, 2, epochs=2, seed=0))
    assert len(batches) == 4 and batches[0].batch_size[0] == 2
    pos = torch.nested.as_nested_tensor([torch.zeros(5, 3), torch.zeros(7, 3)], layout=torch.jagged)
    t3 = tu.get_tensordict({"position_ids": pos})
    tu.maybe_fix_3d_position_ids(t3)
    assert [tuple(r.shape) for r in t3["position_ids"].unbind(0)] == [(3, 5), (3, 7)]


def test_misc_utils_batch(tmp_path, monkeypatch):
    from verl_b200.experimental.agent_loop.prometheus_utils import update_prometheus_config
    from verl_b200.experimental.agent_loop.utils import build_gpt_oss_tool_response_text, resolve_config_path
    from verl_b200.utils import attention_utils as au
    from verl_b200.utils import hdfs_io
    from verl_b200.utils.dataset.dataset_utils import DatasetPadMode, SFTTensorCollator
    from verl_b200.utils.dataset.vision_utils import process_image, process_video, smart_resize
    from verl_b200.utils.debug.trajectory_tracker import dump_data, get_trajectory_tracker
    from verl_b200.utils.logger import LocalLogger
    from verl_b200.utils.profiler.performance import GPUMemoryLogger, gather_timing, reduce_timing, simple_timer
    from verl_b200.utils.ray_utils import auto_await, parallel_put
    from verl_b200.utils.torch_dtypes import PrecisionType

    assert PrecisionType.to_dtype("bf16") is torch.bfloat16 and PrecisionType.to_str(torch.float16) == "fp16"
    assert PrecisionType.is_fp32(32) and PrecisionType.supported_type("mixed")

    x = torch.arange(24.).view(2, 4, 3)
    mask = torch.tensor([[1, 1, 0, 0], [1, 1, 1, 0]])
    flat, idx, cu, mx, used = au.unpad_input(x, mask)
    assert flat.shape == (5, 3) and cu.tolist() == [0, 2, 5] and mx == 3 and used.tolist() == [2, 3]
    back = au.pad_input(flat, idx, 2, 4)
    assert torch.equal(back, x * mask[..., None])

    col = SFTTensorCollator(DatasetPadMode.NO_PADDING)([{"input_ids": torch.arange(3), "n": 1}, {"input_ids": torch.arange(5), "n": 2}])
    assert col["input_ids"].is_nested and col["n"] == [1, 2]
    assert SFTTensorCollator("right")([{"a": torch.ones(2)}, {"a": torch.zeros(2)}])["a"].shape == (2, 2)

    assert smart_resize(100, 200, 28) == (112, 196)
    img = process_image(np.zeros((100, 200, 3), dtype=np.uint8))
    assert img.size == (196, 112)
    assert len(process_video({"frames": [np.zeros((56, 56, 3), dtype=np.uint8)] * 10}, nframes=4)) == 4

    monkeypatch.setenv("VERL_ENABLE_TRACKER", "1")
    monkeypatch.setenv("VERL_TRACKER_HDFS_DIR", str(tmp_path / "trk"))
    dump_data({"a": torch.ones(2)}, "step0")
    get_trajectory_tracker().wait_for_hdfs()
    assert torch.equal(torch.load(tmp_path / "trk" / "step0.pth")["a"], torch.ones(2))
    assert hdfs_io.exists(str(tmp_path / "trk")) and not hdfs_io.is_non_local(str(tmp_path))

    timing = {}
    with simple_timer("a", timing):
        pass
    assert "a" in timing and reduce_timing(timing) == timing and gather_timing(timing) == {"a": [timing["a"]]}
    logs = []
    dec = GPUMemoryLogger("role")
    dec.logging_function = logs.append
    assert dec(lambda v: v + 1)(1) == 2 and len(logs) == 2 and logs[0].startswith("Before")
    LocalLogger().log({"x": 1.0, "s": "skip"}, step=1)

    @auto_await
    async def co(v):
        return v * 2

    assert co(2) == 4 and parallel_put([1, 2]) == [1, 2]
    assert "functions.f to=assistant" in build_gpt_oss_tool_response_text([{"content": "r"}], ["f"])
    assert resolve_config_path("trainer/config/ppo_trainer.yaml").endswith("ppo_trainer.yaml")
    with pytest.raises(FileNotFoundError):
        resolve_config_path("nope/none.yaml")
    cfg = {"file": str(tmp_path / "prom" / "prometheus.yml"), "port": 1}
    assert update_prometheus_config(cfg, ["127.0.0.1:8000"], "native")
    import yaml
    assert yaml.safe_load(open(cfg["file"]))["scrape_configs"][0]["static_configs"][0]["targets"] == ["127.0.0.1:8000"]


def test_dynamic_dataset_grows(tmp_path):
    import json

    from verl_b200.experimental.dynamic_dataset import DynamicGenDataset
    from verl_b200.utils.tokenizer import IntTokenizer

    f = tmp_path / "d.jsonl"
    f.write_text("\n".join(json.dumps({"prompt": "1 2 3", "data_source": "x"}) for _ in range(3)))
    cfg = {"datagen": {"path": "verl_b200.experimental.dynamic_dataset.dynamicgen_dataset", "name": "MockDataGenerator"},
           "max_prompt_length": 8}
    ds = DynamicGenDataset(str(f), IntTokenizer(100), cfg)
    assert len(ds) == 4
    ds.on_batch_end(None)
    assert len(ds) == 5 and ds[4]["raw_prompt_ids"] == [1, 2, 3]
    with pytest.raises(AssertionError):
        DynamicGenDataset(str(f), IntTokenizer(100), {"max_prompt_length": 8})


def test_search_utils_retry_and_format(monkeypatch):
    import requests

    from verl_b200.tools.utils import search_r1_like_utils as su

    calls = {"n": 0}

    class R:
        def __init__(self, code, body):
            self.status_code, self._b = code, body

        def raise_for_status(self):
            if self.status_code >= 400:
                raise requests.exceptions.HTTPError(str(self.status_code))

        def json(self):
            return self._b

    def post(url, json=None, timeout=None, headers=None):
        calls["n"] += 1
        if calls["n"] < 3:
            return R(503, {})
        return R(200, {"result": [[{"document": {"contents": "Title A\nbody a"}}], [{"document": {"contents": "T2\nb2"}}]]})

    monkeypatch.setattr(requests, "post", post)
    text, meta = su.perform_single_search_batch("http://x", ["q1", "q2"], topk=1, retry_delay=0.0)
    assert calls["n"] == 3 and meta["status"] == "success" and meta["total_results"] == 2
    assert "Doc 1 (Title: Title A)" in text and "---" in text
    monkeypatch.setattr(requests, "post", lambda *a, **k: R(404, {}))
    resp, err = su.call_search_api("http://x", ["q"], retry_delay=0.0)
    assert resp is None and "API Request Error" in err
    monkeypatch.setattr(requests, "post", lambda *a, **k: R(200, {"result": []}))
    assert su.perform_single_search_batch("http://x", ["q"])[1]["status"] == "no_results"


def test_rollout_tokenizer_adapter():
    from verl_b200.utils.tokenizer import IntTokenizer
    from verl_b200.workers.rollout.tokenizer import HybridEngineBaseTokenizer, TokenizerAdapter

    t = TokenizerAdapter(IntTokenizer(100, eos_token_id=2, pad_token_id=0))
    assert isinstance(t, HybridEngineBaseTokenizer) and t.vocab_size == 100 and sorted(t.all_special_ids) == [0, 2]
    assert t.encode("5 6 7") == [5, 6, 7] and t.decode([5, 2, 6], skip_special_tokens=True) == "5 6"
    assert t.convert_ids_to_tokens([5, 2], skip_special_tokens=True) == ["5"] and t.convert_tokens_to_string(["a", "b"]) == "a b"


def test_mcp_search_parse_weight_keys_and_sharding_manager():
    from verl_b200.protocol import DataProto
    from verl_b200.tools.mcp_base_tool import MCPSearchTool
    from verl_b200.utils.model import convert_weight_keys, extract_multi_modal_inputs
    from verl_b200.workers.sharding_manager import FSDPUlyssesShardingManager

    tool = MCPSearchTool({}, _SCHEMA)
    text, meta = tool._parse_tool_result([{"text": '{"query": "q", "results": ["a", "b"]}'}, {"text": "plain"}, {"image": 1}])
    assert text == "a\nb\nplain" and meta["query_count"] == 1 and meta["total_results"] == 3
    assert tool._parse_tool_result([])[0] == "no search result."
    sd = convert_weight_keys({"module._fsdp_wrapped_module.layers.0.w": 1, "base_model.model.lm_head.weight": 2, "x": 3})
    assert sd == {"layers.0.w": 1, "lm_head.weight": 2, "x": 3}
    mm = extract_multi_modal_inputs([{"pixel_values": torch.ones(2, 3)}, {}, {"pixel_values": torch.zeros(1, 3)}], indices=[0, 2])
    assert mm["pixel_values"].shape == (3, 3)
    mgr = FSDPUlyssesShardingManager(None)  # no sequence parallelism: a pass-through
    d = DataProto.from_dict({"x": torch.arange(4)})
    with mgr:
        assert mgr.postprocess_data(mgr.preprocess_data(d)) is d


def test_hf_rollout_greedy_matches_paged_engine_and_honours_sampling_modes():
    import torch

    from verl_b200 import DataProto
    from verl_b200.models import CausalLM, preset
    from verl_b200.rollout import NativeRolloutEngine, SamplingParams
    from verl_b200.workers.rollout.base import get_rollout_class

    cfg = preset("tiny-qwen2")
    model = CausalLM(cfg, dtype=torch.float32).init_weights(2)
    HF = get_rollout_class("hf", "sync")
    ro = HF(model, {"response_length": 6, "micro_batch_size": 2, "do_sample": True, "temperature": 1.0, "top_k": 0, "top_p": 0.9,
                    "val_kwargs": {"temperature": 0.0001, "top_k": 1, "top_p": 1.0}}, model_config=cfg)
    g = torch.Generator().manual_seed(0)
    lens = [5, 8, 3, 8]
    ids = torch.zeros(4, 8, dtype=torch.long)
    mask = torch.zeros(4, 8, dtype=torch.long)
    for i, n in enumerate(lens):  # left padding
        ids[i, 8 - n:] = torch.randint(3, 2000, (n,), generator=g)
        mask[i, 8 - n:] = 1
    batch = DataProto.from_dict({"input_ids": ids, "attention_mask": mask, "position_ids": (mask.cumsum(-1) - 1).clamp(min=0)},
                                meta_info={"eos_token_id": 2, "pad_token_id": 0, "do_sample": False})
    out = ro.generate_sequences(batch)
    assert out.batch["responses"].shape == (4, 6) and out.batch["input_ids"].shape == (4, 14)
    eng = NativeRolloutEngine(model, max_num_seqs=4, max_model_len=32, max_num_batched_tokens=64, num_blocks=32)
    ref = eng.generate([ids[i][mask[i].bool()].tolist() for i in range(4)], SamplingParams(temperature=0.0, max_tokens=6))
    for i, o in enumerate(ref):
        n = len(o.token_ids)
        assert out.batch["responses"][i, :n].tolist() == o.token_ids
        assert int(out.batch["response_mask"][i].sum()) == n
    # validation sampling with top_k = 1 is greedy as well; plain sampling stays inside the top-p nucleus (finite lps)
    batch.meta_info.update({"do_sample": True, "validate": True})
    assert torch.equal(ro.generate_sequences(batch).batch["responses"], out.batch["responses"])
    batch.meta_info.update({"validate": False, "num_return_sequences": 2})
    s = ro.generate_sequences(batch)
    assert len(s) == 8 and torch.isfinite(s.batch["rollout_log_probs"]).all()
