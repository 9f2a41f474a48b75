

def test_flops_counter_architectures():
    """Analytical FLOPs per architecture family (reference: verl/utils/flops_counter.py; tests/utils/test_flops_counter.py
    checks the same families against hand-computed values)."""
    from types import SimpleNamespace as NS

    from verl_b200.models import preset
    from verl_b200.utils.flops_counter import FlopsCounter

    # dense: 6 * params * tokens + 12 * sum(s^2) * q_size * layers, computed by hand for a small config
    c = NS(model_type="llama", hidden_size=64, num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=3,
           intermediate_size=128, vocab_size=1000)
    per_layer = 64 * 128 * 3 + 64 * (64 + 2 * 32 + 64)
    want = 6 * (per_layer * 3 + 1000 * 64 * 2) * 30 + 12 * (10 * 10 + 20 * 20) * 64 * 3
    got, peak = FlopsCounter(c).estimate_flops([10, 20], 2.0)
    assert abs(got * 1e12 * 2.0 - want) < 1e-3 * want and peak > 0
    # Apertus: two MLP matrices instead of three
    a = NS(**{**vars(c), "model_type": "apertus"})
    assert FlopsCounter(a).estimate_flops([10, 20], 1.0)[0] < FlopsCounter(c).estimate_flops([10, 20], 1.0)[0]
    # sliding-window layers cost less than full attention once sequences are longer than the window
    g = NS(**{**vars(c), "model_type": "gemma3_text", "head_dim": 16, "sliding_window": 8, "sliding_window_pattern": 3})
    full = NS(**{**vars(g), "sliding_window": None})
    assert FlopsCounter(g).estimate_flops([64], 1.0)[0] < FlopsCounter(full).estimate_flops([64], 1.0)[0]
    assert FlopsCounter(g).estimate_flops([4], 1.0)[0] == FlopsCounter(full).estimate_flops([4], 1.0)[0]
    # DeepSeek-V3: ~37 B active parameters per token
    ds = NS(model_type="deepseek_v3", hidden_size=7168, num_attention_heads=128, num_hidden_layers=61, q_lora_rank=1536,
            kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, first_k_dense_replace=3,
            moe_layer_freq=1, num_experts_per_tok=8, n_shared_experts=1, n_routed_experts=256, moe_intermediate_size=2048,
            intermediate_size=18432, vocab_size=129280)
    f1 = FlopsCounter(ds).estimate_flops([1], 1.0)[0] * 1e12 / 6
    assert 36e9 < f1 < 39e9
    # GPT-OSS: experts counted by the number a token is routed to
    o = NS(model_type="gpt_oss", hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
           num_hidden_layers=2, intermediate_size=64, num_local_experts=8, num_experts_per_tok=2, vocab_size=1000,
           sliding_window=4, layer_types=["sliding_attention", "full_attention"])
    o4 = NS(**{**vars(o), "num_experts_per_tok": 4})
    assert FlopsCounter(o4).estimate_flops([16], 1.0)[0] > FlopsCounter(o).estimate_flops([16], 1.0)[0]
    # VL: the vision tower adds work in proportion to the image patches
    v = preset("tiny-qwen2-vl")
    base = FlopsCounter(v).estimate_flops([64], 1.0)[0]
    assert FlopsCounter(v).estimate_flops([64], 1.0, images_seqlens=[16, 64])[0] > base > 0
    # MoE preset and an unknown type
    assert FlopsCounter(preset("tiny-qwen3-moe")).estimate_flops([32], 1.0)[0] > 0
    assert FlopsCounter(NS(model_type="not-a-model")).estimate_flops([32], 1.0)[0] == 0.0


def test_guard_bands_catch_writes_outside_an_allocation():
    """Canary bands around allocations: a write past either edge is reported, writes inside are not."""
    import pytest
    import torch

    from verl_b200.utils.debug.guard_bands import GuardError, guard_allocations

    with guard_allocations("cpu") as g:
        a = torch.empty(10, 3, dtype=torch.float32, device="cpu")
        b = torch.zeros_like(a)
        c = torch.zeros((4,), dtype=torch.int64, device="cpu")
        a.fill_(1.0)
        b.copy_(a)
        c += 7
        assert g.check() == 3 and float(b.sum()) == 30.0 and a.shape == (10, 3) and int(c.sum()) == 28
    assert torch.empty(2).shape == (2,)  # the torch functions are restored
    with pytest.raises(GuardError, match="past the end"):
        with guard_allocations("cpu"):
            a = torch.empty(8, dtype=torch.float32, device="cpu")
            torch.as_strided(a, (9,), (1,)).fill_(0.0)  # a "kernel" that writes one element too many
    with pytest.raises(GuardError, match="before the start"):
        with guard_allocations("cpu") as g:
            a = torch.empty(8, dtype=torch.float32, device="cpu")
            base = g.allocs[0][0]
            base[g.band - 1] = 0
    # requests the guard does not handle fall through to torch
    with guard_allocations("cpu") as g:
        torch.empty(4, device="meta")
        torch.empty(4, device="cpu", pin_memory=False)
        assert g.count == 1


def test_server_adapter_generates_batches_on_the_attached_engine():
    """The rollout backend object (registry names of the reference's engines resolve to it) runs batch generation
    itself: greedy outputs equal the argmax continuation of the same model."""
    import torch

    from verl_b200 import DataProto
    from verl_b200.models import CausalLM, PackedBatch, preset
    from verl_b200.rollout import NativeRolloutEngine
    from verl_b200.workers.rollout.base import get_rollout_class

    cfg = preset("tiny-qwen2")
    model = CausalLM(cfg, dtype=torch.float32).init_weights(0)
    eng = NativeRolloutEngine(model, max_num_seqs=4, max_model_len=48, max_num_batched_tokens=64, num_blocks=32)
    adapter = get_rollout_class("vllm", "async")({"response_length": 5, "ignore_eos": True}, cfg)
    adapter.attach(eng)
    ids = torch.randint(5, 2000, (3, 10), generator=torch.Generator().manual_seed(0))
    mask = torch.ones(3, 10, dtype=torch.long)
    mask[0, :4] = 0
    out = adapter.generate_sequences(DataProto.from_dict({"input_ids": ids, "attention_mask": mask}, meta_info={"do_sample": False}))
    assert out.batch["responses"].shape == (3, 5) and out.batch["input_ids"].shape == (3, 15)
    for b in range(3):
        seq = out.batch["input_ids"][b][out.batch["attention_mask"][b].bool()]
        n = seq.numel()
        with torch.no_grad():
            logits = model(PackedBatch(seq, torch.arange(n), torch.tensor([0, n], dtype=torch.int32), n))
        assert logits[n - 6 : n - 1].argmax(-1).tolist() == out.batch["responses"][b].tolist()


def test_jitter_flavour_of_the_native_library_builds_and_loads():
    """``VERL_B200_JITTER=1`` selects the race-hunting build (``-DVB_JITTER=1``): it is a separate shared object with the
    same C ABI; host-side entry points (the scheduler) work through it."""
    import os
    import subprocess
    import sys

    code = ("from verl_b200.ops import _lib; lib = _lib.load(); assert str(_lib._LIB_PATH).endswith('libverl_b200_jitter.so');"
            "assert lib.vb_abi_version() == 1;"
            "from verl_b200.rollout.engine import Scheduler; s = Scheduler(16, 16, 4, 64, 64); assert s.add(0, [1, 2, 3], 4) == 0;"
            "print('JITTER_OK')")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600,
                       env={**os.environ, "VERL_B200_JITTER": "1"}, cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0 and "JITTER_OK" in r.stdout, (r.stdout[-500:], r.stderr[-2000:])
