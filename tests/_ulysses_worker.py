"""Child of tests/test_ulysses_on_cpu.py: 2 gloo ranks, one decoder layer with and without Ulysses SP."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    dist.init_process_group("gloo")
    rank, sp = dist.get_rank(), dist.get_world_size()
    from verl_b200.models import preset
    from verl_b200.models.transformer import CausalLM, PackedBatch
    from verl_b200.utils import ulysses as U

    cfg = preset("tiny-qwen2")
    torch.manual_seed(0)
    model = CausalLM(cfg, dtype=torch.float32, device="cpu")
    model.init_weights(1)
    lens = [13, 7, 11]  # 31 tokens: not a multiple of 2 -> padding path
    T = sum(lens)
    ids = torch.randint(0, cfg.vocab_size, (T,), generator=torch.Generator().manual_seed(5))
    cu = torch.tensor([0, 13, 20, 31], dtype=torch.int32)
    pos = torch.cat([torch.arange(n) for n in lens])
    rope = model.rope(torch.device("cpu"))
    layer = model.layers[0]

    # reference: whole sequence on one rank
    x_full = model.embed_tokens(ids).detach().requires_grad_(True)
    full = PackedBatch(ids, pos, cu, max(lens))
    h_ref, r_ref = layer(x_full, None, full, rope)
    (h_ref + r_ref).pow(2).sum().backward()
    g_ref = x_full.grad.clone()
    gw_ref = layer.self_attn.qkv_proj.weight.grad.clone()
    layer.zero_grad()

    # Ulysses: every rank holds a slice of the tokens
    U.set_ulysses_sequence_parallel_group(dist.group.WORLD)
    U.validate_ulysses_config(cfg.num_attention_heads, sp)
    layer.self_attn.sp_group = dist.group.WORLD
    ids_l, pos_l, pad = U.ulysses_pad_and_slice_inputs(ids, pos, sp)
    n_l = ids_l.shape[0]
    x_pad, _ = U.ulysses_pad(model.embed_tokens(ids).detach(), 0, sp)
    x_l = x_pad[rank * n_l : (rank + 1) * n_l].clone().requires_grad_(True)
    local = PackedBatch(ids_l, pos_l, cu, max(lens), total_tokens=T)
    h_l, r_l = layer(x_l, None, local, rope)
    out = U.gather_outputs_and_unpad(h_l + r_l, 0, 0, pad, grad_scaler=False)
    torch.testing.assert_close(out, (h_ref + r_ref).detach(), atol=1e-4, rtol=1e-4)
    # loss over the tokens this rank owns (padding excluded); weight grads then add up over ranks
    own = torch.arange(rank * n_l, (rank + 1) * n_l) < T
    ((h_l + r_l)[own]).pow(2).sum().backward()
    torch.testing.assert_close(x_l.grad[own], g_ref[rank * n_l : (rank + 1) * n_l][: int(own.sum())], atol=1e-4, rtol=1e-4)
    gw = layer.self_attn.qkv_proj.weight.grad.clone()
    dist.all_reduce(gw)
    torch.testing.assert_close(gw, gw_ref, atol=1e-3, rtol=1e-3)
    layer.self_attn.sp_group = None
    U.set_ulysses_sequence_parallel_group(None)

    # engine level: sp = 2 over the two ranks (dp = 1) against a single-rank engine on the same batch
    from verl_b200.workers.engine.native import NativeEngine

    class C(dict):
        __getattr__ = dict.get

    optim = C(lr=1e-2, clip_grad=1.0, weight_decay=0.0)
    rows = torch.tensor([i for i in range(T) if i not in (12, 19, 30)])  # not the last token of a sequence
    labels = ids[rows + 1]
    results = []
    for sp_size in (2, 1):
        if sp_size == 1:
            is_init = dist.is_initialized
            dist.is_initialized = lambda: False  # build a world-size-1 engine inside this process
        eng = NativeEngine(cfg, C(ulysses_sequence_parallel_size=sp_size), optim, device="cpu",
                           group=dist.group.WORLD if sp_size > 1 else None, seed=4).initialize()
        if sp_size == 1:
            dist.is_initialized = is_init
        assert eng.get_data_parallel_size() == 1
        with eng.train_mode():
            eng.optimizer_zero_grad()
            lp, ent = eng.forward_logprob(full, rows, labels, 1.0)
            (-(lp.sum()) / rows.numel()).backward()
            gn = eng.optimizer_step()
        results.append((lp.detach().clone(), ent.detach().clone(), float(gn)))
    (lp2, ent2, gn2), (lp1, ent1, gn1) = results
    torch.testing.assert_close(lp2, lp1, atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(ent2, ent1, atol=1e-4, rtol=1e-4)
    assert abs(gn2 - gn1) < 1e-3 * max(1.0, gn1), (gn2, gn1)
    # sharding-manager interface: the group's shares are gathered before, and split again after, the computation
    from verl_b200.protocol import DataProto
    from verl_b200.workers.sharding_manager import FSDPUlyssesShardingManager

    mgr = FSDPUlyssesShardingManager(dist.group.WORLD)
    mine = DataProto.from_dict({"x": torch.arange(3) + 10 * rank})
    with mgr:
        assert U.get_ulysses_sequence_parallel_group() is dist.group.WORLD
        both = mgr.preprocess_data(mine)
        assert both.batch["x"].tolist() == [0, 1, 2, 10, 11, 12]
        back = mgr.postprocess_data(both)
        assert back.batch["x"].tolist() == [10 * rank, 10 * rank + 1, 10 * rank + 2]
    assert U.get_ulysses_sequence_parallel_group() is None
    if rank == 0:
        print("ULYSSES_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
