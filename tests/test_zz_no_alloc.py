"""The allocation-free fused lm_head entry point, called through its exported C symbol.

Collected last on purpose: it has to pass alone and after every other GPU test has used the device.
"""

import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "verl_b200", "lib", "libverl_b200.so")


def _lib():
    lib = ctypes.CDLL(_LIB)
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.vb_lmhead_logprob_fwd_static.argtypes = [P, P, P, I, I, I, F, P, P, P, P, P, P]
    lib.vb_lmhead_logprob_fwd_static.restype = I
    lib.vb_lmhead_logprob_fwd.argtypes = [P, P, P, I, I, I, F, P, P, P, P, P, P, P]
    lib.vb_lmhead_logprob_fwd.restype = I
    lib.vb_lmhead_num_splits.argtypes = [I, I]
    lib.vb_lmhead_num_splits.restype = I
    lib.vb_lmhead_static_scratch_floats.argtypes = []
    lib.vb_lmhead_static_scratch_floats.restype = I
    return lib


def test_static_scratch_matches_existing_entry_point_twice():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    lib = _lib()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    for call, (T, H, V, temp) in enumerate([(777, 512, 32000, 0.8), (1500, 1024, 50304, 1.0)]):
        torch.manual_seed(100 + call)
        hidden = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
        weight = (torch.randn(V, H, device=dev) * 0.05).bfloat16()
        labels = torch.randint(0, V, (T,), device=dev)
        splits = lib.vb_lmhead_num_splits(T, V)
        assert T * splits * 4 <= lib.vb_lmhead_static_scratch_floats()
        scratch = torch.empty(T * splits * 4, dtype=torch.float32, device=dev)
        ref = [torch.empty(T, dtype=torch.float32, device=dev) for _ in range(4)]
        got = [torch.full((T,), float("nan"), dtype=torch.float32, device=dev) for _ in range(4)]
        rc = lib.vb_lmhead_logprob_fwd(hidden.data_ptr(), weight.data_ptr(), labels.data_ptr(), T, H, V, 1.0 / temp,
                                       scratch.data_ptr(), *[t.data_ptr() for t in ref], status.data_ptr(), stream)
        assert rc == 0
        rc = lib.vb_lmhead_logprob_fwd_static(hidden.data_ptr(), weight.data_ptr(), labels.data_ptr(), T, H, V,
                                              1.0 / temp, *[t.data_ptr() for t in got], status.data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert status.tolist()[0] == 0
        for g, r in zip(got, ref):
            assert torch.equal(g, r)
        # and against plain fp32 PyTorch
        logits = (hidden.float() @ weight.float().t()) / temp
        lp = torch.log_softmax(logits, -1)
        torch.testing.assert_close(got[0], lp.gather(1, labels[:, None])[:, 0], atol=2e-3, rtol=2e-3)
        torch.testing.assert_close(got[1], -(lp.exp() * lp).sum(-1), atol=2e-3, rtol=2e-3)


def test_static_scratch_rejects_oversize():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    lib = _lib()
    T, V = 400000, 152064
    assert T * lib.vb_lmhead_num_splits(T, V) * 4 > lib.vb_lmhead_static_scratch_floats()
    # refused before any pointer is touched or any kernel is launched
    rc = lib.vb_lmhead_logprob_fwd_static(None, None, None, T, 3584, V, 1.0, None, None, None, None, None, None)
    assert rc == -4
