"""The allocation-free greedy entry point (lm_argmax_static) against the ordinary one (lm_argmax).

Some callers of the library are given tensors and a stream but may not allocate device memory (a plug-in inside a
frozen decode loop, a step running while the engine's allocator is locked): lm_argmax_static keeps the scratch
that lm_argmax takes from the caller in a fixed array inside the library instead. This file is collected last on
purpose (its name sorts after every other test file): a run that stops at the first failure has then already
run the rest of the suite.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from lithos_metal_b200 import _lib
import lithos_metal_b200 as lm

pytestmark = pytest.mark.gpu


def _logits(rows, vocab, seed, dtype):
    rng = np.random.default_rng(seed)
    z = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
    z[0, vocab - 1] = 90.0                     # the maximum at the very end of a row
    if rows > 1:
        z[1, 5] = z[1, 7] = 50.0               # a tie: the lowest index must win
    if dtype == "bf16":
        codes = oracle.f32_to_bf16(z)
        return torch.from_numpy(codes.view(np.int16)).cuda().view(torch.bfloat16), oracle.bf16_to_f32(codes)
    return torch.from_numpy(z).cuda(), z


@pytest.mark.parametrize("rows,vocab,dtype", [(8, 151936, "bf16"), (1, 151936, "f32"), (64, 151936, "bf16"), (300, 4096, "bf16"), (37, 1000, "f32")])
def test_static_scratch_argmax_equals_the_workspace_one(rows, vocab, dtype):
    L = _lib.lib()
    x, host = _logits(rows, vocab, rows + vocab, dtype)
    expect = lm.argmax(x)                                                    # the existing entry point, caller-owned workspace
    assert expect.cpu().tolist() == host.argmax(-1).tolist()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):                                                    # two calls in a row share the library's scratch
        out = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
        rc = L.lm_argmax_static(x.data_ptr(), _lib.DTYPE_BF16 if dtype == "bf16" else _lib.DTYPE_F32, rows, vocab, x.stride(0) if rows > 1 else vocab,
                                out.data_ptr(), stream)
        assert rc == 0, L.lm_error_string(rc)
        assert torch.equal(out, expect), call                                # bit-exact, like every other token-id check in this suite


def test_static_scratch_rejects_what_does_not_fit():
    L = _lib.lib()
    rows = _lib.ARGMAX_STATIC_MAX_ROWS + 1
    x = torch.zeros(rows, 64, dtype=torch.bfloat16, device="cuda")
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    rc = L.lm_argmax_static(x.data_ptr(), _lib.DTYPE_BF16, rows, 64, 64, out.data_ptr(), None)
    assert rc == -4 and b"supported range" in L.lm_error_string(rc)
    assert L.lm_argmax_static(None, _lib.DTYPE_BF16, 4, 64, 64, out.data_ptr(), None) == -1
    assert L.lm_argmax_static(None, _lib.DTYPE_BF16, 0, 64, 64, None, None) == 0


def test_static_scratch_allocates_nothing_and_survives_a_larger_call_before_a_smaller_one():
    """A call that splits many rows over several blocks dirties most of the library's scratch; the smaller call behind it must
    still be right (the entry point clears what it uses), and neither call may take device memory: the free memory the driver
    reports and the bytes torch has handed out are the same before and after."""
    L = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    big, big_host = _logits(_lib.ARGMAX_STATIC_MAX_ROWS, 32768, 11, "bf16")   # the largest row count the scratch holds
    wide, wide_host = _logits(64, 151936, 12, "bf16")                        # 64 rows x 151936: split over several blocks per row
    small, small_host = _logits(3, 151936, 13, "f32")
    outs = [torch.full((t.shape[0],), -7, dtype=torch.int32, device="cuda") for t in (big, wide, small)]
    L.lm_argmax_static(small.data_ptr(), _lib.DTYPE_F32, 3, 151936, 151936, outs[2].data_ptr(), stream)   # first use on this device: its set-up
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    held0 = torch.cuda.memory_allocated()
    for x, out, code in ((big, outs[0], _lib.DTYPE_BF16), (wide, outs[1], _lib.DTYPE_BF16), (small, outs[2], _lib.DTYPE_F32)):
        out.fill_(-7)
        assert L.lm_argmax_static(x.data_ptr(), code, x.shape[0], x.shape[1], x.stride(0), out.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0 and torch.cuda.memory_allocated() == held0
    for out, host in zip(outs, (big_host, wide_host, small_host)):
        assert out.cpu().tolist() == host.argmax(-1).tolist()
