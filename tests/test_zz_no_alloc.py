"""The allocation-free entry point ``fm_attention_prefill_static_bf16`` (collected last on purpose).

It exists for hosts that cannot allocate device memory around the call — an allocation-free real-time
audio callback, a plugin whose host application owns every device allocation, a process with a fixed
device-memory budget — so its q/k/v
workspace is a fixed array inside the library.  The test drives it through the C ABI twice in a row
(the second call is smaller, so stale rows of the first stay in the workspace) and compares each
result with the ordinary entry point, which takes caller-provided workspaces.
"""
from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 2e-3   # relative L2, the tolerance of the tensor-core parity tests


def _inputs(B, T, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(B, T, 512, device="cuda", generator=g).bfloat16()
    w = (torch.randn(1536, 512, device="cuda", generator=g) * 0.02).bfloat16()
    pos = torch.arange(T, device="cuda", dtype=torch.float32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, 64, 2, device="cuda").float() / 64))
    emb = torch.cat((torch.outer(pos, inv),) * 2, -1)
    return x, w, emb.cos()[None].contiguous(), emb.sin()[None].contiguous()


def test_static_workspace_entry_point_matches_the_regular_one_twice():
    from fast_mimi_b200 import _native
    from oracle.mimi_attention_oracle import rel_l2
    lib = _native.load()
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for B, T, seed in ((32, 250, 1), (3, 199, 2)):
        x, w, cos, sin = _inputs(B, T, seed)
        ws = [torch.empty_like(x), torch.empty_like(x), torch.empty(x.shape, dtype=torch.float16, device="cuda")]
        want = torch.empty(x.shape, dtype=torch.float16, device="cuda")
        got = torch.full(x.shape, float("nan"), dtype=torch.float16, device="cuda")
        rc = lib.fm_attention_prefill_bf16(x.data_ptr(), w.data_ptr(), cos.data_ptr(), sin.data_ptr(), 0,
                                           ws[0].data_ptr(), ws[1].data_ptr(), ws[2].data_ptr(), want.data_ptr(),
                                           B, T, 250, 0.125, 1, status.data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = lib.fm_attention_prefill_static_bf16(x.data_ptr(), w.data_ptr(), cos.data_ptr(), sin.data_ptr(), 0,
                                                  got.data_ptr(), B, T, 250, 0.125, 1, status.data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert lib.fm_read_status(status.data_ptr(), stream) == 0
        assert torch.isfinite(got.float()).all()
        assert rel_l2(got.float().cpu(), want.float().cpu()) < TOL
        assert torch.equal(got, want)      # same kernels on the same inputs: bit-identical


def test_static_workspace_entry_point_rejects_oversized_calls():
    import fast_mimi_b200 as fm
    from fast_mimi_b200 import _native
    lib = _native.load()
    x, w, cos, sin = _inputs(33, 250, 3)                      # 8250 frames > 8192
    out = torch.zeros(x.shape, dtype=torch.float16, device="cuda")
    rc = lib.fm_attention_prefill_static_bf16(x.data_ptr(), w.data_ptr(), cos.data_ptr(), sin.data_ptr(), 0,
                                              out.data_ptr(), 33, 250, 250, 0.125, 1, None,
                                              torch.cuda.current_stream().cuda_stream)
    assert rc == -5
    torch.cuda.synchronize()
    assert not out.any()                                      # nothing was launched
    with pytest.raises(RuntimeError, match="built-in workspace"):
        fm.ops.attention_prefill_static(x, w, cos, sin, out)
