"""The allocation-free entry point ``fm_attention_prefill_static_bf16`` (collected last on purpose).

It exists for hosts that cannot allocate device memory around the call — an allocation-free real-time
audio callback, a plugin whose host application owns every device allocation, a process with a fixed
device-memory budget — so its q/k/v
workspace is a fixed array inside the library.  The test drives it through the C ABI twice in a row
(the second call is smaller, so stale rows of the first stay in the workspace) and compares each
result with the ordinary entry points, which take caller-provided workspaces, and with the CPU oracle.
That nothing is allocated is checked at driver level (free device memory as cudaMemGetInfo reports it), which
also sees allocations that bypass PyTorch's caching allocator.
"""
from __future__ import annotations

import ctypes
import gc

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
    from oracle import mimi_attention_oracle as O
    lib = _native.load()
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # The first call on a device looks up the built-in array's address (and, with lazy module loading, is what
    # brings the library's device image, the array included, onto the GPU): it comes before the measured calls.
    x, w, cos, sin = _inputs(1, 130, 0)
    warm = torch.empty(x.shape, dtype=torch.float16, device="cuda")
    assert lib.fm_attention_prefill_static_bf16(x.data_ptr(), w.data_ptr(), cos.data_ptr(), sin.data_ptr(), 0,
                                                warm.data_ptr(), 1, 130, 250, 0.125, 1, status.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    for B, T, seed in ((32, 250, 1), (3, 199, 2)):
        x, w, cos, sin = _inputs(B, T, seed)
        ws = [torch.empty_like(x), torch.empty_like(x), torch.empty(x.shape, dtype=torch.float16, device="cuda")]
        want = torch.empty(x.shape, dtype=torch.float16, device="cuda")
        regular = torch.empty(x.shape, dtype=torch.float16, device="cuda")
        got = torch.full(x.shape, float("nan"), dtype=torch.float16, device="cuda")
        # the same two kernels with caller-provided workspaces ...
        rc = lib.fm_qkv_rope_bf16(x.data_ptr(), w.data_ptr(), cos.data_ptr(), sin.data_ptr(), 0, ws[0].data_ptr(),
                                  ws[1].data_ptr(), ws[2].data_ptr(), B, T, 1, status.data_ptr(), stream)
        assert rc == 0
        rc = lib.fm_band_attn_prefill_bf16(ws[0].data_ptr(), ws[1].data_ptr(), ws[2].data_ptr(), want.data_ptr(), B, T,
                                           250, 0.125, 1, status.data_ptr(), stream)
        assert rc == 0
        # ... and the ordinary entry point for a cache-free call
        rc = lib.fm_attention_prefill_bf16(x.data_ptr(), w.data_ptr(), cos.data_ptr(), sin.data_ptr(), 0,
                                           ws[0].data_ptr(), ws[1].data_ptr(), ws[2].data_ptr(), regular.data_ptr(),
                                           B, T, 250, 0.125, 1, status.data_ptr(), stream)
        assert rc == 0
        gc.collect()                                   # tensors of earlier tests must not be released mid-measurement
        torch.cuda.synchronize()
        before_torch = torch.cuda.memory_allocated()
        free_before, _ = torch.cuda.mem_get_info()
        rc = lib.fm_attention_prefill_static_bf16(x.data_ptr(), w.data_ptr(), cos.data_ptr(), sin.data_ptr(), 0,
                                                  got.data_ptr(), B, T, 250, 0.125, 1, status.data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after >= free_before               # no device allocation by any route
        assert torch.cuda.memory_allocated() <= before_torch
        assert lib.fm_read_status(status.data_ptr(), stream) == 0
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want)                  # same kernels on the same inputs: bit-identical
        assert O.rel_l2(got.float().cpu(), regular.float().cpu()) < TOL
        if B <= 4:                                     # and against the CPU oracle
            cos_c, sin_c = O.rope_tables(torch.arange(T))
            q, k, v = O.qkv_project(x.float().cpu(), *w.float().cpu().chunk(3, 0))
            q, k = O.apply_rope(q, k, cos_c, sin_c)
            ref = O.band_attention(q, k, v).transpose(1, 2).reshape(B, T, 512)
            assert O.rel_l2(got.float().cpu(), ref) < TOL


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
