"""Size-independent properties of the tensor-core path at the full benchmark sizes."""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def _qkv(B, T, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda dt: (torch.randn(B, T, 512, device="cuda", generator=g) / 2).to(dt)
    return mk(torch.bfloat16), mk(torch.bfloat16), mk(torch.float16)


def test_rows_of_ones_and_clip_independence_at_config3_size():
    import fast_mimi_b200 as fm
    B, T = 512, 250
    q, k, v = _qkv(B, T, 0)
    st = fm.ops.new_status("cuda")
    ones = torch.ones_like(v)
    out = fm.ops.band_attention_prefill(q, k, ones, status=st)
    assert fm.ops.read_status(st) == 0
    # softmax rows sum to one: attention over constant values returns the constant
    assert (out.float() - 1).abs().max() < 2e-3
    full = fm.ops.band_attention_prefill(q, k, v)
    alone = fm.ops.band_attention_prefill(q[77:78].contiguous(), k[77:78].contiguous(), v[77:78].contiguous())
    assert torch.equal(full[77:78], alone)          # clips never mix: bit-identical


def test_causality_and_window_are_exact_at_config4_size():
    import fast_mimi_b200 as fm
    B, T, W = 16, 2500, 250
    q, k, v = _qkv(B, T, 1)
    base = fm.ops.band_attention_prefill(q, k, v, window=W)
    k2, v2 = k.clone(), v.clone()
    k2[:, 2000:] = 0; v2[:, 2000:] = 1          # future of rows < 2000
    k2[:, :500] = 0; v2[:, :500] = -1           # out of window for rows >= 749
    pert = fm.ops.band_attention_prefill(q, k2, v2, window=W)
    assert torch.equal(base[:, 749:2000], pert[:, 749:2000])
    assert not torch.equal(base[:, 2000:], pert[:, 2000:])
    assert torch.isfinite(base.float()).all()


def test_decode_step_equals_prefill_last_row():
    """A ring filled by streaming T frames gives the same last-frame output as a T-frame prefill."""
    import fast_mimi_b200 as fm
    from oracle import mimi_attention_oracle as O
    torch.manual_seed(5)
    S, T = 64, 300
    w = (torch.randn(1536, 512, device="cuda") * 0.02).bfloat16()
    xs = torch.randn(S, T, 512, device="cuda").bfloat16()
    cos, sin = (t.cuda() for t in O.rope_tables(torch.arange(T)))
    pre = fm.ops.attention_prefill(xs, w, cos[None], sin[None])
    ring = fm.MimiKVRing(1, S, 250, device="cuda")
    for t in range(T):
        out = fm.ops.decode_step(xs[:, t].contiguous(), w, cos[None, t:t + 1], sin[None, t:t + 1], ring.ring_k[0],
                                 ring.ring_v[0], t)
        if t in (0, 1, 249, 250, 299):
            assert O.rel_l2(out.cpu(), pre[:, t].float().cpu()) < 2e-3, t


def test_prefill_and_decode_replay_inside_a_cuda_graph():
    """The entry points launch on the caller's stream without allocating, synchronising or reading back, so a
    captured graph replays them: prefill on new input, and streaming steps whose positions live in device
    memory (the reference captures its whole transformer the same way,
    src/fast_mimi/_optimized_runtime.py:1221-1241)."""
    import fast_mimi_b200 as fm
    from oracle import mimi_attention_oracle as O
    ops = fm.ops
    torch.manual_seed(9)
    dev = "cuda"
    B, T, S = 6, 250, 32
    w = (torch.randn(1536, 512, device=dev) * 0.02).bfloat16()
    cos, sin = (t.to(dev) for t in O.rope_tables(torch.arange(T)))
    x = torch.randn(B, T, 512, device=dev).bfloat16()
    ws = tuple(torch.empty(B, T, 512, dtype=dt, device=dev) for dt in (torch.bfloat16, torch.bfloat16, torch.float16))
    out = torch.empty(B, T, 512, dtype=torch.float16, device=dev)
    st = ops.new_status(dev)
    ops.attention_prefill(x, w, cos[None], sin[None], workspace=ws, out=out, status=st)     # warm-up outside capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ops.attention_prefill(x, w, cos[None], sin[None], workspace=ws, out=out, status=st)
    x2 = torch.randn(B, T, 512, device=dev).bfloat16()
    want = ops.attention_prefill(x2, w, cos[None], sin[None])
    x.copy_(x2)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, want)

    # streaming: one captured step, replayed with the position, the RoPE row and the input updated in place
    ring_g, ring_e = fm.MimiKVRing(1, S, 250, device=dev), fm.MimiKVRing(1, S, 250, device=dev)
    xs = torch.zeros(S, 512, dtype=torch.bfloat16, device=dev)
    pos = torch.zeros(S, dtype=torch.int32, device=dev)
    c1, s1 = torch.zeros(1, 1, 64, device=dev), torch.zeros(1, 1, 64, device=dev)
    qw = torch.empty_like(xs)
    o = torch.empty(S, 512, device=dev)
    scratch = fm.MimiKVRing(1, S, 250, device=dev)
    ops.decode_step(xs, w, c1, s1, scratch.ring_k[0], scratch.ring_v[0], 0, stream_pos=pos, q_workspace=qw, out=o, status=st)
    torch.cuda.synchronize()
    step = torch.cuda.CUDAGraph()
    with torch.cuda.graph(step):
        ops.decode_step(xs, w, c1, s1, ring_g.ring_k[0], ring_g.ring_v[0], 0, stream_pos=pos, q_workspace=qw, out=o, status=st)
    for t in range(6):
        frame = torch.randn(S, 512, device=dev).bfloat16()
        xs.copy_(frame); pos.fill_(t); c1.copy_(cos[t].view(1, 1, 64)); s1.copy_(sin[t].view(1, 1, 64))
        step.replay()
        eager = ops.decode_step(frame, w, cos[None, t:t + 1], sin[None, t:t + 1], ring_e.ring_k[0], ring_e.ring_v[0], t)
        torch.cuda.synchronize()
        # the eager call knows the position on the host and may take the short-ring kernel: same numbers up to
        # the order of the FP32 sums
        assert O.rel_l2(o.cpu(), eager.cpu()) < 1e-5, t
    assert ops.read_status(st) == 0
