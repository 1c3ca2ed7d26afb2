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
