"""FP32 verification kernels vs the golden fixtures and the CPU oracle: max-abs <= 1e-5."""
from __future__ import annotations

import pytest
import torch

from conftest import load_golden
from oracle import mimi_attention_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-5   # north-star tolerance for the FP32 verification kernel (max-abs)


def _gpu(t):
    return t.cuda()


def test_isolated_op_config2_matches_golden():
    import fast_mimi_b200 as fm
    g = load_golden("isolated_T250.npz")
    gen = torch.Generator().manual_seed(int(g["seed"]))
    q, k, v = (torch.randn(1, 8, 250, 64, generator=gen) / 8 for _ in range(3))
    cos, sin = O.rope_tables(torch.arange(250))
    qf = _gpu(q).transpose(1, 2).contiguous()     # [B,T,H,D]
    kf = _gpu(k).transpose(1, 2).contiguous()
    fm.ops.rope_fp32_(qf, _gpu(cos)[None], _gpu(sin)[None])
    fm.ops.rope_fp32_(kf, _gpu(cos)[None], _gpu(sin)[None])
    rows = g["rows"]
    assert (qf.transpose(1, 2)[0][:, rows].cpu() - g["q_rot"]).abs().max() < 1e-6
    out = fm.window_attention_fp32(qf.transpose(1, 2), kf.transpose(1, 2), _gpu(v), scale=0.125, window=250)
    assert (out[0][:, rows].cpu() - g["out"]).abs().max() < TOL


def test_long_band_T700_matches_golden():
    import fast_mimi_b200 as fm
    g = load_golden("band_T700.npz")
    gen = torch.Generator().manual_seed(int(g["seed"]))
    q, k, v = (torch.randn(1, 8, 700, 64, generator=gen) / 8 for _ in range(3))
    cos, sin = O.rope_tables(torch.arange(700))
    qr, kr = O.apply_rope(q, k, cos, sin)
    out = fm.window_attention_fp32(_gpu(qr), _gpu(kr), _gpu(v), scale=0.125, window=250)
    assert (out[0][:, g["rows"]].cpu() - g["out"]).abs().max() < TOL


def _tiny_module(g):
    import fast_mimi_b200 as fm
    m = fm.MimiAttentionB200(16, 2, 8, sliding_window=8, precision="fp32").cuda()
    with torch.no_grad():
        for name in ("q", "k", "v", "o"):
            getattr(m, f"{name}_proj").weight.copy_(g[f"w{name}"])
    return m


def test_tiny_attention_layer_matches_golden():
    g = load_golden("tiny_attention_layer.npz")
    m = _tiny_module(g)
    x = _gpu(g["x"])
    cos, sin = O.rope_tables(torch.arange(x.shape[1]), head_dim=8)
    out, weights = m(x, None, None, (_gpu(cos)[None], _gpu(sin)[None]))
    assert weights is None
    assert (out.cpu() - g["out"]).abs().max() < TOL


@pytest.mark.parametrize("name", ["tiny_cached_chunks.npz", "tiny_cached_decode.npz"])
def test_tiny_cached_calls_match_golden(name):
    """Chunked streaming with a cache (the reference's test_parity.py:56-110 scenarios at module level)."""
    g = load_golden(name)
    m = _tiny_module(g)
    cache = m.new_cache(1, g["x0"].shape[0], "cuda")
    for i, t in enumerate(g["chunks"].tolist()):
        past = cache.get_seq_length()
        cos, sin = O.rope_tables(torch.arange(past, past + t), head_dim=8)
        out, _ = m(_gpu(g[f"x{i}"]), None, cache, (_gpu(cos)[None], _gpu(sin)[None]))
        assert (out.cpu() - g[f"out{i}"]).abs().max() < TOL, i
        assert cache.get_seq_length() == int(g["seq_lengths"][i])
        assert cache.key_cache[0].shape[1] <= 7
    # the cache keeps [B,T,H,D]; the reference keeps [B,H,T,D]
    assert (cache.key_cache[0].transpose(1, 2).cpu() - g["final_key_cache"]).abs().max() < TOL
    assert (cache.value_cache[0].transpose(1, 2).cpu() - g["final_value_cache"]).abs().max() < TOL


@pytest.mark.parametrize("T,window,H,D", [(1, 250, 8, 64), (2, 250, 8, 64), (65, 250, 8, 64), (251, 250, 8, 64),
                                          (313, 250, 8, 64), (40, 8, 2, 8), (33, 5, 3, 96), (17, 1, 1, 256)])
def test_generic_geometries_match_oracle(T, window, H, D):
    import fast_mimi_b200 as fm
    gen = torch.Generator().manual_seed(T * 1000 + window)
    q, k, v = (torch.randn(2, H, T, D, generator=gen) / 4 for _ in range(3))
    ref = O.band_attention(q, k, v, window=window, scale=D ** -0.5)
    out = fm.window_attention_fp32(_gpu(q), _gpu(k), _gpu(v), scale=D ** -0.5, window=window)
    assert (out.cpu() - ref).abs().max() < TOL


def test_offsets_of_a_cached_chunk_match_oracle():
    """Query chunk at positions 300..311 against keys 58..311 (249 cached + 12 new), window 250."""
    import fast_mimi_b200 as fm
    gen = torch.Generator().manual_seed(9)
    q = torch.randn(1, 8, 12, 64, generator=gen) / 4
    k, v = (torch.randn(1, 8, 261 - 7, 64, generator=gen) / 4 for _ in range(2))
    ref = O.band_attention(q, k, v, q_offset=300, k_offset=58, window=250, scale=0.125)
    out = fm.ops.band_attention_fp32(_gpu(q), _gpu(k), _gpu(v), window=250, scale=0.125, q_offset=300, k_offset=58)
    assert (out.cpu() - ref).abs().max() < TOL


def test_empty_inputs_are_accepted():
    import fast_mimi_b200 as fm
    q = torch.empty(0, 8, 4, 64, device="cuda")
    out = fm.ops.band_attention_fp32(q, q, q, window=250, scale=0.125)
    assert out.shape == q.shape
