"""Pin the CPU oracle against outputs of the reference itself (tests/golden/*.npz)."""
from __future__ import annotations

import torch

from conftest import load_golden, regen_attention_layer, regen_projections
from oracle import mimi_attention_oracle as O

TOL = 2e-6   # FP32 reassociation noise between the oracle's eager softmax and the reference's SDPA


def test_pairs_match_published_counts():
    assert (O.pairs(125), O.pairs(250), O.pairs(2500)) == (7875, 31375, 593875)


def test_rope_tables_and_isolated_op_match_reference():
    g = load_golden("isolated_T250.npz")
    gen = torch.Generator().manual_seed(int(g["seed"]))
    q, k, v = (torch.randn(1, 8, 250, 64, generator=gen) / 8 for _ in range(3))
    assert torch.equal(q[0, 0, :4], g["q_head0"]) and torch.equal(v[0, 7, -4:], g["v_head7"])
    cos, sin = O.rope_tables(torch.arange(250))
    rows = g["rows"]
    assert torch.equal(cos[rows], g["cos"]) and torch.equal(sin[rows], g["sin"])
    qr, kr = O.apply_rope(q, k, cos, sin)
    assert torch.equal(qr[0][:, rows], g["q_rot"])
    out = O.band_attention(qr, kr, v)
    assert (out[0][:, rows] - g["out"]).abs().max() < TOL
    out2 = O.band_attention_sdpa(qr, kr, v)
    assert (out2[0][:, rows] - g["out"]).abs().max() < TOL


def test_long_band_matches_reference():
    g = load_golden("band_T700.npz")
    gen = torch.Generator().manual_seed(int(g["seed"]))
    q, k, v = (torch.randn(1, 8, 700, 64, generator=gen) / 8 for _ in range(3))
    cos, sin = O.rope_tables(torch.arange(700))
    qr, kr = O.apply_rope(q, k, cos, sin)
    out = O.band_attention(qr, kr, v)
    assert (out[0][:, g["rows"]] - g["out"]).abs().max() < TOL


def test_tiny_attention_layer_matches_reference():
    g = load_golden("tiny_attention_layer.npz")
    out = O.attention_forward(g["x"], g["wq"], g["wk"], g["wv"], g["wo"], window=8, num_heads=2)
    assert (out - g["out"]).abs().max() < TOL


def test_full_size_attention_layers_match_reference():
    for name in ("attention_layer_T250.npz", "attention_layer_T313.npz", "attention_layer_T250_fp32.npz"):
        g = load_golden(name)
        x, wq, wk, wv, wo = regen_attention_layer(int(g["seed"]), int(g["b"]), int(g["t"]),
                                                  bf16_inputs="fp32" not in name)
        assert torch.equal(x[0, :2, :8], g["x_probe"]) and torch.equal(wq[:2, :8], g["wq_probe"])
        out = O.attention_forward(x, wq, wk, wv, wo)
        assert (out[:, g["rows"]] - g["out"]).abs().max() < TOL


def _run_cached(g, window, heads):
    cache = O.KVCacheOracle(window=window)
    outs = []
    for i, t in enumerate(g["chunks"].tolist()):
        outs.append(O.attention_forward(g[f"x{i}"], g["wq"], g["wk"], g["wv"], g["wo"], cache=cache,
                                        window=window, num_heads=heads))
        assert cache.get_seq_length() == int(g["seq_lengths"][i])
    return cache, outs


def test_tiny_cached_chunks_and_decode_match_reference():
    for name in ("tiny_cached_chunks.npz", "tiny_cached_decode.npz"):
        g = load_golden(name)
        cache, outs = _run_cached(g, 8, 2)
        for i, out in enumerate(outs):
            assert (out - g[f"out{i}"]).abs().max() < TOL, (name, i)
        assert cache.keys[0].shape[-2] == 7
        assert (cache.keys[0] - g["final_key_cache"]).abs().max() < TOL
        assert (cache.values[0] - g["final_value_cache"]).abs().max() < TOL


def test_mimi_size_cached_chunks_match_reference():
    """Chunked streaming at Mimi's geometry (chunks that cross the window, one-frame steps in between, one chunk
    longer than the window): the oracle against the reference's MimiAttention + MimiKVCache outputs."""
    g = load_golden("cached_chunks_mimi.npz")
    wq, wk, wv, wo = regen_projections(int(g["seed"]))
    cache = O.KVCacheOracle()
    for step, t in enumerate(g["chunks"].tolist()):
        x = torch.randn(int(g["b"]), t, 512).bfloat16().float()
        out = O.attention_forward(x, wq, wk, wv, wo, cache=cache)
        assert (out[:, g[f"rows{step}"]] - g[f"out{step}"]).abs().max() < TOL, step
    assert cache.get_seq_length() == int(g["seq_length"])
    assert (cache.keys[0][:, :, -3:] - g["final_key_cache"]).abs().max() < TOL
    assert (cache.values[0][:, :, -3:] - g["final_value_cache"]).abs().max() < TOL


def test_downsample_conv_matches_reference():
    """The oracle's stride-2 convolution against the reference's MimiConv1d (causal, replicate padding, no bias)."""
    g = load_golden("downsample.npz")
    torch.manual_seed(int(g["seed"]))
    torch.nn.Conv1d(512, 512, 4, 2, bias=False)             # the reference module's own initialisation draws first
    weight = torch.randn(512, 512, 4) / (4 * 512) ** 0.5
    assert torch.equal(weight[:2, :3], g["weight_probe"])
    for t in (125, 250, 7):
        x = torch.randn(2, t, 512)
        y = O.downsample_conv(x, weight)
        assert y.shape[1] == int(g[f"frames{t}"]) == (t + 1) // 2
        assert (y[:, g[f"rows{t}"]] - g[f"out{t}"]).abs().max() < TOL


def test_upsample_conv_matches_reference():
    """The oracle's stride-2 transposed convolution against the reference's MimiConvTranspose1d (depthwise, causal
    trimming, no bias)."""
    g = load_golden("upsample.npz")
    torch.manual_seed(int(g["seed"]))
    torch.nn.ConvTranspose1d(512, 512, 4, 2, groups=512, bias=False)   # the reference module's own initialisation draws first
    weight = torch.randn(512, 1, 4) / 2
    assert torch.equal(weight[:3, 0], g["weight_probe"])
    for t in (63, 125, 1):
        x = torch.randn(2, t, 512)
        y = O.upsample_conv(x, weight)
        assert y.shape[1] == int(g[f"frames{t}"]) == 2 * t
        assert (y[:, g[f"rows{t}"]] - g[f"out{t}"]).abs().max() < TOL


def test_ring_decode_260_matches_reference():
    g = load_golden("ring_decode_260.npz")
    wq, wk, wv, wo = regen_projections(int(g["seed"]))
    cache = O.KVCacheOracle()
    keep = g["keep_steps"].tolist()
    got = []
    for step in range(260):
        x = torch.randn(2, 1, 512).bfloat16().float()
        out = O.attention_forward(x, wq, wk, wv, wo, cache=cache)
        if step in keep:
            got.append(out)
    assert cache.get_seq_length() == 260 and cache.keys[0].shape[-2] == 249
    assert (torch.stack(got) - g["outs"]).abs().max() < TOL
    assert (cache.keys[0][:, :, -3:] - g["final_key_cache"]).abs().max() < TOL


def test_tiny_stack_prefill_and_chunked_match_reference():
    g = load_golden("tiny_stack.npz")
    params = {k[2:]: v for k, v in g.items() if k.startswith("p.")}

    def run(x, cache):
        past = cache.get_seq_length(0) if cache is not None else 0
        for layer in range(2):
            p = {k[len(f"layers.{layer}."):]: v for k, v in params.items() if k.startswith(f"layers.{layer}.")}
            x = O.transformer_layer(x, p, cache=cache, layer=layer, window=8, num_heads=2, past_length=past)
        return x

    assert (run(g["x"], None) - g["full"]).abs().max() < TOL
    cache = O.KVCacheOracle(window=8)
    outs = [run(g["x"][:, a:b], cache) for a, b in ((0, 5), (5, 6), (6, 13), (13, 14), (14, 21))]
    assert (torch.cat(outs, 1) - g["chunked"]).abs().max() < TOL


def test_layer_block_restatements_equal_the_library_calls_the_reference_makes():
    """layer_norm / mlp / out_proj_residual are explicit formulas; the reference calls nn.LayerNorm, nn.Linear
    and F.gelu (src/fast_mimi/model.py:1999, 2021-2024, 2052-2061).  The golden two-layer stack pins them through
    transformer_layer; this pins each on its own at Mimi's widths."""
    import torch.nn.functional as F
    g = torch.Generator().manual_seed(3)
    x = torch.randn(5, 7, 512, generator=g) * 2 + 0.3
    w, b = torch.rand(512, generator=g) + 0.5, torch.randn(512, generator=g) * 0.1
    assert (O.layer_norm(x, w, b, 1e-5) - F.layer_norm(x, (512,), w, b, 1e-5)).abs().max() < 2e-6
    fc1, fc2 = torch.randn(2048, 512, generator=g) * 0.04, torch.randn(512, 2048, generator=g) * 0.02
    assert torch.equal(O.mlp(x, fc1, fc2), F.linear(F.gelu(F.linear(x, fc1)), fc2))
    wo, s = torch.randn(512, 512, generator=g) * 0.04, torch.rand(512, generator=g)
    assert torch.equal(O.out_proj_residual(x, wo, s, x), x + F.linear(x, wo) * s)


def test_rvq_restatement_matches_the_reference_quantizer():
    """oracle.rvq_encode / rvq_decode against codes and decoded sums that the reference's
    MimiResidualVectorQuantizer produced (tests/golden/rvq_codes.npz) for the same seeded constants."""
    import torch.nn.functional as F
    from conftest import rvq_recipe
    g = load_golden("rvq_codes.npz")
    gen, embed_sum, usage, proj = rvq_recipe(31, 7)
    emb = torch.randn(2, 512, 40, generator=gen) * 3
    assert torch.equal(emb[0, :4, :4], g["emb_probe"])
    books = embed_sum / usage.clamp(min=1e-5)[:, :, None]
    x = F.conv1d(emb, proj[:, :, None]).permute(0, 2, 1).reshape(-1, 256)       # input_proj, frames as rows
    codes = O.rvq_encode(x, books).view(7, 2, 40)
    assert torch.equal(codes, g["codes"])
    dec = O.rvq_decode(codes.view(7, 80), books).view(2, 40, 256).permute(0, 2, 1)
    assert torch.equal(dec[:, :, ::13], g["quantized_probe"])
