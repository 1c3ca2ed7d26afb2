"""The blocks around the attention core (LayerNorm, o_proj / MLP linears with fused GELU, layer scale and
residual add) and the whole transformer layer built from them, vs the CPU oracle."""
from __future__ import annotations

import pytest
import torch

from oracle import mimi_attention_oracle as O

pytestmark = pytest.mark.gpu

ROUND = {torch.float16: 5e-4, torch.bfloat16: 4e-3, torch.float32: 2e-6}   # one rounding of the result


@pytest.mark.parametrize("x_dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows", [1, 33, 2500])
def test_layer_norm_matches_oracle(rows, x_dtype):
    import fast_mimi_b200 as fm
    torch.manual_seed(5)
    x = (torch.randn(rows, 512) * 3 + 0.7).to(x_dtype)
    w, b = torch.rand(512) + 0.5, torch.randn(512) * 0.1
    ref = O.layer_norm(x.float(), w, b, 1e-5)
    for out_dtype in (torch.float16, torch.bfloat16):
        got = fm.ops.layer_norm(x.cuda(), w.cuda(), b.cuda(), eps=1e-5, out_dtype=out_dtype)
        assert got.dtype == out_dtype and O.rel_l2(got.float().cpu(), ref) < ROUND[out_dtype]
    exact = fm.ops.layer_norm(x.cuda(), w.cuda(), b.cuda(), out_dtype=torch.float16).float().cpu()
    assert (exact - ref.half().float()).abs().max() <= 2e-3      # within an FP16 ulp of the rounded oracle


@pytest.mark.parametrize("shape", [(512, 512), (512, 2048), (2048, 512), (64, 256)])
@pytest.mark.parametrize("rows", [1, 300, 5000])
def test_linear_epilogues_match_oracle(rows, shape):
    """Every epilogue (plain, GELU, scale, scale + residual, in place) for the three output types and both
    input types, over the layer's three weight shapes and ragged row counts."""
    import fast_mimi_b200 as fm
    K, N = shape
    torch.manual_seed(rows + K)
    st = fm.ops.new_status("cuda")
    for in_dtype in (torch.float16, torch.bfloat16):
        a = torch.randn(rows, K).to(in_dtype)
        w = (torch.randn(N, K) / K ** 0.5).to(in_dtype)
        s = torch.rand(N) + 0.2
        for out_dtype in (torch.float32, torch.float16, torch.bfloat16):
            r = torch.randn(rows, N).to(out_dtype)
            acc = torch.nn.functional.linear(a.float(), w.float())
            cases = [(None, None, None, acc), ("gelu", None, None, torch.nn.functional.gelu(acc)),
                     (None, s, r, r.float() + s * acc), ("gelu", s, None, s * torch.nn.functional.gelu(acc))]
            for act, scale, resid, ref in cases:
                got = fm.ops.linear(a.cuda(), w.cuda(), scale=None if scale is None else scale.cuda(),
                                    residual=None if resid is None else resid.cuda(), activation=act,
                                    out_dtype=out_dtype, status=st)
                assert got.dtype == out_dtype and got.shape == (rows, N)
                assert O.rel_l2(got.float().cpu(), ref) < max(ROUND[out_dtype], 2e-5), (in_dtype, out_dtype, act)
            buf = r.cuda().clone()
            fm.ops.linear(a.cuda(), w.cuda(), scale=s.cuda(), residual=buf, out=buf, status=st)
            assert O.rel_l2(buf.float().cpu(), r.float() + s * acc) < max(ROUND[out_dtype], 2e-5)
    assert fm.ops.read_status(st) == 0


def test_linear_rejects_bad_geometry():
    import fast_mimi_b200 as fm
    a = torch.zeros(4, 100, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError):
        fm.ops.linear(a, torch.zeros(256, 100, dtype=torch.float16, device="cuda"))
    with pytest.raises(RuntimeError):
        fm.ops.linear(torch.zeros(4, 128, dtype=torch.float16, device="cuda"),
                      torch.zeros(100, 128, dtype=torch.float16, device="cuda"))


def _layer_params(seed):
    g = torch.Generator().manual_seed(seed)
    n = lambda *s, std=1.0: torch.randn(*s, generator=g) * std
    return {
        "self_attn.q_proj.weight": n(512, 512, std=0.04), "self_attn.k_proj.weight": n(512, 512, std=0.04),
        "self_attn.v_proj.weight": n(512, 512, std=0.04), "self_attn.o_proj.weight": n(512, 512, std=0.04),
        "mlp.fc1.weight": n(2048, 512, std=0.04), "mlp.fc2.weight": n(512, 2048, std=0.02),
        "input_layernorm.weight": torch.rand(512, generator=g) * 0.2 + 0.9, "input_layernorm.bias": n(512, std=0.01),
        "post_attention_layernorm.weight": torch.rand(512, generator=g) * 0.2 + 0.9,
        "post_attention_layernorm.bias": n(512, std=0.01),
        "self_attn_layer_scale.scale": torch.rand(512, generator=g) * 0.2 + 0.05,
        "mlp_layer_scale.scale": torch.rand(512, generator=g) * 0.2 + 0.05,
    }


@pytest.mark.parametrize("stream_dtype", [torch.float32, torch.bfloat16])
def test_transformer_layer_matches_oracle(stream_dtype):
    """Whole layer (seven launches) vs the oracle's FP32 layer on FP32 parameters that are not 16-bit
    representable.  The parity metric is taken on what the layer ADDS to the residual stream, which is where
    all of the 16-bit operand rounding lands; the stream itself (FP32 case) must then agree to 1e-4."""
    import fast_mimi_b200 as fm
    p = _layer_params(21)
    torch.manual_seed(22)
    B, T = 3, 250
    x = torch.randn(B, T, 512)
    if stream_dtype != torch.float32:
        x = x.to(stream_dtype).float()
    ref = O.transformer_layer(x, p)
    layer = fm.MimiTransformerLayerB200().cuda()
    layer.load_state_dict(p, strict=True)
    layer = layer.to(stream_dtype)
    cos, sin = O.rope_tables(torch.arange(T))
    out, weights = layer(x.to(stream_dtype).cuda(), None, None, (cos.cuda()[None], sin.cuda()[None]), False)
    assert weights is None and out.dtype == stream_dtype and out.shape == x.shape
    got = out.float().cpu()
    if stream_dtype == torch.float32:
        assert O.rel_l2(got - x, ref - x) < 2e-3
        assert O.rel_l2(got, ref) < 1e-4
    else:
        assert O.rel_l2(got, ref) < 6e-3      # BF16 parameters and a BF16 residual stream


def test_transformer_layer_shares_parameters_with_the_module_it_replaces():
    import fast_mimi_b200 as fm
    src = fm.MimiTransformerLayerB200().cuda()
    new = fm.MimiTransformerLayerB200.from_reference(src)
    assert new.mlp.fc1.weight is src.mlp.fc1.weight and new.self_attn.q_proj.weight is src.self_attn.q_proj.weight
    assert sorted(new.state_dict()) == sorted(src.state_dict())


def test_install_layers_replaces_every_layer_and_keeps_the_numbers():
    """install_layers on a module with a `layers` ModuleList (the reference's MimiTransformerModel attribute):
    every entry becomes a MimiTransformerLayerB200 that shares the parameters, so a two-layer pass gives the same
    result as before and matches the oracle."""
    import torch.nn as nn
    import fast_mimi_b200 as fm
    stack = nn.Module()
    stack.layers = nn.ModuleList([fm.MimiTransformerLayerB200(layer_idx=i) for i in range(2)])
    params = [_layer_params(50 + i) for i in range(2)]
    for layer, p in zip(stack.layers, params):
        layer.load_state_dict(p, strict=True)
    stack = stack.cuda()
    T = 200
    x = torch.randn(2, T, 512, generator=torch.Generator().manual_seed(52))
    cos, sin = O.rope_tables(torch.arange(T))
    pe = (cos.cuda()[None], sin.cuda()[None])

    def run(mod):
        h = x.cuda()
        for layer in mod.layers:
            h, _ = layer(h, None, None, pe, False)
        return h.cpu()

    before = run(stack)
    old_weight = stack.layers[1].mlp.fc2.weight
    fm.install_layers(stack)
    assert all(isinstance(l, fm.MimiTransformerLayerB200) for l in stack.layers)
    assert stack.layers[1].mlp.fc2.weight is old_weight
    assert torch.equal(run(stack), before)
    ref = x
    for p in params:
        ref = O.transformer_layer(ref, p)
    assert O.rel_l2(before - x, ref - x) < 2e-3
