"""The two stride-2 convolutions around the quantiser on the GPU: the downsampling convolution after the encoder
transformer (row gather + split-precision tensor-core products) and the depthwise transposed convolution before the
decoder transformer (elementwise), vs the reference's outputs (golden fixtures) and the CPU oracle."""
from __future__ import annotations

import pytest
import torch

from conftest import load_golden
from oracle import mimi_attention_oracle as O

pytestmark = pytest.mark.gpu
# max-abs relative to max |y|.  FP32-grade accuracy is the point of the split-precision products; the reference's own
# FP32 convolution carries a rounding of this order over its 2048-term sums (a different summation order), so the bar
# is a few units of FP32 epsilon times sqrt(2048), far below the 5e-4 of a plain FP16 product.
TOL = 1e-5


def _weight_parts(weight):
    import fast_mimi_b200 as fm
    return fm.ops.split_half(weight.permute(0, 2, 1).reshape(weight.shape[0], -1).contiguous().cuda())


def test_downsample_matches_the_reference_fixture():
    import fast_mimi_b200 as fm
    g = load_golden("downsample.npz")
    torch.manual_seed(int(g["seed"]))
    torch.nn.Conv1d(512, 512, 4, 2, bias=False)
    weight = torch.randn(512, 512, 4) / (4 * 512) ** 0.5
    parts = _weight_parts(weight)
    for t in (125, 250, 7):
        x = torch.randn(2, t, 512)
        y = fm.ops.downsample_conv(x.cuda(), parts).cpu()
        want = g[f"out{t}"]
        assert y.shape == (2, (t + 1) // 2, 512)
        err = float((y[:, g[f"rows{t}"]] - want).abs().max() / want.abs().max())
        print(f"downsample T={t}: max error / max |y| vs the reference = {err:.2e}")
        assert err < TOL
    fm.check_status()


@pytest.mark.parametrize("B,T", [(1, 1), (3, 2), (2, 33), (64, 250), (5, 251)])
def test_downsample_matches_the_oracle(B, T):
    import fast_mimi_b200 as fm
    g = torch.Generator().manual_seed(B * 1000 + T)
    weight = torch.randn(512, 512, 4, generator=g) / 45
    x = torch.randn(B, T, 512, generator=g) * 2
    y = fm.ops.downsample_conv(x.cuda(), _weight_parts(weight)).cpu()
    want = O.downsample_conv(x, weight)
    assert y.shape == want.shape
    assert float((y - want).abs().max() / want.abs().max()) < TOL


def test_downsample_module_keeps_the_reference_call_shape():
    """MimiDownsampleB200 takes [B, C, T] and returns [B, C, ceil(T / 2)] like MimiConv1d.forward, sharing the weight."""
    import types
    import fast_mimi_b200 as fm
    conv = torch.nn.Conv1d(512, 512, 4, 2, bias=False).cuda()
    ref = types.SimpleNamespace(conv=conv, causal=True, pad_mode="replicate")
    mod = fm.MimiDownsampleB200(ref)
    x = torch.randn(2, 512, 77, device="cuda")
    y = mod(x)
    want = O.downsample_conv(x.cpu().transpose(1, 2), conv.weight.detach().cpu()).transpose(1, 2)
    assert y.shape == (2, 512, 39)
    assert float((y.cpu() - want).abs().max() / want.abs().max()) < TOL
    with pytest.raises(RuntimeError):
        mod(x, padding_cache=object())
    with pytest.raises(RuntimeError):
        mod(x.cpu())


def test_upsample_matches_the_reference_fixture_and_the_oracle():
    import fast_mimi_b200 as fm
    g = load_golden("upsample.npz")
    torch.manual_seed(int(g["seed"]))
    torch.nn.ConvTranspose1d(512, 512, 4, 2, groups=512, bias=False)
    weight = torch.randn(512, 1, 4) / 2
    w = weight.reshape(512, 4).contiguous().cuda()
    for t in (63, 125, 1):
        x = torch.randn(2, t, 512)
        y = fm.ops.upsample2(x.cuda(), w).cpu()
        assert y.shape == (2, 2 * t, 512)
        assert float((y[:, g[f"rows{t}"]] - g[f"out{t}"]).abs().max()) < 1e-6      # two FP32 products and one add
        assert float((y - O.upsample_conv(x, weight)).abs().max()) < 1e-6


def test_upsample_module_keeps_the_reference_call_shape():
    import types
    import fast_mimi_b200 as fm
    convtr = torch.nn.ConvTranspose1d(512, 512, 4, 2, groups=512, bias=False).cuda()
    ref = types.SimpleNamespace(conv=convtr, padding_left=0, padding_right=2)
    mod = fm.MimiUpsampleB200(ref)
    x = torch.randn(3, 512, 40, device="cuda")
    y = mod(x)
    want = O.upsample_conv(x.cpu().transpose(1, 2), convtr.weight.detach().cpu()).transpose(1, 2)
    assert y.shape == (3, 512, 80)
    assert float((y.cpu() - want).abs().max()) < 1e-6
    with pytest.raises(RuntimeError):
        mod(x.cpu())
    with pytest.raises(ValueError):
        fm.MimiUpsampleB200(types.SimpleNamespace(conv=torch.nn.ConvTranspose1d(512, 512, 4, 2, bias=False)))
