"""Shared test plumbing: the ``gpu`` marker, repo-root imports and golden-fixture loading."""
from __future__ import annotations

import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name: str) -> dict:
    with np.load(os.path.join(GOLDEN, name)) as z:
        return {k: torch.from_numpy(np.asarray(z[k])) if z[k].dtype.kind in "fiub" and z[k].ndim > 0
                else z[k].item() for k in z.files}


@pytest.fixture(scope="session")
def golden():
    return load_golden


def regen_projections(seed: int, hidden: int = 512, std: float = 0.02, bf16_inputs: bool = True):
    """Rebuild the seeded weights of ``tests/golden/make_golden.py`` without the reference: four
    bias-free Linear(hidden, hidden) constructed in q,k,v,o order (their default init consumes the
    RNG), re-initialised N(0, std^2) in the same order; q/k/v weights rounded to BF16-representable
    values as the generator does for the full-size fixtures.  Leaves the RNG where x is drawn next."""
    torch.manual_seed(seed)
    lins = [torch.nn.Linear(hidden, hidden, bias=False) for _ in range(4)]
    for lin in lins:
        torch.nn.init.normal_(lin.weight, std=std)
    wq, wk, wv, wo = (lin.weight.detach() for lin in lins)
    if not bf16_inputs:
        return wq, wk, wv, wo
    return wq.bfloat16().float(), wk.bfloat16().float(), wv.bfloat16().float(), wo


def regen_attention_layer(seed: int, b: int, t: int, hidden: int = 512, std: float = 0.02,
                          bf16_inputs: bool = True):
    """Weights as ``regen_projections`` then x ~ N(0,1), rounded to BF16-representable values unless the
    fixture was generated from full FP32 inputs."""
    wq, wk, wv, wo = regen_projections(seed, hidden, std, bf16_inputs)
    x = torch.randn(b, t, hidden)
    if bf16_inputs:
        x = x.bfloat16().float()
    return x, wq, wk, wv, wo


def fill_state_by_recipe(state: dict, seed: int = 0) -> dict:
    """Deterministic weights for a full-size Mimi model, independent of module construction order: walk the
    state dict in key order and draw every tensor from one seeded generator (codebook usage U[0.5,1.5),
    codebook sums N(0,1), LayerNorm weights U[0.9,1.1), biases N(0,0.01^2), layer scales 0.01, matrices and
    convolution kernels N(0, 1/fan_in)).  The reference's own fixture does the same with other constants
    (tests/conftest.py:41-53 of the reference); a default-constructed model has all-zero codebooks."""
    import math
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, v in state.items():
            if name.endswith(".initialized"):
                v.fill_(1)
            elif name.endswith(".cluster_usage"):
                v.copy_(torch.rand(v.shape, generator=g) + 0.5)
            elif name.endswith(".embed_sum"):
                v.copy_(torch.randn(v.shape, generator=g))
            elif "layernorm.weight" in name:
                v.copy_(torch.rand(v.shape, generator=g) * 0.2 + 0.9)
            elif "layernorm.bias" in name or name.endswith(".bias"):
                v.copy_(torch.randn(v.shape, generator=g) * 0.01)
            elif name.endswith("layer_scale.scale"):
                v.fill_(0.01)
            elif v.dim() >= 2:
                v.copy_(torch.randn(v.shape, generator=g) / math.sqrt(v[0].numel()))
            else:
                v.copy_(torch.randn(v.shape, generator=g) * 0.05)
    return state


def synthetic_audio(seed: int = 0, seconds: int = 5, rate: int = 24000) -> torch.Tensor:
    """benchmark config 1 input: harmonic series f0~U[90,250] Hz, 20 partials at 1/k amplitude, 4 Hz AM
    envelope, N(0,0.01) noise, normalised to 0.1 RMS; shape [1, 1, seconds*rate]."""
    import math
    g = torch.Generator().manual_seed(seed)
    n = seconds * rate
    t = torch.arange(n, dtype=torch.float64) / rate
    f0 = 90.0 + 160.0 * torch.rand(1, generator=g, dtype=torch.float64)
    sig = sum(torch.sin(2 * math.pi * f0 * k * t) / k for k in range(1, 21))
    sig = sig * (0.6 + 0.4 * torch.sin(2 * math.pi * 4.0 * t))
    sig = sig + 0.01 * torch.randn(n, generator=g, dtype=torch.float64)
    sig = sig * (0.1 / sig.pow(2).mean().sqrt())
    return sig.float().view(1, 1, n)


def rvq_recipe(seed: int, layers: int, entries: int = 2048, dim: int = 256, hidden: int = 512):
    """Seeded residual-quantiser constants: codebook buffers as the reference's own fixture randomises them
    (embed_sum ~ N(0,1), cluster_usage ~ U[0.5,1.5); tests/conftest.py:41-53 of the reference), an input
    projection ~ N(0, 1/hidden) and embeddings are drawn by the caller from the same generator."""
    g = torch.Generator().manual_seed(seed)
    embed_sum = torch.randn(layers, entries, dim, generator=g)
    usage = torch.rand(layers, entries, generator=g) + 0.5
    proj = torch.randn(dim, hidden, generator=g) / hidden ** 0.5
    return g, embed_sum, usage, proj
