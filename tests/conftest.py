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


def regen_projections(seed: int, hidden: int = 512, std: float = 0.02):
    """Rebuild the seeded weights of ``tests/golden/make_golden.py`` without the reference: four
    bias-free Linear(hidden, hidden) constructed in q,k,v,o order (their default init consumes the
    RNG), re-initialised N(0, std^2) in the same order; q/k/v weights rounded to BF16-representable
    values as the generator does for the full-size fixtures.  Leaves the RNG where x is drawn next."""
    torch.manual_seed(seed)
    lins = [torch.nn.Linear(hidden, hidden, bias=False) for _ in range(4)]
    for lin in lins:
        torch.nn.init.normal_(lin.weight, std=std)
    wq, wk, wv, wo = (lin.weight.detach() for lin in lins)
    return wq.bfloat16().float(), wk.bfloat16().float(), wv.bfloat16().float(), wo


def regen_attention_layer(seed: int, b: int, t: int, hidden: int = 512, std: float = 0.02):
    """Weights as ``regen_projections`` then x ~ N(0,1) rounded to BF16-representable values."""
    wq, wk, wv, wo = regen_projections(seed, hidden, std)
    x = torch.randn(b, t, hidden).bfloat16().float()
    return x, wq, wk, wv, wo
