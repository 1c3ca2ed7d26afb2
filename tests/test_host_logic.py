"""CPU-side tests: ABI surface, loader behaviour, ring bookkeeping, sharding (incl. 2-rank gloo)."""
from __future__ import annotations

import ctypes
import os
import re
import subprocess
import sys

import pytest
import torch

from conftest import ROOT


def _header_functions():
    text = open(os.path.join(ROOT, "include", "fast_mimi_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"\bint\s+(fm_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S)


def test_library_exports_every_declared_symbol():
    from fast_mimi_b200 import _build, _native
    if not os.path.exists(_build.LIB_PATH):
        _build.build()
    lib = ctypes.CDLL(_build.LIB_PATH)      # loading needs no GPU
    declared = _header_functions()
    assert len(declared) >= 10
    for name, args in declared:
        assert hasattr(lib, name), name
        assert name in _native.SIGNATURES, name
        n_args = 0 if args.strip() in ("", "void") else len(args.split(","))
        assert n_args == len(_native.SIGNATURES[name]), name
    assert set(_native.SIGNATURES) == {n for n, _ in declared}
    lib.fm_abi_version.restype = ctypes.c_int
    assert lib.fm_abi_version() == 2


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from fast_mimi_b200 import _native
    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setattr(_native, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(_native.NativeLibraryMissing):
        _native.load()


def test_no_product_module_imports_the_oracle():
    for dirpath, _, files in os.walk(os.path.join(ROOT, "fast_mimi_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.replace("oracle's", ""), f


def test_ring_bookkeeping_matches_reference_cache_semantics():
    """get_seq_length / get_mask_sizes must equal MimiKVCache's (src/fast_mimi/model.py:473-505), which
    the oracle restates and the golden fixtures pin."""
    from fast_mimi_b200 import MimiKVRing
    from oracle.mimi_attention_oracle import KVCacheOracle
    ring = MimiKVRing(2, 3, 8, device="cpu")
    ref = KVCacheOracle(window=8)
    for step, t in enumerate([1, 1, 3, 1, 9, 1, 1]):
        assert ring.get_mask_sizes(t) == ref.get_mask_sizes(t)
        kv = torch.zeros(3, 8, t, 64)
        ref.update(kv, kv, 0)
        ring.advance(0, t)
        assert ring.get_seq_length() == ref.get_seq_length()
    assert ring.get_seq_length(5) == 0
    with pytest.raises(ValueError):
        ring.configure_sliding_window(9)
    with pytest.raises(ValueError):
        MimiKVRing(1, 1, 257, device="cpu")


def test_ring_ordered_view_wraps():
    from fast_mimi_b200 import MimiKVRing
    ring = MimiKVRing(1, 1, 4, device="cpu")
    for pos in range(6):
        ring.ring_k[0][:, :, pos % 4] = pos
        ring.advance(0, 1)
    k, _ = ring.ordered(0)
    assert k[0, 0, :, 0].tolist() == [2, 3, 4, 5]


def test_shard_bounds_cover_everything_once():
    from fast_mimi_b200 import shard_bounds
    for n in (0, 1, 7, 16, 512, 4096):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_bounds(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


_GLOO_WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["FM_ROOT"])
from fast_mimi_b200 import shard, gather_to_host
from oracle import mimi_attention_oracle as O
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
g = torch.Generator().manual_seed(0)
q, k, v = (torch.randn(5, 8, 40, 64, generator=g) for _ in range(3))   # 5 clips over 2 ranks: 3 + 2
mine = O.band_attention(shard(q, world, rank), shard(k, world, rank), shard(v, world, rank), window=16)
full = gather_to_host(mine)
if rank == 0:
    ref = O.band_attention(q, k, v, window=16)
    assert full.shape == ref.shape and torch.equal(full, ref)
    print("GLOO_OK")
dist.destroy_process_group()
"""


def test_two_rank_clip_sharding_and_host_gather_over_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_GLOO_WORKER)
    env = dict(os.environ, FM_ROOT=ROOT, OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29617", str(script)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert res.returncode == 0, res.stderr[-2000:]
    assert "GLOO_OK" in res.stdout


def test_layer_module_keeps_the_reference_parameter_names():
    """State-dict keys of the drop-in layer are those of the reference's MimiTransformerLayer
    (src/fast_mimi/model.py:2017-2026 with MimiAttention :1728-1747, MimiMLP :1987-1988, MimiLayerScale :1468)."""
    import fast_mimi_b200 as fm
    want = {"self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.o_proj.weight",
            "mlp.fc1.weight", "mlp.fc2.weight", "input_layernorm.weight", "input_layernorm.bias",
            "post_attention_layernorm.weight", "post_attention_layernorm.bias", "self_attn_layer_scale.scale",
            "mlp_layer_scale.scale"}
    layer = fm.MimiTransformerLayerB200()
    assert set(layer.state_dict()) == want
    import pytest
    import torch
    with pytest.raises(RuntimeError):        # no CPU path
        layer(torch.zeros(1, 4, 512), None, None, (torch.zeros(1, 4, 64), torch.zeros(1, 4, 64)), False)


def test_rope_tables_match_the_oracle():
    """fast_mimi_b200.rope_tables against the oracle's restatement (which the fixtures pin to the tables of the
    reference's MimiRotaryEmbedding), including non-zero and per-clip position offsets."""
    import torch
    import fast_mimi_b200 as fm
    from oracle import mimi_attention_oracle as O
    pos = torch.stack([torch.arange(0, 40), torch.arange(1000, 1040)])
    cos, sin = fm.rope_tables(pos)
    assert cos.shape == (2, 40, 64) and cos.dtype == torch.float32
    for b in range(2):
        oc, os_ = O.rope_tables(pos[b])
        assert torch.equal(cos[b], oc) and torch.equal(sin[b], os_)
    assert torch.equal(cos[..., :32], cos[..., 32:])
