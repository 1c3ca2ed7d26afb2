"""Drop-in replacement for the reference's transformer layer on B200.

``MimiTransformerLayerB200.forward`` keeps the signature and return type of the reference's
``MimiTransformerLayer.forward`` (src/fast_mimi/model.py:2026-2061) and its sub-module names
(``self_attn``, ``mlp.fc1``, ``mlp.fc2``, ``input_layernorm``, ``post_attention_layernorm``,
``self_attn_layer_scale.scale``, ``mlp_layer_scale.scale``), so state dicts are interchangeable.

The whole layer runs on this package's kernels, six launches for a call without cache on clips of 129-256 frames
(seven for other lengths, where projection + RoPE and the attention are two kernels):

    LayerNorm -> QKV projection + RoPE + banded attention -> o_proj + layer scale + residual
              -> LayerNorm -> fc1 + GELU -> fc2 + layer scale + residual

The residual stream keeps the caller's dtype (FP32 stays FP32: both residual adds happen in the FP32 epilogue
of a GEMM); only the operands of the tensor-core products are rounded to 16 bit.  Calls with a cache (a
``MimiKVRing``) differ only in the attention core: ring decode for one new frame per stream, the chunk path for
several; LayerNorms, projections and the MLP are the same kernels.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .attention import MimiAttentionB200


class _LayerScale(nn.Module):
    """Per-channel factor, as the reference's ``MimiLayerScale`` (src/fast_mimi/model.py:1454-1480)."""

    def __init__(self, channels: int, initial: float = 0.01) -> None:
        super().__init__()
        self.scale = nn.Parameter(torch.full((channels,), initial))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.scale * x


class _MLP(nn.Module):
    """``fc2(gelu(fc1(x)))`` with bias-free linears (src/fast_mimi/model.py:1987-1999)."""

    def __init__(self, hidden: int, intermediate: int) -> None:
        super().__init__()
        self.fc1 = nn.Linear(hidden, intermediate, bias=False)
        self.fc2 = nn.Linear(intermediate, hidden, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.fc2(F.gelu(self.fc1(x)))


class _Cast16:
    """16-bit copies of parameters, rebuilt when the parameter (or the requested type) changes."""

    def __init__(self) -> None:
        self._store: dict = {}

    def get(self, name: str, p: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        key = (p.data_ptr(), p._version, p.device, dtype)
        hit = self._store.get(name)
        if hit is None or hit[0] != key:
            hit = (key, p.detach().to(dtype).contiguous())
            self._store[name] = hit
        return hit[1]


class MimiTransformerLayerB200(nn.Module):
    def __init__(self, hidden_size: int = 512, intermediate_size: int = 2048, num_heads: int = 8, head_dim: int = 64,
                 sliding_window: int = 250, layer_idx: int = 0, norm_eps: float = 1e-5,
                 layer_scale_initial_scale: float = 0.01, value_dtype: torch.dtype = torch.float16) -> None:
        super().__init__()
        self.self_attn = MimiAttentionB200(hidden_size, num_heads, head_dim, sliding_window, layer_idx, "tc", value_dtype)
        self.mlp = _MLP(hidden_size, intermediate_size)
        self.input_layernorm = nn.LayerNorm(hidden_size, eps=norm_eps)
        self.post_attention_layernorm = nn.LayerNorm(hidden_size, eps=norm_eps)
        self.self_attn_layer_scale = _LayerScale(hidden_size, layer_scale_initial_scale)
        self.mlp_layer_scale = _LayerScale(hidden_size, layer_scale_initial_scale)
        self._cast = _Cast16()

    @classmethod
    def from_reference(cls, layer: nn.Module, value_dtype: torch.dtype = torch.float16) -> "MimiTransformerLayerB200":
        """Build from a module with the reference layer's attributes; every parameter is shared, not copied."""
        attn = layer.self_attn
        new = cls(attn.q_proj.in_features, layer.mlp.fc1.out_features, attn.num_heads, attn.head_dim,
                  attn.sliding_window, attn.layer_idx, layer.input_layernorm.eps, value_dtype=value_dtype)
        new.self_attn = attn if isinstance(attn, MimiAttentionB200) else MimiAttentionB200.from_reference(
            attn, "tc", value_dtype)
        new.mlp = layer.mlp
        new.input_layernorm = layer.input_layernorm
        new.post_attention_layernorm = layer.post_attention_layernorm
        new.self_attn_layer_scale = layer.self_attn_layer_scale
        new.mlp_layer_scale = layer.mlp_layer_scale
        return new

    def forward(self, hidden_states: torch.Tensor, attention_mask: torch.Tensor | None, past_key_values,
                position_embeddings: tuple[torch.Tensor, torch.Tensor], output_attentions: bool = False,
                canonical_window_mask: bool = False) -> tuple[torch.Tensor, torch.Tensor | None]:
        if output_attentions:
            raise RuntimeError("attention probabilities are not materialised by the B200 kernels")
        if not hidden_states.is_cuda:
            raise RuntimeError("MimiTransformerLayerB200 runs on a CUDA device only; there is no CPU path")
        if attention_mask is not None and attention_mask.dim() != 4:
            raise RuntimeError("key-padding masks are not supported; pass None or the 4-D causal band mask")
        if self.mlp.fc1.bias is not None or self.self_attn.o_proj.bias is not None:
            raise RuntimeError("the fused layer expects bias-free projections, as in Mimi's checkpoints")
        attn = self.self_attn
        x = hidden_states.contiguous()
        stream_dtype = x.dtype
        tc = attn._tc_input_dtype(x)
        cos, sin = (t.to(torch.float32).contiguous() for t in position_embeddings)
        ln1, ln2 = self.input_layernorm, self.post_attention_layernorm
        f32 = lambda p: p.detach().float().contiguous()       # no copy for FP32 parameters
        h = ops.layer_norm(x, f32(ln1.weight), f32(ln1.bias), eps=ln1.eps, out_dtype=tc)
        if past_key_values is None:
            core = ops.attention_prefill(h, attn.packed_qkv_weight(tc), cos, sin, window=attn.sliding_window,
                                         scale=attn.scaling, value_dtype=attn.value_dtype)
        else:
            core = attn._forward_tc(h, past_key_values, cos, sin)      # ring decode (FP32 result) or chunk path
            if core.dtype not in ops._VALUE_CODES:
                core = core.to(attn.value_dtype)
        x1 = ops.linear(core, attn.out_weight(core.dtype), scale=f32(self.self_attn_layer_scale.scale), residual=x,
                        out_dtype=stream_dtype)
        h2 = ops.layer_norm(x1, f32(ln2.weight), f32(ln2.bias), eps=ln2.eps, out_dtype=tc)
        g = ops.linear(h2, self._cast.get("fc1", self.mlp.fc1.weight, tc), activation="gelu", out_dtype=tc)
        x2 = ops.linear(g, self._cast.get("fc2", self.mlp.fc2.weight, tc), scale=f32(self.mlp_layer_scale.scale),
                        residual=x1, out_dtype=stream_dtype)
        return x2, None


def install_layers(transformer: nn.Module, value_dtype: torch.dtype = torch.float16) -> nn.Module:
    """Replace every layer of a reference ``MimiTransformerModel`` (its ``layers`` ModuleList,
    src/fast_mimi/model.py:2064-2232) by a ``MimiTransformerLayerB200`` that shares its parameters."""
    for i, layer in enumerate(transformer.layers):
        transformer.layers[i] = MimiTransformerLayerB200.from_reference(layer, value_dtype)
    return transformer
