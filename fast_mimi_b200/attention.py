"""Drop-in replacement for the reference's attention module on B200.

``MimiAttentionB200.forward`` keeps the signature and return type of the reference's
``MimiAttention.forward`` (src/fast_mimi/model.py:1870-1878) and the parameter names
``q_proj / k_proj / v_proj / o_proj`` (src/fast_mimi/model.py:1728-1747), so it can be assigned to
``layer.self_attn`` of a reference ``MimiTransformerLayer`` (call site src/fast_mimi/model.py:2051-2058)
and load the same state dict.  Two execution modes, no fallback between them:

``precision="tc"``   tensor-core path: BF16 projection GEMM with FP32 RoPE epilogue, banded tcgen05
                     attention, ring-buffer decode.  Mimi geometry only (512 / 8 heads / 64).
``precision="fp32"`` FP32 verification kernels on CUDA cores, generic in heads / head_dim / window,
                     including chunked calls with a cache.

``o_proj`` (inside the reference call's return value, src/fast_mimi/model.py:1961) runs on the same
tensor-core GEMM kernel (``ops.out_proj``); in FP32 mode it is a PyTorch linear on the kernel's FP32 output.

Cached calls (``past_key_values`` = a ``MimiKVRing``): one new frame per stream takes the ring-decode kernels,
several new frames (chunked streaming, src/fast_mimi/model.py:2176-2205) take ``ops.attention_chunk``.

The kernels never synchronise and report a timed-out device wait only through the device status word: call
``fast_mimi_b200.check_status()`` wherever the surrounding code synchronises anyway (before results leave the GPU).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .kv_ring import LinearKVCache, MimiKVRing


def native_window_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, *, scale: float,
                            window: int, value_dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """Tensor-core banded attention with the signature of the reference's ``_native_window_attention``
    (src/fast_mimi/model.py:1589-1596): rotated ``query, key`` and ``value`` shaped ``[B, 8, T, 64]``
    (any strides, any float dtype) -> attention result shaped like ``query`` in ``query.dtype``."""
    ops._need(query.dim() == 4 and query.shape[1] == ops.HEADS and query.shape[3] == ops.HEAD_DIM,
              "query must be [B, 8, T, 64]")
    ops._need(key.shape == query.shape and value.shape == query.shape, "key/value must match query")
    B, H, T, D = query.shape

    def frames(t, dtype):   # [B,H,T,D] -> contiguous [B,T,H*D] (a no-op view for the reference's layout)
        return t.transpose(1, 2).to(dtype).contiguous().view(B, T, H * D)

    out = ops.band_attention_prefill(frames(query, torch.bfloat16), frames(key, torch.bfloat16),
                                     frames(value, value_dtype), window=window, scale=scale)
    return out.view(B, T, H, D).transpose(1, 2).to(query.dtype)


def window_attention_fp32(query, key, value, *, scale, window, q_offset=0, k_offset=0):
    """FP32 verification counterpart of ``native_window_attention`` (``[B,H,T,D]`` in and out)."""
    return ops.band_attention_fp32(query.float(), key.float(), value.float(), window=window, scale=scale,
                                   q_offset=q_offset, k_offset=k_offset)


def window_attention_nlc(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, *, scale: float = 0.125,
                         window: int = 250, value_dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """Banded attention that returns the frame-major ``[B, T, 512]`` tensor ``o_proj`` consumes, as the
    reference's long-sequence helper ``_window_attention_nlc(query, key, value)`` does
    (src/fast_mimi/_optimized_runtime.py:1718-1846): rotated ``query, key`` and ``value`` shaped ``[B, 8, T, 64]``
    in, no transpose of the result (it is the kernels' native layout), result in ``query.dtype``.  Where the
    reference re-batches 64-query blocks against 320 keys, the long-clip kernel walks 128-query tiles over
    rings of K / V tiles and reads every byte once."""
    ops._need(query.dim() == 4 and query.shape[1] == ops.HEADS and query.shape[3] == ops.HEAD_DIM,
              "query must be [B, 8, T, 64]")
    ops._need(key.shape == query.shape and value.shape == query.shape, "key/value must match query")
    B, H, T, D = query.shape

    def frames(t, dtype):
        return t.transpose(1, 2).to(dtype).contiguous().view(B, T, H * D)

    out = ops.band_attention_prefill(frames(query, torch.bfloat16), frames(key, torch.bfloat16),
                                     frames(value, value_dtype), window=window, scale=scale)
    return out.to(query.dtype)


def rope_tables(position_ids: torch.Tensor, *, head_dim: int = 64, theta: float = 10000.0) -> tuple[torch.Tensor, torch.Tensor]:
    """The ``position_embeddings`` pair the attention entry points take: FP32 ``cos, sin`` shaped
    ``[batch, frames, head_dim]`` for absolute ``position_ids [batch, frames]``, computed like the reference's
    ``MimiRotaryEmbedding.forward`` (src/fast_mimi/model.py:1499-1535): ``inv_freq = theta^(-2j/head_dim)`` in
    FP32, frequencies by an FP32 product with autocast off, both halves of the table equal."""
    ops._need(position_ids.dim() == 2, "position_ids must be [batch, frames]")
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    inv_freq = inv_freq.to(position_ids.device)
    with torch.autocast(device_type=position_ids.device.type, enabled=False):
        freqs = position_ids.float()[:, :, None] * inv_freq[None, None, :]
        emb = torch.cat((freqs, freqs), dim=-1)
        return emb.cos().contiguous(), emb.sin().contiguous()


class MimiAttentionB200(nn.Module):
    def __init__(self, hidden_size: int = 512, num_heads: int = 8, head_dim: int = 64, sliding_window: int = 250,
                 layer_idx: int = 0, precision: str = "tc", value_dtype: torch.dtype = torch.float16,
                 input_dtype: torch.dtype | None = None) -> None:
        super().__init__()
        if precision not in ("tc", "fp32"):
            raise ValueError("precision must be 'tc' or 'fp32'")
        if precision == "tc" and (hidden_size, num_heads, head_dim) != (512, 8, 64):
            raise ValueError("the tensor-core path is built for hidden 512, 8 heads of 64")
        self.layer_idx = layer_idx
        self.num_heads = num_heads
        self.num_key_value_heads = num_heads       # GQA groups = 1 (src/fast_mimi/config.py:108-109)
        self.head_dim = head_dim
        self.scaling = 1.0 / math.sqrt(head_dim)
        self.sliding_window = sliding_window
        self.precision = precision
        self.value_dtype = value_dtype
        # Type in which activations and the packed projection weight reach the tensor core.  None = FP16
        # for FP32 / FP16 callers (8x finer rounding than BF16 at the same rate; LayerNorm-ed activations
        # and weights are far inside its range) and BF16 for BF16 callers.
        self.input_dtype = input_dtype
        self.q_proj = nn.Linear(hidden_size, num_heads * head_dim, bias=False)
        self.k_proj = nn.Linear(hidden_size, num_heads * head_dim, bias=False)
        self.v_proj = nn.Linear(hidden_size, num_heads * head_dim, bias=False)
        self.o_proj = nn.Linear(num_heads * head_dim, hidden_size, bias=False)
        self._packed: torch.Tensor | None = None
        self._packed_key: tuple | None = None
        self._wo16: torch.Tensor | None = None
        self._wo16_key: tuple | None = None

    @classmethod
    def from_reference(cls, attn: nn.Module, precision: str = "tc",
                       value_dtype: torch.dtype = torch.float16) -> "MimiAttentionB200":
        """Build from a module that has the reference's attributes; the four projections are shared,
        not copied, so the surrounding model's state dict is unchanged."""
        if getattr(attn, "num_key_value_groups", 1) != 1:
            raise ValueError("grouped-query attention is not part of Mimi's configuration")
        if attn.q_proj.bias is not None:
            raise ValueError("attention projections must be bias-free")
        new = cls(attn.q_proj.in_features, attn.num_heads, attn.head_dim, attn.sliding_window, attn.layer_idx,
                  precision, value_dtype)
        new.q_proj, new.k_proj, new.v_proj, new.o_proj = attn.q_proj, attn.k_proj, attn.v_proj, attn.o_proj
        return new

    def new_cache(self, num_layers: int, num_streams: int, device) -> MimiKVRing | LinearKVCache:
        if self.precision == "tc":
            return MimiKVRing(num_layers, num_streams, self.sliding_window, device=device,
                              value_dtype=self.value_dtype)
        return LinearKVCache(num_layers, self.sliding_window)

    def packed_qkv_weight(self, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """``cat(Wq, Wk, Wv)`` as a 16-bit ``[1536, 512]`` tensor, rebuilt when a projection weight changes
        (the reference packs once the same way: src/fast_mimi/_packed_qkv.py:139-150)."""
        ws = (self.q_proj.weight, self.k_proj.weight, self.v_proj.weight)
        key = tuple((w.data_ptr(), w._version, w.device) for w in ws) + (dtype,)
        if self._packed is None or self._packed_key != key:
            self._packed = torch.cat([w.detach() for w in ws], dim=0).to(dtype).contiguous()
            self._packed_key = key
        return self._packed

    def out_weight(self, dtype: torch.dtype) -> torch.Tensor:
        """``o_proj.weight`` as a 16-bit tensor, rebuilt when the weight changes."""
        w = self.o_proj.weight
        key = (w.data_ptr(), w._version, w.device, dtype)
        if self._wo16 is None or self._wo16_key != key:
            self._wo16 = w.detach().to(dtype).contiguous()
            self._wo16_key = key
        return self._wo16

    def _tc_input_dtype(self, hidden_states: torch.Tensor) -> torch.dtype:
        if self.input_dtype is not None:
            return self.input_dtype
        return torch.bfloat16 if hidden_states.dtype == torch.bfloat16 else torch.float16

    # -------------------------------------------------------------------------------------------
    def forward(self, hidden_states: torch.Tensor, attention_mask: torch.Tensor | None, past_key_values,
                position_embeddings: tuple[torch.Tensor, torch.Tensor], output_attentions: bool = False,
                canonical_window_mask: bool = False) -> tuple[torch.Tensor, torch.Tensor | None]:
        if output_attentions:
            raise RuntimeError("attention probabilities are not materialised by the B200 kernels")
        if not hidden_states.is_cuda:
            raise RuntimeError("MimiAttentionB200 runs on a CUDA device only; there is no CPU path")
        if attention_mask is not None and attention_mask.dim() != 4:
            raise RuntimeError("key-padding masks are not supported; pass None or the 4-D causal band mask")
        # A 4-D mask is the caller's dense rendering of the causal band (src/fast_mimi/model.py:2194-2205);
        # the kernels derive the same band from positions and never read it.
        cos, sin = position_embeddings
        if self.precision == "fp32":
            core = self._forward_fp32(hidden_states, past_key_values, cos, sin)
        else:
            core = self._forward_tc(hidden_states, past_key_values, cos, sin)
            if self.o_proj.bias is None:
                # the kernels' 16-bit result feeds the output projection as it is (the one-frame decode kernel
                # returns FP32, rounded here once)
                if core.dtype not in ops._VALUE_CODES:
                    core = core.to(self.value_dtype)
                out_dtype = hidden_states.dtype if hidden_states.dtype in ops._VALUE_CODES else torch.float16
                out = ops.out_proj(core, self.out_weight(core.dtype), out_dtype=out_dtype)
                return out.to(hidden_states.dtype), None
        return self.o_proj(core.to(self.o_proj.weight.dtype)), None

    def _forward_tc(self, hidden_states, cache, cos, sin):
        B, T, _ = hidden_states.shape
        in_dtype = self._tc_input_dtype(hidden_states)
        x = hidden_states.to(in_dtype).contiguous()
        cos = cos.to(torch.float32).contiguous()
        sin = sin.to(torch.float32).contiguous()
        w = self.packed_qkv_weight(in_dtype)
        if cache is None:
            return ops.attention_prefill(x, w, cos, sin, window=self.sliding_window, scale=self.scaling,
                                         value_dtype=self.value_dtype)
        if not isinstance(cache, MimiKVRing):
            return self._forward_tc_foreign_cache(x, w, cos, sin, cache)
        ops._need(cache.num_streams == B, "cache was created for a different number of streams")
        ops._need(cache.sliding_window == self.sliding_window, "cache window differs from the module's")
        pos = cache.get_seq_length(self.layer_idx)
        ring_k, ring_v = cache.ring_k[self.layer_idx], cache.ring_v[self.layer_idx]
        if T == 1:
            out = ops.decode_step(x.view(B, 512), w, cos, sin, ring_k, ring_v, pos, scale=self.scaling)
        else:
            # several new frames on top of the cache: chunked streaming (src/fast_mimi/model.py:2176-2205)
            out = ops.attention_chunk(x, w, cos, sin, ring_k, ring_v, pos, window=self.sliding_window,
                                      scale=self.scaling)
        cache.advance(self.layer_idx, T)
        return out.view(B, T, 512)

    def _forward_tc_foreign_cache(self, x, w, cos, sin, cache):
        """A cache object that is not a ``MimiKVRing`` but speaks the reference's ``MimiKVCache`` protocol
        (``get_seq_length``, ``update`` returning the visible K / V: src/fast_mimi/model.py:435-471), e.g. the cache
        ``MimiTransformerModel.forward`` creates by itself under ``use_cache=True``.  Projection and attention run on
        the tensor-core kernels; the cache keeps its own storage (its rotated K / V are the kernels' 16-bit values,
        so nothing is rounded twice) and the visible rows are laid out frame-major for the attention kernel by
        PyTorch copies.  Slower than the ring (the reference's concatenate-and-crop stays), same results."""
        if not (hasattr(cache, "update") and hasattr(cache, "get_seq_length")):
            raise RuntimeError("past_key_values must be a MimiKVRing or offer MimiKVCache's update / get_seq_length")
        B, T, _ = x.shape
        q, k, v = ops.qkv_rope(x, w, cos, sin, value_dtype=self.value_dtype)
        heads = lambda t: t.view(B, T, self.num_heads, self.head_dim).transpose(1, 2)
        k_all, v_all = cache.update(heads(k).float(), heads(v).float(), self.layer_idx)     # [B, 8, Tk, 64]
        Tk = k_all.shape[2]
        frames = lambda t, dt: t.transpose(1, 2).reshape(B, Tk, self.num_heads * self.head_dim).to(dt).contiguous()
        return ops.band_attention_chunk(q, frames(k_all, torch.bfloat16), frames(v_all, self.value_dtype),
                                        window=self.sliding_window, scale=self.scaling)

    def _forward_fp32(self, hidden_states, cache, cos, sin):
        B, T, _ = hidden_states.shape
        H, D = self.num_heads, self.head_dim
        x = hidden_states.float()
        q = ops.linear_fp32(x, self.q_proj.weight.float()).view(B, T, H, D)
        k = ops.linear_fp32(x, self.k_proj.weight.float()).view(B, T, H, D)
        v = ops.linear_fp32(x, self.v_proj.weight.float()).view(B, T, H, D)
        ops.rope_fp32_(q, cos, sin)
        ops.rope_fp32_(k, cos, sin)
        q_off = k_off = 0
        if cache is not None:
            if not isinstance(cache, LinearKVCache):
                raise RuntimeError("the FP32 verification path needs a LinearKVCache (see new_cache)")
            q_off = cache.get_seq_length(self.layer_idx)
            k_off = max(q_off - self.sliding_window + 1, 0)
            k, v = cache.update(k, v, self.layer_idx)
        out = ops.band_attention_fp32(q, k, v, window=self.sliding_window, scale=self.scaling, q_offset=q_off,
                                      k_offset=k_off, frame_major=True)
        return out.view(B, T, H * D).to(hidden_states.dtype)


def install(transformer: nn.Module, precision: str = "tc", value_dtype: torch.dtype = torch.float16) -> nn.Module:
    """Swap ``layer.self_attn`` of every layer of a reference-style transformer stack (an object with a
    ``layers`` ModuleList whose items have ``self_attn``) for ``MimiAttentionB200``."""
    for layer in transformer.layers:
        layer.self_attn = MimiAttentionB200.from_reference(layer.self_attn, precision, value_dtype)
    return transformer
