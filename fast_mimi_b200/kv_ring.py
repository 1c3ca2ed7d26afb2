"""Per-stream KV ring: the streaming state of the attention path.

Host-side mirror of the reference's ``MimiKVCache`` (src/fast_mimi/model.py:363-522) with the same
bookkeeping interface (``get_seq_length``, ``get_mask_sizes``, ``configure_sliding_window``) so that
``MimiTransformerModel.forward`` (src/fast_mimi/model.py:2176-2191) can drive it unchanged.  Storage
differs: instead of concatenating and cropping ``window-1`` rows every step, each layer owns a ring of
``window`` slots per (stream, head), ``[streams, 8, window, 64]``, and the frame at absolute position p
lives in slot ``p % window``.  The projection kernel writes the slot; nothing is copied or shifted.
"""
from __future__ import annotations

import torch


class MimiKVRing:
    def __init__(self, num_layers: int, num_streams: int, sliding_window: int = 250, *,
                 device: torch.device | str = "cuda", value_dtype: torch.dtype = torch.float16,
                 num_heads: int = 8, head_dim: int = 64) -> None:
        if sliding_window <= 0:
            raise ValueError("sliding_window must be positive")
        if sliding_window > 256:
            raise ValueError("the ring decode kernel supports windows of at most 256 frames")
        if value_dtype not in (torch.float16, torch.bfloat16):
            raise ValueError("value_dtype must be torch.float16 or torch.bfloat16")
        self.sliding_window = sliding_window
        self.num_layers = num_layers
        self.num_streams = num_streams
        self.value_dtype = value_dtype
        shape = (num_layers, num_streams, num_heads, sliding_window, head_dim)
        # Zero-filled so that no slot ever holds a non-finite bit pattern.
        self.ring_k = torch.zeros(shape, dtype=torch.bfloat16, device=device)
        self.ring_v = torch.zeros(shape, dtype=value_dtype, device=device)
        self._cumulative_lengths = [0] * num_layers

    # ---- bookkeeping with MimiKVCache's semantics -------------------------------------------
    def configure_sliding_window(self, sliding_window: int) -> None:
        if sliding_window != self.sliding_window:
            raise ValueError("cache sliding_window does not match the model configuration")

    def get_seq_length(self, layer_idx: int = 0) -> int:
        if layer_idx >= len(self._cumulative_lengths):
            return 0
        return self._cumulative_lengths[layer_idx]

    def get_mask_sizes(self, query_length: int, layer_idx: int = 0) -> tuple[int, int]:
        cumulative = self.get_seq_length(layer_idx)
        key_offset = max(cumulative - self.sliding_window + 1, 0)
        if cumulative >= self.sliding_window:
            return self.sliding_window - 1 + query_length, key_offset
        return cumulative + query_length, key_offset

    def advance(self, layer_idx: int, frames: int) -> None:
        self._cumulative_lengths[layer_idx] += frames

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int) -> tuple[torch.Tensor, torch.Tensor]:
        """``MimiKVCache.update`` (src/fast_mimi/model.py:435-471) on ring storage, for a caller that projects and
        rotates K / V itself (the reference's own attention module): ``key_states, value_states [streams, 8, T, 64]``
        are the call's new rows; returns the visible rows for this call (the newest ``window - 1`` cached rows in
        position order, then the new rows), in the callers' dtype, and stores the new rows in their slots.  The
        B200 attention module does not go through here: its kernels write the ring themselves."""
        past = self.get_seq_length(layer_idx)
        w = self.sliding_window
        T = key_states.shape[2]
        keep = min(past, w - 1)
        old = (torch.arange(past - keep, past, device=self.ring_k.device) % w)
        k_old = self.ring_k[layer_idx][:, :, old].to(key_states.dtype)
        v_old = self.ring_v[layer_idx][:, :, old].to(value_states.dtype)
        first = max(T - w, 0)
        slots = (torch.arange(past + first, past + T, device=self.ring_k.device) % w)
        self.ring_k[layer_idx][:, :, slots] = key_states[:, :, first:].to(self.ring_k.dtype)
        self.ring_v[layer_idx][:, :, slots] = value_states[:, :, first:].to(self.ring_v.dtype)
        self.advance(layer_idx, T)
        return torch.cat((k_old, key_states), dim=2), torch.cat((v_old, value_states), dim=2)

    def to(self, device) -> "MimiKVRing":
        """Move the rings to ``device`` (``MimiKVCache.to``, src/fast_mimi/model.py:507)."""
        self.ring_k = self.ring_k.to(device)
        self.ring_v = self.ring_v.to(device)
        return self

    def reset(self) -> None:
        self._cumulative_lengths = [0] * self.num_layers

    # ---- views used by tests --------------------------------------------------------------
    def ordered(self, layer_idx: int) -> tuple[torch.Tensor, torch.Tensor]:
        """K and V of one layer in position order, ``[streams, 8, n, 64]`` with n = min(len, window):
        what the reference's cache plus the newest row would hold."""
        n = self.get_seq_length(layer_idx)
        w = self.sliding_window
        if n <= w:
            idx = torch.arange(n, device=self.ring_k.device)
        else:
            idx = torch.arange(n - w, n, device=self.ring_k.device) % w
        return self.ring_k[layer_idx][:, :, idx], self.ring_v[layer_idx][:, :, idx]

    def bytes(self) -> int:
        return self.ring_k.numel() * 2 + self.ring_v.numel() * 2


class LinearKVCache:
    """FP32 cache with the reference's physical layout (last window-1 rotated rows, concatenated with
    the new rows per call) for the FP32 verification path; semantics of
    src/fast_mimi/model.py:435-505."""

    def __init__(self, num_layers: int, sliding_window: int) -> None:
        self.sliding_window = sliding_window
        self.key_cache: list[torch.Tensor | None] = [None] * num_layers
        self.value_cache: list[torch.Tensor | None] = [None] * num_layers
        self._cumulative_lengths = [0] * num_layers

    def configure_sliding_window(self, sliding_window: int) -> None:
        if sliding_window != self.sliding_window:
            raise ValueError("cache sliding_window does not match the model configuration")

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self._cumulative_lengths[layer_idx] if layer_idx < len(self._cumulative_lengths) else 0

    def get_mask_sizes(self, query_length: int, layer_idx: int = 0) -> tuple[int, int]:
        cumulative = self.get_seq_length(layer_idx)
        key_offset = max(cumulative - self.sliding_window + 1, 0)
        if cumulative >= self.sliding_window:
            return self.sliding_window - 1 + query_length, key_offset
        return cumulative + query_length, key_offset

    def update(self, key: torch.Tensor, value: torch.Tensor, layer_idx: int):
        """``key``/``value`` are ``[B, T, H, D]`` (frame-major).  Returns the visible K/V."""
        new = key.shape[1]
        if self.key_cache[layer_idx] is not None:
            key = torch.cat((self.key_cache[layer_idx], key), dim=1)
            value = torch.cat((self.value_cache[layer_idx], value), dim=1)
        self._cumulative_lengths[layer_idx] += new
        keep = self.sliding_window - 1
        self.key_cache[layer_idx] = key[:, -keep:] if keep > 0 else key[:, :0]
        self.value_cache[layer_idx] = value[:, -keep:] if keep > 0 else value[:, :0]
        return key.contiguous(), value.contiguous()
