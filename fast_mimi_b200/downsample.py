"""Drop-ins for the two stride-2 convolutions around the quantiser.

``MimiUpsampleB200`` replaces ``MimiModel.upsample`` (``MimiConvTranspose1d(512, 512, kernel 4, stride 2, groups=512,
bias=False)``, src/fast_mimi/model.py:2745-2753): one channel per group makes it elementwise.

``MimiDownsampleB200`` replaces ``MimiModel.downsample`` (the stride-2 convolution between the encoder transformer and
the quantiser: ``MimiConv1d(512, 512, kernel 4, stride 2, bias=False, pad_mode="replicate")``,
src/fast_mimi/model.py:2734-2744) on B200.

``MimiDownsampleB200(conv)(hidden_states [B, C, T], padding_cache=None) -> [B, C_out, ceil(T / 2)]`` keeps the call
signature of ``MimiConv1d.forward`` for the offline (cache-free) case; ``frames`` is the same computation on the
frame-major ``[B, T, C]`` tensor the transformer produces, which avoids both transposes.  Streaming calls with a
padding cache are not implemented here and raise.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import ops


class MimiDownsampleB200(nn.Module):
    def __init__(self, conv: nn.Module) -> None:
        """``conv``: a module with the reference's ``MimiConv1d`` attributes (``conv`` = ``nn.Conv1d``, ``causal``,
        ``pad_mode``); its weight is shared, not copied."""
        super().__init__()
        inner = conv.conv
        if inner.bias is not None or inner.groups != 1 or inner.dilation[0] != 1:
            raise ValueError("the downsampling convolution must be dense, undilated and bias-free")
        if not getattr(conv, "causal", True) or getattr(conv, "pad_mode", "replicate") != "replicate":
            raise ValueError("only the causal, replicate-padded form of Mimi's configuration is built")
        self.conv = inner
        self.kernel, self.stride = inner.kernel_size[0], inner.stride[0]
        self._parts = None
        self._key = None

    def _weight_parts(self):
        w = self.conv.weight
        key = (w.data_ptr(), w._version, w.device)
        if self._parts is None or self._key != key:
            # W2[c_out, j * C + c_in] = W[c_out, c_in, j]: the row layout of ops.downsample_conv
            w2 = w.detach().float().permute(0, 2, 1).reshape(w.shape[0], -1).contiguous()
            self._parts, self._key = ops.split_half(w2), key
        return self._parts

    def frames(self, x: torch.Tensor) -> torch.Tensor:
        """``x [B, T, C]`` (frame-major) -> ``[B, ceil(T / stride), C_out]`` float32."""
        return ops.downsample_conv(x.float().contiguous(), self._weight_parts(), kernel=self.kernel, stride=self.stride)

    def forward(self, hidden_states: torch.Tensor, padding_cache=None) -> torch.Tensor:
        if padding_cache is not None:
            raise RuntimeError("streaming (padding-cache) calls of the downsampling convolution are not built")
        if not hidden_states.is_cuda:
            raise RuntimeError("MimiDownsampleB200 runs on a CUDA device only; there is no CPU path")
        y = self.frames(hidden_states.transpose(1, 2))
        return y.transpose(1, 2).to(hidden_states.dtype)


class MimiUpsampleB200(nn.Module):
    def __init__(self, convtr: nn.Module) -> None:
        """``convtr``: a module with the reference's ``MimiConvTranspose1d`` attributes (``conv`` =
        ``nn.ConvTranspose1d``, ``padding_left`` / ``padding_right``); its weight is shared, not copied."""
        super().__init__()
        inner = convtr.conv
        c = inner.in_channels
        if (inner.bias is not None or inner.groups != c or inner.out_channels != c or inner.kernel_size[0] != 4
                or inner.stride[0] != 2):
            raise ValueError("only Mimi's depthwise, bias-free transposed convolution (kernel 4, stride 2) is built")
        if getattr(convtr, "padding_left", 0) != 0 or getattr(convtr, "padding_right", 2) != 2:
            raise ValueError("only the causal trimming of Mimi's configuration (two trailing frames) is built")
        self.conv = inner

    def frames(self, x: torch.Tensor) -> torch.Tensor:
        """``x [B, T, C]`` (frame-major) -> ``[B, 2T, C]`` float32."""
        w = self.conv.weight.detach().float().reshape(self.conv.in_channels, 4).contiguous()
        return ops.upsample2(x.float().contiguous(), w)

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        if not hidden_states.is_cuda:
            raise RuntimeError("MimiUpsampleB200 runs on a CUDA device only; there is no CPU path")
        return self.frames(hidden_states.transpose(1, 2)).transpose(1, 2).to(hidden_states.dtype)
