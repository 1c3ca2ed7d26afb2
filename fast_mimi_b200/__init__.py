"""B200 (sm_100a) kernels for the self-attention of Mimi's encoder / decoder transformers.

Public surface:
  MimiAttentionB200        drop-in for the reference's ``MimiAttention`` (same forward signature)
  native_window_attention  drop-in for the reference's ``_native_window_attention``
  window_attention_nlc     drop-in for the reference's long-sequence ``_window_attention_nlc`` ([B, T, 512] result)
  rope_tables              the FP32 cos / sin tables of the reference's ``MimiRotaryEmbedding``
  MimiTransformerLayerB200 drop-in for the reference's ``MimiTransformerLayer`` (whole layer on these kernels)
  MimiSplitRVQB200         encode / decode of the reference's split residual vector quantiser
  MimiDownsampleB200       the stride-2 convolution between the encoder transformer and the quantiser
  MimiUpsampleB200         the stride-2 transposed convolution between the quantiser and the decoder transformer
  MimiKVRing               streaming KV state with ``MimiKVCache``'s bookkeeping interface
  ops                      tensor-level wrappers over the C ABI (include/fast_mimi_b200.h)
  check_status             synchronise and raise if a kernel recorded an error in the device status word
"""
from . import ops
from .ops import check_status
from .attention import (MimiAttentionB200, install, native_window_attention, rope_tables, window_attention_fp32,
                        window_attention_nlc)
from .downsample import MimiDownsampleB200, MimiUpsampleB200
from .kv_ring import LinearKVCache, MimiKVRing
from .layer import MimiTransformerLayerB200, install_layers
from .rvq import MimiRVQB200, MimiSplitRVQB200
from .sharding import gather_to_host, shard, shard_bounds

__all__ = ["MimiAttentionB200", "MimiTransformerLayerB200", "install_layers", "MimiRVQB200", "MimiSplitRVQB200", "MimiDownsampleB200", "MimiUpsampleB200", "MimiKVRing", "LinearKVCache", "install", "native_window_attention",
           "window_attention_fp32", "window_attention_nlc", "rope_tables", "ops", "check_status", "shard", "shard_bounds", "gather_to_host"]
