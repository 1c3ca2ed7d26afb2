"""benchmark config 1 end to end: full Mimi encode (SEANet -> 8-layer transformer -> downsample -> RVQ,
8 codebooks) of 5 s of synthetic audio (and of 10 s and 12 s, which reach the other attention kernels) with the
B200 attention, or the whole B200 transformer layer, swapped into every encoder-transformer layer; RVQ code
frames must match the reference's CPU result (tests/golden/e2e_codes_*s.npz) on >= 99.5 % of frames (a frame
counts only if all 8 codes agree).

The reference checkout is not on the GPU box.  The surrounding model therefore comes from HF Transformers
(library code; the reference's own tests pin themselves bit-exactly to it, tests/test_parity.py:12-29 of the
reference), loaded with the same key-order weight recipe as the fixture; the generator script checked that
HF, the reference module path and the reference functional runtime give identical codes on CPU.
"""
from __future__ import annotations

import pytest
import torch
import torch.nn as nn

from conftest import fill_state_by_recipe, load_golden, synthetic_audio

pytestmark = pytest.mark.gpu


class _HFAttentionAdapter(nn.Module):
    """HF's layer calls self_attn(hidden_states=..., attention_mask=..., position_ids=..., ...) and builds
    the rotary tables inside the attention; the reference (and MimiAttentionB200) receives them from the
    caller.  This adapter computes them with HF's own rotary module and forwards to the drop-in."""

    def __init__(self, hf_attn, layer_idx: int):
        super().__init__()
        import fast_mimi_b200 as fm
        self.rotary_emb = hf_attn.rotary_emb
        self.inner = fm.MimiAttentionB200(hf_attn.hidden_size, hf_attn.num_heads, hf_attn.head_dim,
                                          hf_attn.sliding_window, layer_idx)
        self.inner.q_proj, self.inner.k_proj = hf_attn.q_proj, hf_attn.k_proj
        self.inner.v_proj, self.inner.o_proj = hf_attn.v_proj, hf_attn.o_proj

    def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_values=None,
                output_attentions=False, use_cache=False, **kwargs):
        assert past_key_values is None and not output_attentions
        if position_ids is None:
            position_ids = torch.arange(hidden_states.shape[1], device=hidden_states.device)[None]
        cos, sin = self.rotary_emb(hidden_states, position_ids)
        out, _ = self.inner(hidden_states, None, None, (cos.float(), sin.float()))
        return out, None


class _HFLayerAdapter(nn.Module):
    """Same idea one level up: HF's transformer calls layer(hidden_states, attention_mask=..., position_ids=...,
    ...) and expects a tuple; the drop-in layer takes the reference's positional arguments."""

    def __init__(self, hf_layer):
        super().__init__()
        import fast_mimi_b200 as fm
        self.rotary_emb = hf_layer.self_attn.rotary_emb
        self.inner = fm.MimiTransformerLayerB200.from_reference(hf_layer)

    def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_values=None,
                output_attentions=False, use_cache=False, **kwargs):
        assert past_key_values is None and not output_attentions
        if position_ids is None:
            position_ids = torch.arange(hidden_states.shape[1], device=hidden_states.device)[None]
        cos, sin = self.rotary_emb(hidden_states, position_ids)
        out, _ = self.inner(hidden_states, None, None, (cos.float(), sin.float()), False)
        return (out,)


def _frame_agreement(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a == b).all(dim=1).float().mean())


@pytest.mark.parametrize("seconds", [5, 10, 12])     # 125, 250, 300 transformer frames: general, whole-clip, long-clip kernel
@pytest.mark.parametrize("swap", ["attention", "layers", "layers+rvq"])
def test_rvq_codes_match_reference_with_b200_attention(swap, seconds):
    from transformers import MimiConfig as HFConfig, MimiModel as HFModel
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    g = load_golden(f"e2e_codes_{seconds}s.npz")
    cfg = HFConfig()
    cfg._attn_implementation = "sdpa"
    torch.manual_seed(0)
    model = HFModel(cfg).eval()
    state = fill_state_by_recipe(model.state_dict(), seed=0)
    for key in ("encoder_transformer.layers.0.self_attn.q_proj.weight",
                "decoder_transformer.layers.7.self_attn.o_proj.weight"):
        assert torch.equal(state[key].flatten()[:4], g["probe." + key]), "weight recipe drifted"
    model.load_state_dict(state, strict=True)
    model = model.cuda()
    audio = synthetic_audio(seconds=seconds)
    assert torch.equal(audio[0, 0, :16], g["audio_probe"])
    audio = audio.cuda()
    with torch.inference_mode():
        stock = model.encode(audio, num_quantizers=8).audio_codes.cpu()
        layers = model.encoder_transformer.layers
        for layer_idx, layer in enumerate(layers):
            if swap == "attention":
                layer.self_attn = _HFAttentionAdapter(layer.self_attn, layer_idx)
            else:        # LayerNorms, projections, attention, MLP, layer scales and residual adds: all native
                layers[layer_idx] = _HFLayerAdapter(layer)
        if swap == "layers+rvq":     # ... and the quantiser behind the transformer as well
            import fast_mimi_b200 as fm
            model.quantizer.encode = fm.MimiSplitRVQB200.from_reference(model.quantizer).encode
        ours = model.encode(audio, num_quantizers=8).audio_codes.cpu()
    golden = g["codes"]
    assert ours.shape == golden.shape == (1, 8, (seconds * 25 + 1) // 2)
    stock_vs_ref = _frame_agreement(stock, golden)
    ours_vs_ref = _frame_agreement(ours, golden)
    ours_vs_stock = _frame_agreement(ours, stock)
    print(f"[{swap}, {seconds} s] code-frame agreement: stock GPU vs reference CPU {stock_vs_ref:.4f}, "
          f"B200 attention vs reference CPU {ours_vs_ref:.4f}, B200 attention vs stock GPU {ours_vs_stock:.4f}")
    assert ours_vs_ref >= 0.995
