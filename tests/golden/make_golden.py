"""Generate the golden fixtures in this directory from the reference implementation.

Run in a container that has the reference checkout (it cannot travel to the GPU box):

    PYTHONPATH=/path/to/reference/src python tests/golden/make_golden.py

Every fixture is an ``.npz`` of inputs (or the seed that regenerates them) and the
outputs of the reference's own code: ``MimiAttention`` / ``MimiKVCache`` /
``MimiTransformerModel`` (src/fast_mimi/model.py) and ``PureTorchMimi``
(src/fast_mimi/_functional_runtime.py), all FP32 on CPU.  The reference stores no golden
vectors of its own (its tests recompute against HF Transformers), so these files are the
pin for both the CPU oracle and the CUDA kernels.
"""
from __future__ import annotations

import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

from fast_mimi import MimiConfig, MimiKVCache, MimiModel  # noqa: E402
from fast_mimi._functional_runtime import PureTorchMimi  # noqa: E402
from fast_mimi.model import (MimiAttention, MimiRotaryEmbedding, MimiTransformerModel,  # noqa: E402
                             _apply_rope, _attention_mask)

torch.set_num_threads(8)


def tiny_config() -> MimiConfig:
    # Same geometry as the reference's own test fixture (tests/conftest.py:8-28).
    return MimiConfig(sampling_rate=64, hidden_size=16, num_filters=2, upsampling_ratios=(2, 2),
                      codebook_size=16, codebook_dim=8, num_quantizers=4,
                      vector_quantization_hidden_dimension=8, num_semantic_quantizers=1,
                      upsample_groups=16, num_hidden_layers=2, intermediate_size=32,
                      num_attention_heads=2, num_key_value_heads=2, head_dim=8,
                      max_position_embeddings=128, sliding_window=8, frame_rate_override=8)


def save(name, **arrays):
    out = {k: (v.detach().cpu().numpy() if isinstance(v, torch.Tensor) else np.asarray(v))
           for k, v in arrays.items()}
    np.savez_compressed(os.path.join(HERE, name), **out)
    size = os.path.getsize(os.path.join(HERE, name))
    print(f"{name}: {size/1024:.1f} KiB")


def isolated_op():
    """benchmark config 2: B=1,H=8,D=64,T=250 FP32 q,k,v ~ N(0,1)/8, RoPE, band mask, SDPA."""
    cfg = MimiConfig()
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(1, 8, 250, 64, generator=g) / 8 for _ in range(3))
    rope = MimiRotaryEmbedding(cfg)
    cos, sin = rope(q, torch.arange(250)[None])
    qr, kr = _apply_rope(q, k, cos, sin)
    mask = _attention_mask(batch_size=1, query_length=250, key_length=250, query_offset=0,
                           key_offset=0, sliding_window=250, padding_mask=None, backend="sdpa",
                           dtype=q.dtype, device=q.device)
    out = torch.nn.functional.scaled_dot_product_attention(qr, kr, v, attn_mask=mask, scale=0.125)
    rows = np.array(sorted(set(list(range(0, 250, 9)) + [1, 2, 63, 64, 65, 127, 128, 129, 248, 249])))
    save("isolated_T250.npz", seed=0, rows=rows, cos=cos[0, rows], sin=sin[0, rows],
         q_rot=qr[0, :, rows], out=out[0, :, rows], q_head0=q[0, 0, :4], v_head7=v[0, 7, -4:])


def long_band():
    """Config 4 geometry at reduced batch: B=1, T=700 > 2 windows, so most rows see a full
    250-key band that starts after position 0."""
    cfg = MimiConfig()
    g = torch.Generator().manual_seed(4)
    q, k, v = (torch.randn(1, 8, 700, 64, generator=g) / 8 for _ in range(3))
    cos, sin = MimiRotaryEmbedding(cfg)(q, torch.arange(700)[None])
    qr, kr = _apply_rope(q, k, cos, sin)
    mask = _attention_mask(batch_size=1, query_length=700, key_length=700, query_offset=0,
                           key_offset=0, sliding_window=250, padding_mask=None, backend="sdpa",
                           dtype=q.dtype, device=q.device)
    out = torch.nn.functional.scaled_dot_product_attention(qr, kr, v, attn_mask=mask, scale=0.125)
    rows = np.array(sorted(set(list(range(0, 700, 37)) + [249, 250, 251, 383, 384, 499, 500, 699])))
    save("band_T700.npz", seed=4, rows=rows, out=out[0, :, rows])


def _round_bf16_(attn):
    """Make the projection inputs BF16-representable (q/k/v weights; o_proj stays FP32) so that the
    BF16 tensor-core path and the FP32 reference consume identical values."""
    with torch.no_grad():
        for lin in (attn.q_proj, attn.k_proj, attn.v_proj):
            lin.weight.copy_(lin.weight.bfloat16().float())


def attention_layer(name, cfg, b, t, seed, rows=None, bf16_inputs=False):
    """One reference MimiAttention layer, no cache: x -> (out after o_proj)."""
    torch.manual_seed(seed)
    attn = MimiAttention(cfg, 0, "sdpa").eval()
    for p in attn.parameters():
        torch.nn.init.normal_(p, std=0.02 if cfg.hidden_size == 512 else 0.2)
    x = torch.randn(b, t, cfg.hidden_size)
    if bf16_inputs:
        _round_bf16_(attn)
        x = x.bfloat16().float()
    cos, sin = MimiRotaryEmbedding(cfg)(x, torch.arange(t)[None])
    mask = _attention_mask(batch_size=b, query_length=t, key_length=t, query_offset=0, key_offset=0,
                           sliding_window=cfg.sliding_window, padding_mask=None, backend="sdpa",
                           dtype=x.dtype, device=x.device)
    with torch.inference_mode():
        out, _ = attn(x, mask, None, (cos, sin))
    arrays = dict(seed=seed, b=b, t=t)
    if rows is None:
        arrays.update(x=x, wq=attn.q_proj.weight, wk=attn.k_proj.weight, wv=attn.v_proj.weight,
                      wo=attn.o_proj.weight, out=out)
    else:
        rows = np.array(rows)
        arrays.update(rows=rows, out=out[:, rows], x_probe=x[0, :2, :8],
                      wq_probe=attn.q_proj.weight[:2, :8], wo_probe=attn.o_proj.weight[:2, :8])
    save(name, **arrays)


def cached_streams(name, cfg, b, chunks, seed, keep_steps=None, std=0.2, bf16_inputs=False):
    """Reference MimiTransformerModel-style cached calls of ONE attention layer: the caller
    bookkeeping of model.py:2176-2206 (positions, mask sizes) followed by MimiAttention with a
    MimiKVCache.  ``chunks`` is the list of per-call frame counts."""
    torch.manual_seed(seed)
    attn = MimiAttention(cfg, 0, "sdpa").eval()
    for p in attn.parameters():
        torch.nn.init.normal_(p, std=std)
    if bf16_inputs:
        _round_bf16_(attn)
    rope = MimiRotaryEmbedding(cfg)
    cache = MimiKVCache(1, sliding_window=cfg.sliding_window)
    xs, outs, seqs = [], [], []
    for step, t in enumerate(chunks):
        x = torch.randn(b, t, cfg.hidden_size)
        if bf16_inputs:
            x = x.bfloat16().float()
        past = cache.get_seq_length()
        pos = torch.arange(past, past + t)[None]
        k_len, k_off = cache.get_mask_sizes(t)
        mask = _attention_mask(batch_size=b, query_length=t, key_length=k_len, query_offset=past,
                               key_offset=k_off, sliding_window=cfg.sliding_window, padding_mask=None,
                               backend="sdpa", dtype=x.dtype, device=x.device)
        with torch.inference_mode():
            out, _ = attn(x, mask, cache, rope(x, pos))
        seqs.append(cache.get_seq_length())
        assert cache.key_cache[0].shape[-2] <= cfg.sliding_window - 1
        if keep_steps is None or step in keep_steps:
            xs.append(x.numpy()); outs.append(out.numpy())
    arrays = dict(seed=seed, b=b, chunks=np.array(chunks), seq_lengths=np.array(seqs),
                  final_key_cache=cache.key_cache[0], final_value_cache=cache.value_cache[0])
    if keep_steps is None:
        arrays.update(wq=attn.q_proj.weight, wk=attn.k_proj.weight, wv=attn.v_proj.weight,
                      wo=attn.o_proj.weight)
        for i, (x, o) in enumerate(zip(xs, outs)):
            arrays[f"x{i}"] = x; arrays[f"out{i}"] = o
    else:
        arrays.update(keep_steps=np.array(sorted(keep_steps)), outs=np.stack(outs),
                      final_key_cache=cache.key_cache[0][:, :, -3:], final_value_cache=cache.value_cache[0][:, :, -3:])
    save(name, **arrays)


def cached_chunks_mimi(name="cached_chunks_mimi.npz", chunks=(12, 50, 1, 200, 1, 37, 260, 3), b=2, seed=21):
    """The reference's chunked streaming scenario (tests/test_parity.py:56-81 of the reference) at Mimi's own
    geometry: one MimiAttention layer + MimiKVCache driven with the caller bookkeeping of model.py:2176-2206,
    BF16-representable weights and inputs.  The chunk lengths cross the window (12+50+1+200 = 263 > 250), include
    one-frame steps between chunks and a chunk longer than the window.  Inputs are regenerated from the seed;
    every fifth output row of each chunk (plus its first and last) is stored."""
    cfg = MimiConfig()
    torch.manual_seed(seed)
    attn = MimiAttention(cfg, 0, "sdpa").eval()
    for p in attn.parameters():
        torch.nn.init.normal_(p, std=0.02)
    _round_bf16_(attn)
    rope = MimiRotaryEmbedding(cfg)
    cache = MimiKVCache(1, sliding_window=cfg.sliding_window)
    arrays = dict(seed=seed, b=b, chunks=np.array(chunks))
    for step, t in enumerate(chunks):
        x = torch.randn(b, t, cfg.hidden_size).bfloat16().float()
        past = cache.get_seq_length()
        k_len, k_off = cache.get_mask_sizes(t)
        mask = _attention_mask(batch_size=b, query_length=t, key_length=k_len, query_offset=past, key_offset=k_off,
                               sliding_window=cfg.sliding_window, padding_mask=None, backend="sdpa", dtype=x.dtype,
                               device=x.device)
        with torch.inference_mode():
            out, _ = attn(x, mask, cache, rope(x, torch.arange(past, past + t)[None]))
        rows = np.array(sorted(set(list(range(0, t, 5)) + [t - 1])))
        arrays[f"rows{step}"] = rows
        arrays[f"out{step}"] = out[:, rows]
    arrays.update(final_key_cache=cache.key_cache[0][:, :, -3:], final_value_cache=cache.value_cache[0][:, :, -3:],
                  seq_length=cache.get_seq_length())
    save(name, **arrays)


def transformer_stack_tiny():
    """Two-layer tiny MimiTransformerModel, prefill then cached steps (shared cache, layer
    positions taken from layer 0 as the reference does)."""
    cfg = tiny_config()
    g = torch.Generator().manual_seed(1234)
    model = MimiTransformerModel(cfg, "sdpa").eval()
    state = model.state_dict()
    for name, value in state.items():       # same recipe as tests/conftest.py:44-53
        if name.endswith("layernorm.weight"):
            value.copy_(torch.rand(value.shape, generator=g) * 0.2 + 0.9)
        else:
            value.copy_(torch.randn(value.shape, generator=g) * 0.05)
    model.load_state_dict(state)
    x = torch.randn(2, 21, cfg.hidden_size, generator=g)
    with torch.inference_mode():
        full = model(x).last_hidden_state
        cache = MimiKVCache(2, sliding_window=cfg.sliding_window)
        outs = [model(x[:, a:b], past_key_values=cache).last_hidden_state
                for a, b in ((0, 5), (5, 6), (6, 13), (13, 14), (14, 21))]
    save("tiny_stack.npz", x=x, full=full, chunked=torch.cat(outs, 1),
         **{"p." + k: v for k, v in state.items()})


def end_to_end_codes(seconds: int = 5):
    """benchmark config 1: full Mimi forward on CPU (5 s synthetic audio, 8 codebooks; also 10 s and 12 s, whose
    250 and 300 transformer frames reach the whole-clip and the long-clip attention kernels) with the weight recipe
    of tests/conftest.py::fill_state_by_recipe, through the reference MimiModel and its functional runtime;
    HF Transformers' MimiModel (the implementation the reference's own tests compare against) is loaded with
    the same state and must give the same codes, which is what lets it stand in on the GPU box."""
    sys.path.insert(0, os.path.dirname(HERE))
    from conftest import fill_state_by_recipe, synthetic_audio
    torch.manual_seed(0)
    model = MimiModel(MimiConfig(), attention_backend="sdpa").eval()
    state = fill_state_by_recipe(model.state_dict(), seed=0)
    model.load_state_dict(state)
    audio = synthetic_audio(seconds=seconds)
    with torch.inference_mode():
        codes = model.encode(audio, num_quantizers=8).audio_codes
        functional = PureTorchMimi(model)
        enc_tr_in = functional.encoder(audio).transpose(1, 2)
        enc_tr_out = functional.transformer(enc_tr_in, "encoder_transformer")
        f_codes = functional.quantizer_encode(functional.downsample(enc_tr_out.transpose(1, 2)), 8)
    assert torch.equal(f_codes.reshape(codes.shape), codes), "functional runtime disagrees with the module path"
    from transformers import MimiConfig as HFConfig, MimiModel as HFModel
    hf_cfg = HFConfig(**MimiConfig().to_dict())
    hf_cfg._attn_implementation = "sdpa"
    hf = HFModel(hf_cfg).eval()
    assert list(hf.state_dict()) == list(state)
    hf.load_state_dict(state, strict=True)
    with torch.inference_mode():
        hf_codes = hf.encode(audio, num_quantizers=8).audio_codes
    assert torch.equal(hf_codes, codes), "HF Transformers disagrees with the reference"
    probe = {k: state[k].flatten()[:4] for k in
             ("encoder_transformer.layers.0.self_attn.q_proj.weight",
              "decoder_transformer.layers.7.self_attn.o_proj.weight",
              "quantizer.semantic_residual_vector_quantizer.layers.0.codebook.embed_sum")}
    save(f"e2e_codes_{seconds}s.npz", codes=codes, audio_probe=audio[0, 0, :16], enc_tr_in_probe=enc_tr_in[0, ::25, :8],
         enc_tr_out_probe=enc_tr_out[0, ::25, :8], distinct_codes=len(torch.unique(codes)),
         **{"probe." + k: v for k, v in probe.items()})
    print("codes", tuple(codes.shape), "distinct", len(torch.unique(codes)))


def downsample():
    """The reference's stride-2 ``downsample`` convolution (MimiModel.downsample, model.py:2734-2744) on seeded
    transformer-output-like frames of odd and even lengths; outputs at a few frames."""
    from fast_mimi.model import MimiConv1d
    cfg = MimiConfig()
    torch.manual_seed(51)
    conv = MimiConv1d(cfg, cfg.hidden_size, cfg.hidden_size, 4, stride=2, bias=False, pad_mode="replicate").eval()
    with torch.no_grad():
        conv.conv.weight.copy_(torch.randn(conv.conv.weight.shape) / (4 * cfg.hidden_size) ** 0.5)
    arrays = dict(seed=51, weight_probe=conv.conv.weight[:2, :3])
    for t in (125, 250, 7):
        x = torch.randn(2, t, cfg.hidden_size)
        with torch.inference_mode():
            y = conv(x.transpose(1, 2)).transpose(1, 2)               # [2, ceil(t/2), 512]
        rows = np.array(sorted(set([0, 1, 2, y.shape[1] // 2, y.shape[1] - 2, y.shape[1] - 1])))
        arrays[f"rows{t}"] = rows
        arrays[f"out{t}"] = y[:, rows]
        arrays[f"frames{t}"] = y.shape[1]
    save("downsample.npz", **arrays)


def upsample():
    """The reference's stride-2 ``upsample`` transposed convolution (MimiModel.upsample, model.py:2745-2753) on seeded
    frames; outputs at a few frames."""
    from fast_mimi.model import MimiConvTranspose1d
    cfg = MimiConfig()
    torch.manual_seed(52)
    convtr = MimiConvTranspose1d(cfg, cfg.hidden_size, cfg.hidden_size, 4, stride=2, bias=False,
                                 groups=cfg.upsample_groups).eval()
    with torch.no_grad():
        convtr.conv.weight.copy_(torch.randn(convtr.conv.weight.shape) / 2)
    arrays = dict(seed=52, weight_probe=convtr.conv.weight[:3, 0])
    for t in (63, 125, 1):
        x = torch.randn(2, t, cfg.hidden_size)
        with torch.inference_mode():
            y = convtr(x.transpose(1, 2)).transpose(1, 2)             # [2, 2t, 512]
        rows = np.array(sorted(set([0, 1, 2, 3, y.shape[1] // 2, y.shape[1] - 2, y.shape[1] - 1]) & set(range(y.shape[1]))))
        arrays[f"rows{t}"] = rows
        arrays[f"out{t}"] = y[:, rows]
        arrays[f"frames{t}"] = y.shape[1]
    save("upsample.npz", **arrays)


def rvq_codes():
    """Residual quantiser stack of the reference (7 layers, 2048 x 256 codebooks, 1x1 input projection) on seeded
    embeddings [2, 512, 40]: codes, and the decoded sum before the output projection at a few frames."""
    sys.path.insert(0, os.path.dirname(HERE))
    from conftest import rvq_recipe
    from fast_mimi.model import MimiResidualVectorQuantizer
    cfg = MimiConfig()
    layers = 7
    g, embed_sum, usage, proj = rvq_recipe(31, layers)
    emb = torch.randn(2, cfg.hidden_size, 40, generator=g) * 3
    rvq = MimiResidualVectorQuantizer(cfg, layers).eval()
    with torch.no_grad():
        rvq.input_proj.weight.copy_(proj[:, :, None])
        for i, layer in enumerate(rvq.layers):
            layer.codebook.embed_sum.copy_(embed_sum[i])
            layer.codebook.cluster_usage.copy_(usage[i])
            layer.codebook._embed = None
    with torch.inference_mode():
        codes = rvq.encode(emb)                                   # [layers, 2, 40]
        quantized = codes.new_zeros((), dtype=torch.float32)
        for index, indices in enumerate(codes):
            quantized = quantized + rvq.layers[index].decode(indices)   # [2, 256, 40]
    save("rvq_codes.npz", codes=codes, quantized_probe=quantized[:, :, ::13], emb_probe=emb[0, :4, :4],
         distinct=len(torch.unique(codes)))
    print("rvq codes", tuple(codes.shape), "distinct", len(torch.unique(codes)))


if __name__ == "__main__":
    isolated_op()
    long_band()
    attention_layer("tiny_attention_layer.npz", tiny_config(), 2, 21, seed=11)
    attention_layer("attention_layer_T250.npz", MimiConfig(), 2, 250, seed=1,
                    rows=sorted(set(list(range(0, 250, 17)) + [127, 128, 249])), bf16_inputs=True)
    attention_layer("attention_layer_T250_fp32.npz", MimiConfig(), 2, 250, seed=3,
                    rows=sorted(set(list(range(0, 250, 17)) + [127, 128, 249])), bf16_inputs=False)
    attention_layer("attention_layer_T313.npz", MimiConfig(), 1, 313, seed=2,
                    rows=sorted(set(list(range(0, 313, 23)) + [249, 250, 251, 312])), bf16_inputs=True)
    cached_streams("tiny_cached_chunks.npz", tiny_config(), 2, [4, 4, 4, 4, 4, 1, 1, 3, 9, 1], seed=12)
    cached_streams("tiny_cached_decode.npz", tiny_config(), 1, [1] * 12, seed=13)
    cached_streams("ring_decode_260.npz", MimiConfig(), 2, [1] * 260, seed=5, std=0.02,
                   keep_steps={0, 1, 2, 127, 248, 249, 250, 251, 259}, bf16_inputs=True)
    cached_chunks_mimi()
    transformer_stack_tiny()
    for seconds in (5, 10, 12):
        end_to_end_codes(seconds)
    rvq_codes()
    downsample()
    upsample()
