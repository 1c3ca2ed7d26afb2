"""The drop-in modules inside the REFERENCE's own model classes.

``oracle/make_ref.py`` places the reference's Python package under the git-ignored ``oracle/_ref`` (it travels with
the working tree to the GPU box like the built library); where it is absent these tests skip.  They exercise what
no adapter can: ``fast_mimi_b200.install`` / ``install_layers`` on a reference ``MimiTransformerModel``, driven by
``MimiTransformerModel.forward`` (src/fast_mimi/model.py:2129-2232) with the 4-D mask, ``(cos, sin)`` and cache
protocol it builds itself, inside ``MimiModel.encode`` (src/fast_mimi/model.py:3070-3137).
"""
from __future__ import annotations

import pytest
import torch

import oracle
from conftest import fill_state_by_recipe, load_golden, synthetic_audio

ref = oracle.import_reference()
if ref is None:
    pytest.skip("the reference package is not under oracle/_ref (run oracle/make_ref.py)", allow_module_level=True)

from fast_mimi import MimiConfig, MimiKVCache, MimiModel  # noqa: E402
from fast_mimi.model import MimiTransformerModel  # noqa: E402


def test_install_keeps_the_reference_state_dict():
    """Swapping the modules in must not change a single state-dict key or their order (the reference's own
    parity test loads checkpoints with strict=True: tests/test_parity.py:15-21 of the reference)."""
    import fast_mimi_b200 as fm
    torch.manual_seed(0)
    for swap in (fm.install, fm.install_layers):
        stack = MimiTransformerModel(MimiConfig(), "sdpa").eval()
        before = [(k, v.data_ptr()) for k, v in stack.state_dict().items()]
        assert len(before) == 96
        swap(stack)
        after = [(k, v.data_ptr()) for k, v in stack.state_dict().items()]
        assert after == before                     # same names, same order, same storage (shared, not copied)
        stack.load_state_dict({k: v.clone() for k, v in stack.state_dict().items()}, strict=True)
        with pytest.raises(RuntimeError, match="CUDA"):
            stack(torch.zeros(1, 4, 512))          # no CPU path: fails loudly instead of falling back


def test_kv_ring_follows_the_reference_cache_protocol():
    """get_seq_length / get_mask_sizes / configure_sliding_window of the ring against MimiKVCache itself."""
    import fast_mimi_b200 as fm
    ring = fm.MimiKVRing(2, 1, 250, device="cpu")
    cache = MimiKVCache(2, sliding_window=250)
    ring.configure_sliding_window(250)
    with pytest.raises(ValueError):
        ring.configure_sliding_window(128)
    for t in (3, 100, 1, 200, 1, 300):
        assert ring.get_seq_length() == cache.get_seq_length()
        assert ring.get_mask_sizes(t) == cache.get_mask_sizes(t)
        k = torch.zeros(1, 8, t, 64)
        for layer in range(2):
            cache.update(k, k, layer)
            ring.advance(layer, t)
    assert ring.get_seq_length(1) == cache.get_seq_length(1) == 605


def _frame_agreement(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a == b).all(dim=1).float().mean())


def _reference_model(device):
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.manual_seed(0)
    model = MimiModel(MimiConfig(), attention_backend="sdpa").eval()
    model.load_state_dict(fill_state_by_recipe(model.state_dict(), seed=0))
    return model.to(device)


@pytest.mark.gpu
@pytest.mark.parametrize("seconds", [5, 10, 12])
@pytest.mark.parametrize("swap", ["attention", "layers", "layers+downsample+rvq"])
def test_codes_through_the_reference_model_match_its_cpu_result(swap, seconds):
    """benchmark config 1 inside the reference's MimiModel: encode() hands the installed modules its own mask and
    rotary tables; code frames vs the reference's CPU codes (tests/golden/e2e_codes_*s.npz) >= 99.5 %."""
    import fast_mimi_b200 as fm
    g = load_golden(f"e2e_codes_{seconds}s.npz")
    model = _reference_model("cuda")
    audio = synthetic_audio(seconds=seconds).cuda()
    with torch.inference_mode():
        stock = model.encode(audio, num_quantizers=8).audio_codes.cpu()
        (fm.install if swap == "attention" else fm.install_layers)(model.encoder_transformer)
        if swap == "layers+downsample+rvq":      # encoder transformer -> downsample -> quantiser: one native chain
            model.downsample = fm.MimiDownsampleB200(model.downsample)
            model.quantizer.encode = fm.MimiSplitRVQB200.from_reference(model.quantizer).encode
        ours = model.encode(audio, num_quantizers=8).audio_codes.cpu()
    fm.check_status()
    golden = g["codes"]
    print(f"[reference MimiModel, {swap}, {seconds} s] code-frame agreement with the reference's CPU codes: "
          f"stock GPU {_frame_agreement(stock, golden):.4f}, B200 modules {_frame_agreement(ours, golden):.4f}")
    assert ours.shape == golden.shape
    assert _frame_agreement(ours, golden) >= 0.995


@pytest.mark.gpu
@pytest.mark.parametrize("swap", ["attention", "layers"])
def test_chunked_streaming_encode_through_the_reference_model(swap):
    """Streaming encode (src/fast_mimi/model.py:3070-3137, use_streaming=True): 12 s of audio in chunks of 5, 1, 20,
    1, 48 and 75 code frames (10 .. 150 transformer frames per call, crossing the 250-frame window).  The stock
    model runs with the reference's MimiKVCache, the swapped one with a MimiKVRing driven through the same
    configure_sliding_window / get_seq_length / get_mask_sizes calls of MimiTransformerModel.forward."""
    import fast_mimi_b200 as fm
    model = _reference_model("cuda")
    audio = synthetic_audio(seconds=12).cuda()
    frames = [5, 1, 20, 1, 48, 75]

    def stream(kv):
        pc, out, a = None, [], 0
        for n in frames:
            chunk = audio[:, :, a * 1920:(a + n) * 1920]
            res = model.encode(chunk, num_quantizers=8, encoder_past_key_values=kv, padding_cache=pc, use_streaming=True)
            kv, pc = res.encoder_past_key_values, res.padding_cache
            out.append(res.audio_codes)
            a += n
        return torch.cat(out, dim=-1).cpu(), kv

    with torch.inference_mode():
        stock, _ = stream(None)
        (fm.install if swap == "attention" else fm.install_layers)(model.encoder_transformer)
        ring = fm.MimiKVRing(len(model.encoder_transformer.layers), 1, 250, device="cuda")
        ours, kv = stream(ring)
    fm.check_status()
    assert kv is ring and ring.get_seq_length() == 300
    offline = load_golden("e2e_codes_12s.npz")["codes"]
    print(f"[streaming, {swap}] code-frame agreement: B200 ring vs stock streaming {_frame_agreement(ours, stock):.4f}, "
          f"stock streaming vs the reference's offline CPU codes {_frame_agreement(stock, offline):.4f}")
    assert ours.shape == stock.shape == (1, 8, 150)
    assert _frame_agreement(ours, stock) >= 0.995


@pytest.mark.gpu
def test_streaming_with_the_reference_own_cache_object():
    """use_streaming=True without handing in a ring: MimiTransformerModel.forward creates a MimiKVCache by itself
    (src/fast_mimi/model.py:2166-2170) and the installed modules must work with it through update()."""
    import fast_mimi_b200 as fm
    model = _reference_model("cuda")
    audio = synthetic_audio(seconds=12).cuda()
    frames = [30, 2, 70, 1, 47]

    def stream():
        kv, pc, out, a = None, None, [], 0
        for n in frames:
            res = model.encode(audio[:, :, a * 1920:(a + n) * 1920], num_quantizers=8, encoder_past_key_values=kv,
                               padding_cache=pc, use_streaming=True)
            kv, pc = res.encoder_past_key_values, res.padding_cache
            out.append(res.audio_codes)
            a += n
        return torch.cat(out, dim=-1).cpu(), kv

    with torch.inference_mode():
        stock, _ = stream()
        fm.install(model.encoder_transformer)
        ours, kv = stream()
    fm.check_status()
    assert isinstance(kv, MimiKVCache) and kv.get_seq_length() == 300
    print(f"[streaming with the reference's MimiKVCache] code-frame agreement with stock: {_frame_agreement(ours, stock):.4f}")
    assert _frame_agreement(ours, stock) >= 0.995


@pytest.mark.gpu
def test_decode_through_the_reference_model_with_the_native_chain():
    """The decoder side inside the reference's MimiModel.decode (src/fast_mimi/model.py:3139-3220): quantiser decode,
    upsample and the eight decoder-transformer layers on this library's kernels, the SEANet decoder the reference's.
    Waveform against the stock model on the same GPU (FP32, TF32 off) for the reference's CPU codes of 5 s of audio."""
    import fast_mimi_b200 as fm
    from oracle import mimi_attention_oracle as O
    model = _reference_model("cuda")
    codes = load_golden("e2e_codes_5s.npz")["codes"].cuda()
    with torch.inference_mode():
        stock = model.decode(codes).audio_values.cpu()
        fm.install_layers(model.decoder_transformer)
        model.upsample = fm.MimiUpsampleB200(model.upsample)
        model.quantizer.decode = fm.MimiSplitRVQB200.from_reference(model.quantizer).decode
        ours = model.decode(codes).audio_values.cpu()
    fm.check_status()
    err = O.rel_l2(ours, stock)
    print(f"[reference MimiModel.decode, native quantiser decode + upsample + decoder transformer] waveform rel-L2 vs stock: {err:.2e}")
    assert ours.shape == stock.shape
    assert err < 2e-3
