"""Tensor-level wrappers over the C ABI: validate geometry, then launch on the current stream.

Validation style follows the reference's native wrappers (dtype / shape / contiguity / device checks
raising ``RuntimeError`` before the launch: src/fast_mimi/_native_cutlass.py:126-149).  PyTorch is
used only for device memory and streams.
"""
from __future__ import annotations

import torch

from . import _native

HIDDEN, HEADS, HEAD_DIM = 512, 8, 64
_VALUE_CODES = {torch.bfloat16: 0, torch.float16: 1}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(f"unexpected attention geometry: {msg}")


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _check_frames(t: torch.Tensor, name: str, dtype: torch.dtype, rows: int | None = None) -> None:
    _need(t.is_cuda, f"{name} must be a CUDA tensor")
    _need(t.dtype == dtype, f"{name} must be {dtype}, got {t.dtype}")
    _need(t.is_contiguous(), f"{name} must be contiguous")
    _need(t.shape[-1] == HIDDEN, f"{name} last dimension must be {HIDDEN}")
    if rows is not None:
        _need(t.numel() == rows * HIDDEN, f"{name} must hold {rows} frames")


_INPUT_DTYPES = (torch.bfloat16, torch.float16)


def _check_projection_inputs(x: torch.Tensor, w_qkv: torch.Tensor) -> int:
    """x and the packed weight must share one 16-bit float type; returns the dtype-flag bit for FP16."""
    _need(x.dtype in _INPUT_DTYPES, f"x must be bfloat16 or float16, got {x.dtype}")
    _check_frames(x, "x", x.dtype)
    _need(w_qkv.is_cuda and w_qkv.dtype == x.dtype and w_qkv.is_contiguous()
          and tuple(w_qkv.shape) == (3 * HIDDEN, HIDDEN), f"w_qkv must be contiguous {x.dtype} [1536, 512]")
    return 2 if x.dtype == torch.float16 else 0


def _check_tables(cos: torch.Tensor, sin: torch.Tensor, B: int, T: int) -> int:
    for name, t in (("cos", cos), ("sin", sin)):
        _need(t.is_cuda and t.dtype == torch.float32 and t.is_contiguous(), f"{name} must be contiguous CUDA float32")
        _need(t.dim() == 3 and t.shape[1] == T and t.shape[2] == HEAD_DIM and t.shape[0] in (1, B),
              f"{name} must be [1 or {B}, {T}, {HEAD_DIM}], got {tuple(t.shape)}")
    _need(cos.shape == sin.shape, "cos and sin must have the same shape")
    return 0 if cos.shape[0] == 1 else T * HEAD_DIM


_default_status: dict = {}


def default_status(device) -> torch.Tensor:
    """The per-device status word used when a call does not pass its own.  Once a kernel has recorded
    a bounded-wait timeout in it, later kernels given the same word return at once; check it with
    ``read_status(default_status(dev))`` and clear it with ``.zero_()``."""
    dev = torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    st = _default_status.get(dev)
    if st is None:
        st = _default_status[dev] = torch.zeros(1, dtype=torch.int32, device=dev)
    return st


def _status_ptr(status, like: torch.Tensor) -> int:
    return (default_status(like.device) if status is None else status).data_ptr()


def new_status(device) -> torch.Tensor:
    """A zeroed device status word for the bounded-wait error codes."""
    return torch.zeros(1, dtype=torch.int32, device=device)


def read_status(status: torch.Tensor) -> int:
    """Synchronise the current stream and return the status word (0 = every wait completed)."""
    return _native.load().fm_read_status(status.data_ptr(), _stream())


STATUS_NAMES = {101: "a TMA completion barrier never flipped", 102: "a tensor-core completion barrier never flipped",
                103: "a consumer never released a buffer", 104: "a device-side bounds check failed "
                "(for instance a negative stream position)",
                105: "an input that must be finite was not (no quantiser entry could be chosen)"}


def check_status(device=None, status: torch.Tensor | None = None) -> None:
    """Synchronise the current stream and raise ``RuntimeError`` if a kernel recorded an error in the status
    word (``status``, or the device's default word).  The word is sticky: once it is non-zero every later
    kernel handed the same word returns without doing its work, so results produced since the last check
    must be discarded; clear it with ``.zero_()`` after handling the error.  The kernels never synchronise,
    so callers of the attention / layer modules call this at their own synchronisation points."""
    st = default_status(device if device is not None else torch.cuda.current_device()) if status is None else status
    code = read_status(st)
    if code != 0:
        raise RuntimeError(f"fast_mimi_b200: device status {code} ({STATUS_NAMES.get(code, 'unknown code')}); "
                           "outputs written since the last check are not valid; clear the word with .zero_()")


def qkv_rope(x, w_qkv, cos, sin, *, value_dtype=torch.float16, out=None, status=None):
    """``x [B,T,512] bf16`` -> rotated ``q, k`` (bf16) and ``v`` (value_dtype), each ``[B,T,512]``."""
    lib = _native.load()
    _need(x.dim() == 3, "x must be [B, T, 512]")
    B, T, _ = x.shape
    in_flag = _check_projection_inputs(x, w_qkv)
    bstride = _check_tables(cos, sin, B, T)
    if out is None:
        out = (torch.empty(x.shape, dtype=torch.bfloat16, device=x.device),
               torch.empty(x.shape, dtype=torch.bfloat16, device=x.device),
               torch.empty(x.shape, dtype=value_dtype, device=x.device))
    q, k, v = out
    _check_frames(q, "q", torch.bfloat16, B * T)
    _check_frames(k, "k", torch.bfloat16, B * T)
    _check_frames(v, "v", value_dtype, B * T)
    rc = lib.fm_qkv_rope_bf16(x.data_ptr(), w_qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), bstride,
                              q.data_ptr(), k.data_ptr(), v.data_ptr(), B, T, _VALUE_CODES[value_dtype] | in_flag,
                              _status_ptr(status, x), _stream())
    _native.check(rc, "fm_qkv_rope_bf16")
    return q, k, v


def out_proj(attn, w_o, *, layer_scale=None, residual=None, out_dtype=None, out=None, status=None):
    """``residual + layer_scale * (attn @ w_o.T)`` for ``attn [..., 512]`` and ``w_o [512, 512]`` of one 16-bit
    float type; ``residual`` and the result have ``out_dtype`` (default: ``attn``'s).  ``layer_scale`` is a
    ``[512]`` float32 vector.  This is ``o_proj`` plus the layer's scale and residual add."""
    lib = _native.load()
    _need(attn.dtype in _INPUT_DTYPES, f"attn must be bfloat16 or float16, got {attn.dtype}")
    _check_frames(attn, "attn", attn.dtype)
    _need(w_o.is_cuda and w_o.dtype == attn.dtype and w_o.is_contiguous() and tuple(w_o.shape) == (HIDDEN, HIDDEN),
          f"w_o must be contiguous {attn.dtype} [512, 512]")
    frames = attn.numel() // HIDDEN
    out_dtype = out_dtype or (out.dtype if out is not None else attn.dtype)
    _need(out_dtype in _VALUE_CODES, "the output must be float16 or bfloat16")
    if out is None:
        out = torch.empty(attn.shape, dtype=out_dtype, device=attn.device)
    _check_frames(out, "out", out_dtype, frames)
    if residual is not None:
        _check_frames(residual, "residual", out_dtype, frames)
    if layer_scale is not None:
        _need(layer_scale.is_cuda and layer_scale.dtype == torch.float32 and layer_scale.is_contiguous()
              and layer_scale.numel() == HIDDEN, "layer_scale must be contiguous CUDA float32 [512]")
    flags = _VALUE_CODES[out_dtype] | (2 if attn.dtype == torch.float16 else 0)
    rc = lib.fm_out_proj_f16(attn.data_ptr(), w_o.data_ptr(),
                             layer_scale.data_ptr() if layer_scale is not None else None,
                             residual.data_ptr() if residual is not None else None, out.data_ptr(), frames, flags,
                             _status_ptr(status, attn), _stream())
    _native.check(rc, "fm_out_proj_f16")
    return out


_OUT_CODES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def linear(a, w, *, scale=None, residual=None, activation=None, out_dtype=None, out=None, status=None):
    """``residual + scale * act(a @ w.T)`` on the tensor core for ``a [..., K]`` and ``w [N, K]`` of one 16-bit
    float type (K a multiple of 64, N of 256).  ``activation``: ``None`` or ``"gelu"`` (exact erf form);
    ``scale``: ``[N]`` float32; ``residual`` and the result: ``out_dtype`` (bfloat16, float16 or float32;
    default ``a``'s type), shaped ``[..., N]``.  Covers the MLP's two linears and the output projection of
    the reference's transformer layer with their GELU / layer scale / residual add folded in."""
    lib = _native.load()
    _need(a.is_cuda and a.dtype in _INPUT_DTYPES and a.is_contiguous(), "a must be a contiguous CUDA bfloat16/float16 tensor")
    _need(w.is_cuda and w.dtype == a.dtype and w.is_contiguous() and w.dim() == 2 and w.shape[1] == a.shape[-1],
          f"w must be contiguous {a.dtype} [N, {a.shape[-1]}]")
    N, K = w.shape
    _need(K % 64 == 0 and N % 256 == 0, "K must be a multiple of 64 and N a multiple of 256")
    _need(activation in (None, "gelu"), "activation must be None or 'gelu'")
    rows = a.numel() // K
    out_dtype = out_dtype or (out.dtype if out is not None else a.dtype)
    _need(out_dtype in _OUT_CODES, "the output must be bfloat16, float16 or float32")
    shape = tuple(a.shape[:-1]) + (N,)
    if out is None:
        out = torch.empty(shape, dtype=out_dtype, device=a.device)
    for name, t in (("out", out), ("residual", residual)):
        if t is not None:
            _need(t.is_cuda and t.dtype == out_dtype and t.is_contiguous() and t.numel() == rows * N,
                  f"{name} must be a contiguous {out_dtype} tensor of {rows} x {N}")
    if scale is not None:
        _need(scale.is_cuda and scale.dtype == torch.float32 and scale.is_contiguous() and scale.numel() == N,
              f"scale must be contiguous CUDA float32 [{N}]")
    rc = lib.fm_linear_f16(a.data_ptr(), w.data_ptr(), scale.data_ptr() if scale is not None else None,
                           residual.data_ptr() if residual is not None else None, out.data_ptr(), rows, N, K,
                           1 if a.dtype == torch.float16 else 0, _OUT_CODES[out_dtype],
                           1 if activation == "gelu" else 0, _status_ptr(status, a), _stream())
    _native.check(rc, "fm_linear_f16")
    return out


def layer_norm(x, weight, bias, *, eps=1e-5, out_dtype=torch.float16, out=None):
    """LayerNorm over the 512 channels of ``x [..., 512]`` (float32, float16 or bfloat16) in FP32 arithmetic,
    result rounded once to ``out_dtype`` (float16 or bfloat16) for the projections that consume it."""
    lib = _native.load()
    _need(x.dtype in _OUT_CODES, "x must be bfloat16, float16 or float32")
    _check_frames(x, "x", x.dtype)
    _need(out_dtype in _VALUE_CODES, "the output must be float16 or bfloat16")
    for name, t in (("weight", weight), ("bias", bias)):
        _need(t.is_cuda and t.dtype == torch.float32 and t.is_contiguous() and t.numel() == HIDDEN,
              f"{name} must be contiguous CUDA float32 [512]")
    rows = x.numel() // HIDDEN
    if out is None:
        out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    _check_frames(out, "out", out_dtype, rows)
    rc = lib.fm_layernorm_f16(x.data_ptr(), _OUT_CODES[x.dtype], weight.data_ptr(), bias.data_ptr(), float(eps),
                              out.data_ptr(), _VALUE_CODES[out_dtype], rows, _stream())
    _native.check(rc, "fm_layernorm_f16")
    return out


def band_attention_prefill(q, k, v, *, window=250, scale=0.125, out=None, status=None):
    """Banded causal attention over rotated ``q, k [B,T,512] bf16`` and ``v [B,T,512]`` (fp16 or bf16)."""
    lib = _native.load()
    _need(q.dim() == 3, "q must be [B, T, 512]")
    B, T, _ = q.shape
    _check_frames(q, "q", torch.bfloat16)
    _check_frames(k, "k", torch.bfloat16, B * T)
    _need(v.dtype in _VALUE_CODES, "v must be float16 or bfloat16")
    _check_frames(v, "v", v.dtype, B * T)
    if out is None:
        out = torch.empty_like(v)
    _check_frames(out, "out", v.dtype, B * T)
    rc = lib.fm_band_attn_prefill_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, T, window,
                                       scale, _VALUE_CODES[v.dtype], _status_ptr(status, q), _stream())
    _native.check(rc, "fm_band_attn_prefill_bf16")
    return out


def attention_prefill(x, w_qkv, cos, sin, *, window=250, scale=0.125, value_dtype=torch.float16,
                      workspace=None, out=None, status=None):
    """Projection + RoPE + banded attention for a call without cache; returns ``[B,T,512]`` value_dtype.  Whole clips
    of 129 .. 256 frames run as one kernel (no q / k / v in memory: ``workspace`` is not used and not allocated);
    other lengths as the projection kernel followed by the attention kernel that fits the clip length."""
    lib = _native.load()
    _need(x.dim() == 3, "x must be [B, T, 512]")
    B, T, _ = x.shape
    in_flag = _check_projection_inputs(x, w_qkv)
    bstride = _check_tables(cos, sin, B, T)
    one_kernel = 128 < T <= 256
    if workspace is None and not one_kernel:
        workspace = (torch.empty(x.shape, dtype=torch.bfloat16, device=x.device),
                     torch.empty(x.shape, dtype=torch.bfloat16, device=x.device),
                     torch.empty(x.shape, dtype=value_dtype, device=x.device))
    ptrs = (None, None, None)
    if workspace is not None:
        q, k, v = workspace
        _check_frames(q, "q workspace", torch.bfloat16, B * T)
        _check_frames(k, "k workspace", torch.bfloat16, B * T)
        _check_frames(v, "v workspace", value_dtype, B * T)
        ptrs = (q.data_ptr(), k.data_ptr(), v.data_ptr())
    if out is None:
        out = torch.empty(x.shape, dtype=value_dtype, device=x.device)
    _check_frames(out, "out", value_dtype, B * T)
    if B == 0 or T == 0:
        return out
    rc = lib.fm_attention_prefill_bf16(x.data_ptr(), w_qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), bstride,
                                       *ptrs, out.data_ptr(), B, T, window,
                                       scale, _VALUE_CODES[value_dtype] | in_flag, _status_ptr(status, x), _stream())
    _native.check(rc, "fm_attention_prefill_bf16")
    return out


def band_attention_chunk(q, k, v, *, window=250, scale=0.125, out=None, status=None):
    """Banded attention of ``q [B,Tq,512]`` (bf16, rotated) against ``k, v [B,Tk,512]`` with ``Tk >= Tq``: the last
    ``Tq`` key rows are the queries' own frames, the rows before them older (cached) ones.  Returns ``[B,Tq,512]``."""
    lib = _native.load()
    _need(q.dim() == 3 and k.dim() == 3, "q and k must be [B, T, 512]")
    B, Tq, _ = q.shape
    Tk = k.shape[1]
    _need(Tk >= Tq and k.shape[0] == B, "k must hold at least the queries' own frames")
    _check_frames(q, "q", torch.bfloat16)
    _check_frames(k, "k", torch.bfloat16, B * Tk)
    _need(v.dtype in _VALUE_CODES, "v must be float16 or bfloat16")
    _check_frames(v, "v", v.dtype, B * Tk)
    if out is None:
        out = torch.empty(q.shape, dtype=v.dtype, device=q.device)
    _check_frames(out, "out", v.dtype, B * Tq)
    rc = lib.fm_band_attn_chunk_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, Tq, Tk, window, scale,
                                     _VALUE_CODES[v.dtype], _status_ptr(status, q), _stream())
    _native.check(rc, "fm_band_attn_chunk_bf16")
    return out


def attention_fused(x, w_qkv, cos, sin, *, window=250, scale=0.125, value_dtype=torch.float16, out=None, status=None):
    """Projection + RoPE + banded attention in one kernel for clips of 128 < T <= 256 frames: ``x [B,T,512]`` ->
    ``[B,T,512]`` value_dtype, no q / k / v workspace (they stay in shared and tensor memory)."""
    lib = _native.load()
    _need(x.dim() == 3, "x must be [B, T, 512]")
    B, T, _ = x.shape
    _need(128 < T <= 256, "the fused kernel takes clips of 129 .. 256 frames")
    in_flag = _check_projection_inputs(x, w_qkv)
    bstride = _check_tables(cos, sin, B, T)
    _need(value_dtype in _VALUE_CODES, "value_dtype must be float16 or bfloat16")
    if out is None:
        out = torch.empty(x.shape, dtype=value_dtype, device=x.device)
    _check_frames(out, "out", value_dtype, B * T)
    rc = lib.fm_attention_fused_bf16(x.data_ptr(), w_qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), bstride,
                                     out.data_ptr(), B, T, window, scale, _VALUE_CODES[value_dtype] | in_flag,
                                     _status_ptr(status, x), _stream())
    _native.check(rc, "fm_attention_fused_bf16")
    return out


def attention_chunk(x, w_qkv, cos, sin, ring_k, ring_v, past, *, window=250, scale=0.125, workspace=None, out=None,
                    status=None):
    """A cached call with ``T`` new frames per stream: ``x [S,T,512]`` at absolute positions ``past .. past+T-1``
    (``cos, sin [1 or S, T, 64]`` are their tables) attends to the ``min(past, window-1)`` newest frames already in
    the ring plus itself, then the new rotated K / V rows enter the ring ``[S,8,slots,64]``.  Returns
    ``[S,T,512]`` in the ring's value type.  ``workspace``: optional ``(q, k, v, k_lin, v_lin)`` buffers of
    ``[S,T,512]`` (bf16, bf16, value type) and ``[S, min(past, window-1) + T, 512]`` (bf16, value type)."""
    lib = _native.load()
    _need(x.dim() == 3, "x must be [S, T, 512]")
    S, T, _ = x.shape
    past = int(past)
    _need(past >= 0, "past must not be negative")
    in_flag = _check_projection_inputs(x, w_qkv)
    bstride = _check_tables(cos, sin, S, T)
    _need(ring_k.dim() == 4 and ring_k.shape[0] == S and ring_k.shape[1] == HEADS and ring_k.shape[3] == HEAD_DIM
          and ring_k.is_cuda and ring_k.dtype == torch.bfloat16 and ring_k.is_contiguous(),
          "ring_k must be contiguous bf16 [S, 8, slots, 64]")
    _need(ring_v.is_cuda and ring_v.dtype in _VALUE_CODES and ring_v.is_contiguous() and ring_v.shape == ring_k.shape,
          "ring_v must match ring_k (float16 or bfloat16)")
    slots = ring_k.shape[2]
    _need(slots >= window, "the ring must have at least `window` slots")
    vdt = ring_v.dtype
    delta = min(past, window - 1)
    if workspace is None:
        mk = lambda rows, dt: torch.empty((S, rows, HIDDEN), dtype=dt, device=x.device)
        workspace = (mk(T, torch.bfloat16), mk(T, torch.bfloat16), mk(T, vdt),
                     mk(delta + T, torch.bfloat16) if delta else None, mk(delta + T, vdt) if delta else None)
    q, k, v, k_lin, v_lin = workspace
    _check_frames(q, "q workspace", torch.bfloat16, S * T)
    _check_frames(k, "k workspace", torch.bfloat16, S * T)
    _check_frames(v, "v workspace", vdt, S * T)
    if delta:
        _check_frames(k_lin, "k_lin workspace", torch.bfloat16, S * (delta + T))
        _check_frames(v_lin, "v_lin workspace", vdt, S * (delta + T))
    if out is None:
        out = torch.empty(x.shape, dtype=vdt, device=x.device)
    _check_frames(out, "out", vdt, S * T)
    rc = lib.fm_attention_chunk_bf16(x.data_ptr(), w_qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), bstride,
                                     q.data_ptr(), k.data_ptr(), v.data_ptr(), _ptr(k_lin) if delta else None,
                                     _ptr(v_lin) if delta else None, ring_k.data_ptr(), ring_v.data_ptr(), out.data_ptr(),
                                     S, T, past, slots, window, scale, _VALUE_CODES[vdt] | in_flag,
                                     _status_ptr(status, x), _stream())
    _native.check(rc, "fm_attention_chunk_bf16")
    return out


STATIC_MAX_FRAMES = 8192


def attention_prefill_static(x, w_qkv, cos, sin, out, *, window=250, scale=0.125, status=None):
    """``attention_prefill`` for hosts that must not allocate device memory while it runs (an
    allocation-free real-time audio callback, a plugin whose host application owns all device memory, a
    process with a fixed device-memory budget):
    the q/k/v workspace is a fixed 24 MiB array inside the library, so at most ``STATIC_MAX_FRAMES`` frames
    (B*T <= 8192) per call, and ``out`` must be supplied by the caller.  Calls share that workspace: do not
    let two of them overlap on the GPU.  Make the first call on a device outside any stream capture."""
    lib = _native.load()
    _need(x.dim() == 3, "x must be [B, T, 512]")
    B, T, _ = x.shape
    in_flag = _check_projection_inputs(x, w_qkv)
    bstride = _check_tables(cos, sin, B, T)
    _need(out is not None and out.dtype in _VALUE_CODES, "out must be a float16 or bfloat16 tensor supplied by the caller")
    _check_frames(out, "out", out.dtype, B * T)
    if B * T > STATIC_MAX_FRAMES:
        raise RuntimeError(f"{B * T} frames exceed the built-in workspace of {STATIC_MAX_FRAMES} frames; "
                           "use attention_prefill with caller-provided workspaces")
    rc = lib.fm_attention_prefill_static_bf16(x.data_ptr(), w_qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), bstride,
                                              out.data_ptr(), B, T, window, scale, _VALUE_CODES[out.dtype] | in_flag,
                                              _status_ptr(status, x), _stream())
    _native.check(rc, "fm_attention_prefill_static_bf16")
    return out


def decode_step(x, w_qkv, cos, sin, ring_k, ring_v, position, *, scale=0.125, q_workspace=None, out=None,
                stream_pos=None, status=None):
    """One streaming step.  ``x [S,512] bf16``; ``ring_k/ring_v [S,8,slots,64]``; the new frame of
    stream s has absolute position ``position + stream_pos[s]``.  Returns ``[S,512] float32``."""
    lib = _native.load()
    _need(x.dim() == 2, "x must be [S, 512]")
    _need(int(position) >= 0, "position must not be negative")
    S = x.shape[0]
    in_flag = _check_projection_inputs(x, w_qkv)
    bstride = 0 if cos.shape[0] == 1 else HEAD_DIM
    _check_tables(cos, sin, S, 1)
    _need(ring_k.dim() == 4 and ring_k.shape[0] == S and ring_k.shape[1] == HEADS and ring_k.shape[3] == HEAD_DIM,
          "ring_k must be [S, 8, slots, 64]")
    slots = ring_k.shape[2]
    _need(ring_k.is_cuda and ring_k.dtype == torch.bfloat16 and ring_k.is_contiguous(), "ring_k must be contiguous bf16")
    _need(ring_v.is_cuda and ring_v.dtype in _VALUE_CODES and ring_v.is_contiguous()
          and ring_v.shape == ring_k.shape, "ring_v must match ring_k (float16 or bfloat16)")
    if stream_pos is not None:
        _need(stream_pos.is_cuda and stream_pos.dtype == torch.int32 and stream_pos.numel() == S
              and stream_pos.is_contiguous(), "stream_pos must be a contiguous CUDA int32 [S]")
    if q_workspace is None:
        q_workspace = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
    _check_frames(q_workspace, "q workspace", torch.bfloat16, S)
    if out is None:
        out = torch.empty((S, HIDDEN), dtype=torch.float32, device=x.device)
    _need(out.is_cuda and out.dtype == torch.float32 and out.is_contiguous() and out.numel() == S * HIDDEN,
          "out must be contiguous float32 [S, 512]")
    rc = lib.fm_decode_step_bf16(x.data_ptr(), w_qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), bstride,
                                 _ptr(stream_pos), int(position), q_workspace.data_ptr(), ring_k.data_ptr(),
                                 ring_v.data_ptr(), out.data_ptr(), S, slots, scale, _VALUE_CODES[ring_v.dtype] | in_flag,
                                 _status_ptr(status, x), _stream())
    _native.check(rc, "fm_decode_step_bf16")
    return out


class DecodePlan:
    """A validated, pre-bound ``decode_step`` for a fixed set of buffers: geometry is checked once, and each
    ``step`` is a single native call (the per-call checks of ``decode_step`` cost more host time than the
    kernels of a nearly empty ring take).  Buffers must stay alive and unchanged in place."""

    def __init__(self, x, w_qkv, ring_k, ring_v, *, scale=0.125, q_workspace=None, out=None, status=None):
        self._lib = _native.load()
        S = x.shape[0]
        cos = torch.zeros(1, 1, HEAD_DIM, device=x.device)
        # run the full validation once through the checked entry point's helpers
        _need(x.dim() == 2, "x must be [S, 512]")
        in_flag = _check_projection_inputs(x, w_qkv)
        _check_tables(cos, cos, S, 1)
        _need(ring_k.dim() == 4 and ring_k.shape[0] == S and ring_k.shape[1] == HEADS and ring_k.shape[3] == HEAD_DIM
              and ring_k.is_cuda and ring_k.dtype == torch.bfloat16 and ring_k.is_contiguous(),
              "ring_k must be contiguous bf16 [S, 8, slots, 64]")
        _need(ring_v.is_cuda and ring_v.dtype in _VALUE_CODES and ring_v.is_contiguous() and ring_v.shape == ring_k.shape,
              "ring_v must match ring_k (float16 or bfloat16)")
        self.q_workspace = (torch.empty(x.shape, dtype=torch.bfloat16, device=x.device) if q_workspace is None
                            else q_workspace)
        _check_frames(self.q_workspace, "q workspace", torch.bfloat16, S)
        self.out = torch.empty((S, HIDDEN), dtype=torch.float32, device=x.device) if out is None else out
        _need(self.out.is_cuda and self.out.dtype == torch.float32 and self.out.is_contiguous()
              and self.out.numel() == S * HIDDEN, "out must be contiguous float32 [S, 512]")
        self._keep = (x, w_qkv, ring_k, ring_v, status)
        self._args_head = (x.data_ptr(), w_qkv.data_ptr())
        self._args_tail = (self.q_workspace.data_ptr(), ring_k.data_ptr(), ring_v.data_ptr(), self.out.data_ptr(), S,
                           ring_k.shape[2], float(scale), _VALUE_CODES[ring_v.dtype] | in_flag, _status_ptr(status, x))

    def step(self, position: int, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        """``cos, sin``: contiguous float32 ``[1, 1, 64]`` tables of the new frame's position."""
        if position < 0:
            raise RuntimeError("unexpected attention geometry: position must not be negative")
        rc = self._lib.fm_decode_step_bf16(*self._args_head, cos.data_ptr(), sin.data_ptr(), 0, None, int(position),
                                           *self._args_tail, _stream())
        if rc != 0:
            _native.check(rc, "fm_decode_step_bf16")
        return self.out


def _strides3(t: torch.Tensor, frame_major: bool) -> list[int]:
    # (batch, head, time) strides in elements for a 4-D tensor whose last dim is contiguous.
    if frame_major:     # [B, T, H, D]
        return [t.stride(0), t.stride(2), t.stride(1)]
    return [t.stride(0), t.stride(1), t.stride(2)]   # [B, H, T, D]


def band_attention_fp32(q, k, v, *, window, scale, q_offset=0, k_offset=0, frame_major=False, out=None):
    """FP32 verification attention.  ``q [B,H,Tq,D]``, ``k, v [B,H,Tk,D]`` (or ``[B,T,H,D]`` with
    ``frame_major=True``); any strides with a contiguous last dimension.  Returns a tensor shaped like q."""
    lib = _native.load()
    for name, t in (("q", q), ("k", k), ("v", v)):
        _need(t.is_cuda and t.dtype == torch.float32 and t.dim() == 4 and t.stride(-1) == 1,
              f"{name} must be a 4-D CUDA float32 tensor with a contiguous last dimension")
    if frame_major:
        B, Tq, H, D = q.shape
        Tk = k.shape[1]
    else:
        B, H, Tq, D = q.shape
        Tk = k.shape[2]
    _need(k.shape == v.shape and k.shape[0] == B and k.shape[-1] == D, "k and v must match q in batch/heads/head_dim")
    _need(D <= 256, "head_dim must be at most 256")
    if out is None:
        out = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    _need(out.shape == q.shape and out.dtype == torch.float32 and out.stride(-1) == 1, "out must be shaped like q")
    strides = _strides3(q, frame_major) + _strides3(k, frame_major) + _strides3(v, frame_major) + _strides3(out, frame_major)
    import ctypes
    arr = (ctypes.c_longlong * 12)(*strides)
    rc = lib.fm_band_attn_fp32_verify(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, H, D, Tq, Tk,
                                      int(q_offset), int(k_offset), int(window), float(scale),
                                      ctypes.cast(arr, ctypes.c_void_p), _stream())
    _native.check(rc, "fm_band_attn_fp32_verify")
    return out


def linear_fp32(x, w):
    """``x [..., K] @ w[N, K]^T`` in FP32 on CUDA cores (verification path)."""
    lib = _native.load()
    _need(x.is_cuda and w.is_cuda and x.dtype == torch.float32 and w.dtype == torch.float32, "float32 CUDA tensors")
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    w = w.contiguous()
    _need(x2.shape[1] == w.shape[1], "inner dimensions differ")
    y = torch.empty((x2.shape[0], w.shape[0]), dtype=torch.float32, device=x.device)
    rc = lib.fm_linear_fp32_verify(x2.data_ptr(), w.data_ptr(), y.data_ptr(), x2.shape[0], w.shape[0], x2.shape[1],
                                   _stream())
    _native.check(rc, "fm_linear_fp32_verify")
    return y.view(*x.shape[:-1], w.shape[0])


def rope_fp32_(t, cos, sin):
    """In-place RoPE on ``t [B,T,H,D]`` FP32 with ``cos, sin [1 or B, T, D]``."""
    lib = _native.load()
    _need(t.is_cuda and t.dtype == torch.float32 and t.is_contiguous() and t.dim() == 4, "t must be contiguous [B,T,H,D]")
    B, T, H, D = t.shape
    cos, sin = cos.contiguous().float(), sin.contiguous().float()
    _need(cos.dim() == 3 and cos.shape[1] == T and cos.shape[2] == D and cos.shape[0] in (1, B), "bad cos shape")
    bstride = 0 if cos.shape[0] == 1 else T * D
    rc = lib.fm_rope_fp32_verify(t.data_ptr(), cos.data_ptr(), sin.data_ptr(), B, T, H, D, bstride, _stream())
    _native.check(rc, "fm_rope_fp32_verify")
    return t


# --------------------------------------------------------------------------- residual vector quantisation
RVQ_DIM = 256
# Candidate margins relative to |x| * max|e|: twice the worst-case error of an approximate distance, which is
# 4 * 2^-11 (FP16 rounding of both operands) with FP32 scores and 6 * 2^-11 with FP16-stored scores.
RVQ_TAU_REL = {torch.float32: 4.5e-3, torch.float16: 6.0e-3}


class RVQCodebooks:
    """Device-side constants of a residual quantiser stack, derived once from its codebook vectors
    ``[layers, entries, 256]`` float32 (the reference's ``MimiEuclideanCodebook.embed`` of every layer,
    src/fast_mimi/model.py:2262-2275): FP16 copies for the tensor core, squared norms, largest norm."""

    def __init__(self, codebooks: torch.Tensor) -> None:
        _need(codebooks.is_cuda and codebooks.dtype == torch.float32 and codebooks.dim() == 3
              and codebooks.shape[2] == RVQ_DIM and codebooks.shape[1] % 256 == 0 and codebooks.shape[1] <= 2048,
              "codebooks must be CUDA float32 [layers, entries (multiple of 256, at most 2048), 256]")
        self.vectors = codebooks.contiguous()
        self.half = self.vectors.half().contiguous()
        self.sq = (self.vectors.double() ** 2).sum(-1).float().contiguous()           # [layers, entries]
        self.e_max = [float(v) for v in self.sq.max(dim=1).values.sqrt().cpu()]
        self.layers, self.entries = codebooks.shape[0], codebooks.shape[1]


def rvq_encode(x, books: RVQCodebooks, num_quantizers=None, *, return_candidates=False, scores_dtype=None, status=None):
    """Codes ``[layers, rows]`` int64 of the residual quantiser stack for ``x [rows, 256]`` float32 (the output
    of the branch's ``input_proj``).  Per layer: inner products with all entries on the tensor core (FP16
    operands) pre-select, the exact FP32 distance decides among the candidates, the chosen entry is subtracted.
    By default (``scores_dtype=None``) the products never reach memory: the GEMM's epilogue reduces every 64 of them
    to a 16-byte candidate record.  ``scores_dtype=torch.float16 / torch.float32`` selects the older form in which the
    scores make one round trip through memory in that type.  ``x`` is not modified."""
    lib = _native.load()
    _need(x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.shape[1] == RVQ_DIM, "x must be CUDA float32 [rows, 256]")
    layers = books.layers if num_quantizers is None else int(num_quantizers)
    _need(0 < layers <= books.layers, "num_quantizers out of range")
    rows = x.shape[0]
    resid = x.contiguous().clone()
    resid16 = torch.empty(rows, RVQ_DIM, dtype=torch.float16, device=x.device)
    codes = torch.empty(layers, rows, dtype=torch.int64, device=x.device)
    cand = torch.empty(layers, rows, dtype=torch.int32, device=x.device) if return_candidates else None
    st = _status_ptr(status, x)
    if scores_dtype is None:
        tau_rel = RVQ_TAU_REL[torch.float32]          # FP32 accumulators feed the comparison directly
        tau = torch.empty(rows, dtype=torch.float32, device=x.device)
        records = torch.empty(rows, books.entries // 64, 4, dtype=torch.int32, device=x.device)
        _native.check(lib.fm_rvq_prepare_f32(resid.data_ptr(), resid16.data_ptr(), tau.data_ptr(), rows, books.e_max[0],
                                             tau_rel, _stream()), "fm_rvq_prepare_f32")
        for l in range(layers):
            rc = lib.fm_rvq_candidates_f16(resid16.data_ptr(), books.half[l].data_ptr(), books.sq[l].data_ptr(),
                                           tau.data_ptr(), records.data_ptr(), rows, books.entries, st, _stream())
            _native.check(rc, "fm_rvq_candidates_f16")
            e_next = books.e_max[l + 1] if l + 1 < layers else 0.0
            rc = lib.fm_rvq_select_rec_f32(records.data_ptr(), books.vectors[l].data_ptr(), resid.data_ptr(),
                                           resid16.data_ptr(), codes[l].data_ptr(),
                                           cand[l].data_ptr() if cand is not None else None, tau.data_ptr(), rows,
                                           books.entries, e_next, tau_rel, st, _stream())
            _native.check(rc, "fm_rvq_select_rec_f32")
        return (codes, cand) if return_candidates else codes
    _need(scores_dtype in RVQ_TAU_REL, "scores_dtype must be None, float16 or float32")
    scores = torch.empty(rows, books.entries, dtype=scores_dtype, device=x.device)
    _native.check(lib.fm_rvq_to_half(resid.data_ptr(), resid16.data_ptr(), rows, _stream()), "fm_rvq_to_half")
    for l in range(layers):
        linear(resid16, books.half[l], out_dtype=scores_dtype, out=scores, status=status)
        rc = lib.fm_rvq_select_f32(scores.data_ptr(), _OUT_CODES[scores_dtype], books.sq[l].data_ptr(), books.vectors[l].data_ptr(), resid.data_ptr(),
                                   resid16.data_ptr(), codes[l].data_ptr(), cand[l].data_ptr() if cand is not None else None,
                                   rows, books.entries, books.e_max[l], RVQ_TAU_REL[scores_dtype], st, _stream())
        _native.check(rc, "fm_rvq_select_f32")
    return (codes, cand) if return_candidates else codes


def split_half(x):
    """``x`` (float32, contiguous, a multiple of 8 values) as ``hi + lo`` with both parts float16."""
    lib = _native.load()
    _need(x.is_cuda and x.dtype == torch.float32 and x.is_contiguous() and x.numel() % 8 == 0,
          "x must be a contiguous CUDA float32 tensor with a multiple of 8 values")
    hi = torch.empty(x.shape, dtype=torch.float16, device=x.device)
    lo = torch.empty(x.shape, dtype=torch.float16, device=x.device)
    _native.check(lib.fm_split_half(x.data_ptr(), hi.data_ptr(), lo.data_ptr(), x.numel(), _stream()), "fm_split_half")
    return hi, lo


def linear_split(x, w_parts, *, status=None):
    """``x [rows, K] @ w^T`` with FP32-grade accuracy on the FP16 tensor core: ``x`` float32, ``w_parts`` the pair
    ``split_half(w)`` of a float32 ``[N, K]`` weight.  Three products with FP32 accumulation chained through the
    linear kernel's FP32 residual input: ``hi W_hi + hi W_lo + lo W_hi`` (the dropped ``lo W_lo`` term is below
    2^-22 of the result).  K a multiple of 64, N of 256."""
    w_hi, w_lo = w_parts
    x_hi, x_lo = split_half(x.contiguous())
    y = linear(x_hi, w_lo, out_dtype=torch.float32, status=status)
    y2 = linear(x_lo, w_hi, residual=y, out_dtype=torch.float32, status=status)
    return linear(x_hi, w_hi, residual=y2, out_dtype=torch.float32, out=y, status=status)


def downsample_conv(x, w_parts, *, kernel=4, stride=2, status=None):
    """The stride-2 causal, replicate-padded, bias-free convolution after the encoder transformer on frame-major
    activations: ``x [B, T, C]`` float32 -> ``[B, ceil(T / stride), C_out]`` float32.  ``w_parts`` =
    ``split_half(weight.permute(0, 2, 1).reshape(C_out, kernel * C))`` for an ``nn.Conv1d`` weight
    ``[C_out, C, kernel]``.  FP32-grade accuracy (split-precision tensor-core products)."""
    lib = _native.load()
    _need(x.is_cuda and x.dtype == torch.float32 and x.dim() == 3 and x.is_contiguous(), "x must be contiguous CUDA float32 [B, T, C]")
    B, T, C = x.shape
    w_hi, w_lo = w_parts
    _need(w_hi.shape == w_lo.shape and w_hi.shape[1] == kernel * C, f"weight parts must be [C_out, {kernel * C}]")
    t_out = (T + stride - 1) // stride
    hi = torch.empty(B * t_out, kernel * C, dtype=torch.float16, device=x.device)
    lo = torch.empty_like(hi)
    _native.check(lib.fm_conv_rows_split(x.data_ptr(), hi.data_ptr(), lo.data_ptr(), B, T, C, kernel, stride, _stream()),
                  "fm_conv_rows_split")
    y = linear(hi, w_lo, out_dtype=torch.float32, status=status)
    y2 = linear(lo, w_hi, residual=y, out_dtype=torch.float32, status=status)
    y = linear(hi, w_hi, residual=y2, out_dtype=torch.float32, out=y, status=status)
    return y.view(B, t_out, w_hi.shape[0])


def upsample2(x, weight):
    """The depthwise transposed convolution (kernel 4, stride 2, trailing two frames trimmed) that precedes the decoder
    transformer, on frame-major activations: ``x [B, T, C]`` float32, ``weight [C, 4]`` float32 -> ``[B, 2T, C]``."""
    lib = _native.load()
    _need(x.is_cuda and x.dtype == torch.float32 and x.dim() == 3 and x.is_contiguous(), "x must be contiguous CUDA float32 [B, T, C]")
    B, T, C = x.shape
    _need(weight.is_cuda and weight.dtype == torch.float32 and weight.is_contiguous() and tuple(weight.shape) == (C, 4)
          and C % 4 == 0, f"weight must be contiguous CUDA float32 [{C}, 4]")
    y = torch.empty(B, 2 * T, C, dtype=torch.float32, device=x.device)
    _native.check(lib.fm_upsample2_f32(x.data_ptr(), weight.data_ptr(), y.data_ptr(), B, T, C, _stream()), "fm_upsample2_f32")
    return y


def rvq_decode(codes, books: RVQCodebooks):
    """``sum_l E_l[codes[l]]`` as float32 ``[rows, 256]``, layers added left to right from an FP32 zero (the
    accumulation order of the reference's decode, src/fast_mimi/model.py:2431-2444, before ``output_proj``)."""
    lib = _native.load()
    _need(codes.is_cuda and codes.dtype == torch.int64 and codes.dim() == 2 and codes.is_contiguous(),
          "codes must be contiguous CUDA int64 [layers, rows]")
    layers, rows = codes.shape
    _need(0 < layers <= books.layers, "more code layers than codebooks")
    out = torch.empty(rows, RVQ_DIM, dtype=torch.float32, device=codes.device)
    bad = torch.zeros(1, dtype=torch.int32, device=codes.device)
    rc = lib.fm_rvq_decode_f32(codes.data_ptr(), books.vectors.data_ptr(), out.data_ptr(), rows, layers, books.entries,
                               bad.data_ptr(), _stream())
    _native.check(rc, "fm_rvq_decode_f32")
    if int(bad.item()) != 0:
        raise RuntimeError("rvq_decode: a code index is outside the codebook")
    check_status(codes.device)      # the stream is already synchronised by the read above
    return out
