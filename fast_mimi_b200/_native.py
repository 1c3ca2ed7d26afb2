"""ctypes binding of ``libfast_mimi_b200.so`` (the C ABI declared in ``include/fast_mimi_b200.h``).

Mirrors how the reference binds its own native kernels (``ctypes.CDLL`` with explicit ``argtypes`` and
``restype = c_int``: src/fast_mimi/_native_cutlass.py:110-116), except that nothing is compiled at
call time and there is no fallback: a missing library raises.
"""
from __future__ import annotations

import ctypes
import os
import threading

from ._build import LIB_PATH

_P, _I, _LL, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float

#: name -> argtypes, in header order.  tests/test_host_logic.py checks this table against the header.
SIGNATURES: dict[str, list] = {
    "fm_abi_version": [],
    "fm_qkv_rope_bf16": [_P, _P, _P, _P, _LL, _P, _P, _P, _I, _I, _I, _P, _P],
    "fm_out_proj_f16": [_P, _P, _P, _P, _P, _LL, _I, _P, _P],
    "fm_linear_f16": [_P, _P, _P, _P, _P, _LL, _I, _I, _I, _I, _I, _P, _P],
    "fm_layernorm_f16": [_P, _I, _P, _P, _F, _P, _I, _LL, _P],
    "fm_rvq_select_f32": [_P, _I, _P, _P, _P, _P, _P, _P, _LL, _I, _F, _F, _P, _P],
    "fm_conv_rows_split": [_P, _P, _P, _I, _I, _I, _I, _I, _P],
    "fm_upsample2_f32": [_P, _P, _P, _I, _I, _I, _P],
    "fm_split_half": [_P, _P, _P, _LL, _P],
    "fm_rvq_prepare_f32": [_P, _P, _P, _LL, _F, _F, _P],
    "fm_rvq_candidates_f16": [_P, _P, _P, _P, _P, _LL, _I, _P, _P],
    "fm_rvq_select_rec_f32": [_P, _P, _P, _P, _P, _P, _P, _LL, _I, _F, _F, _P, _P],
    "fm_rvq_to_half": [_P, _P, _LL, _P],
    "fm_rvq_decode_f32": [_P, _P, _P, _LL, _I, _I, _P, _P],
    "fm_band_attn_prefill_bf16": [_P, _P, _P, _P, _I, _I, _I, _F, _I, _P, _P],
    "fm_attention_prefill_bf16": [_P, _P, _P, _P, _LL, _P, _P, _P, _P, _I, _I, _I, _F, _I, _P, _P],
    "fm_band_attn_chunk_bf16": [_P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _P, _P],
    "fm_attention_fused_bf16": [_P, _P, _P, _P, _LL, _P, _I, _I, _I, _F, _I, _P, _P],
    "fm_attention_chunk_bf16": [_P, _P, _P, _P, _LL, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P, _P],
    "fm_attention_prefill_static_bf16": [_P, _P, _P, _P, _LL, _P, _I, _I, _I, _F, _I, _P, _P],
    "fm_decode_step_bf16": [_P, _P, _P, _P, _LL, _P, _I, _P, _P, _P, _P, _I, _I, _F, _I, _P, _P],
    "fm_ring_attn_decode_bf16": [_P, _P, _P, _P, _P, _I, _I, _I, _F, _I, _P, _P],
    "fm_band_attn_fp32_verify": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _P, _P],
    "fm_linear_fp32_verify": [_P, _P, _P, _I, _I, _I, _P],
    "fm_rope_fp32_verify": [_P, _P, _P, _I, _I, _I, _I, _LL, _P],
    "fm_selftest_wait_timeout": [_P, _I, _P, _P],
    "fm_read_status": [_P, _P],
}

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None


class NativeLibraryMissing(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """Load the library once.  Raises ``NativeLibraryMissing`` if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise NativeLibraryMissing(
                    f"{LIB_PATH} is missing: build it with `python -m fast_mimi_b200._build` "
                    "(there is no CPU or PyTorch fallback for these kernels)")
            lib = ctypes.CDLL(LIB_PATH)
            for name, argtypes in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.argtypes = argtypes
                fn.restype = _I
            _lib = lib
    return _lib


def check(rc: int, what: str) -> None:
    """Turn a non-zero native status into an exception, as the reference's launchers do
    (src/fast_mimi/_native_cutlass.py:163-164)."""
    if rc != 0:
        kind = {-1: "rejected geometry", -2: "grid too large", -3: "misaligned pointer",
                -4: "cuTensorMapEncodeTiled unavailable",
                -5: "more frames than the built-in workspace holds",
                -6: "clip length outside the fused kernel's range (128 < T <= 256)"}.get(rc, "CUDA error" if rc > 0 else "error")
        raise RuntimeError(f"{what} failed with status {rc} ({kind})")
