"""ctypes binding of libhexb200.so (the C ABI declared in include/hexb.h).

The library is the product; there is no Python or CPU fallback.  Loading fails loudly when the
shared object has not been built, and every call raises ``HexbError`` on a non-zero status.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libhexb200.so"

HEXB_OK = 0
HEXB_DT_F16 = 1
HEXB_DT_F32 = 2
HEXB_DT_I32 = 6   # the reference's raw-tensor id of Int32 (test/utils/dsp/include/tensor.h:26-38)


class HexbError(RuntimeError):
    """Raised when a libhexb200 entry point returns a non-zero status."""

    def __init__(self, status: int, name: str, detail: str = ""):
        self.status = status
        self.status_name = name
        super().__init__(f"{name} ({status})" + (f": {detail}" if detail else ""))


class DecoderConfig(C.Structure):
    _fields_ = [
        ("n_layers", C.c_int32), ("d_model", C.c_int32), ("n_heads", C.c_int32),
        ("head_dim", C.c_int32), ("d_ff", C.c_int32), ("batch", C.c_int32), ("seq", C.c_int32),
        ("rms_eps", C.c_float),
    ]


class DecoderWeights(C.Structure):
    _fields_ = [(n, C.POINTER(C.c_void_p)) for n in ("wqkv", "wo", "wgu", "wd", "g1", "g2")]


class AttentionDesc(C.Structure):
    """hexb_attention_desc of include/hexb.h."""
    _fields_ = [
        ("Q", C.c_void_p), ("K", C.c_void_p), ("V", C.c_void_p), ("Out", C.c_void_p), ("mask", C.c_void_p),
        ("Z", C.c_int64), ("H", C.c_int64), ("N_Q", C.c_int64), ("N_KV", C.c_int64), ("D", C.c_int64),
        ("strides", C.c_int64 * 12), ("mask_strides", C.c_int64 * 3),
        ("in_dtype", C.c_int), ("out_dtype", C.c_int), ("mask_dtype", C.c_int),
        ("sm_scale", C.c_float), ("causal", C.c_int),
    ]


_i64, _vp, _f, _i = C.c_int64, C.c_void_p, C.c_float, C.c_int

# name -> (restype, argtypes); mirrors include/hexb.h one to one.
PROTOTYPES = {
    "hexb_version": (_i, []),
    "hexb_status_string": (C.c_char_p, [_i]),
    "hexb_last_cuda_error": (C.c_char_p, []),
    "hexb_device_status": (_i, [C.POINTER(_i)]),
    "hexb_selftest_bounded_wait": (_i, [_i, _vp]),
    "hexb_softmax_f32": (_i, [_vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    "hexb_softmax_f16": (_i, [_vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    "hexb_layer_norm_f32": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _f, _vp]),
    "hexb_layer_norm_f16": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _f, _vp]),
    "hexb_rms_norm_f32": (_i, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _f, _vp]),
    "hexb_rms_norm_f16": (_i, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _f, _vp]),
    "hexb_matmul_f16": (_i, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i, _vp]),
    "hexb_matmul_f16_nt": (_i, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i, _vp]),
    "hexb_matmul_swiglu_f16": (_i, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _vp]),
    "hexkl_matmul_f16f16_f32": (_i, [_i64, _i64, _i64, _vp, _vp, _vp]),
    "hexb_linear_f16": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _vp]),
    "hexb_embedding_f16": (_i, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp]),
    "hexb_iota": (_i, [_i, _vp, _i64, _vp]),
    "hexb_cumsum": (_i, [_i, _vp, _vp, _i64, _i64, _i64, _i, _vp]),
    "hexb_attention_fwd_ex": (_i, [C.POINTER(AttentionDesc), _vp]),
    "hexb_attention_fwd_f16": (_i, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, C.POINTER(_i64), _f, _i, _vp]),
    "hexb_attention_fwd_f32": (_i, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, C.POINTER(_i64), _f, _i, _vp]),
    "hexb_silu_f32": (_i, [_vp, _vp, _i64, _vp]),
    "hexb_silu_f16": (_i, [_vp, _vp, _i64, _vp]),
    "hexb_swiglu_f16": (_i, [_vp, _vp, _i64, _i64, _vp]),
    "hexb_unary": (_i, [_i, _i, _vp, _vp, _i64, _vp]),
    "hexb_binary": (_i, [_i, _i, _vp, _vp, _vp, _i64, _vp]),
    "hexb_sum": (_i, [_i, _vp, _vp, _i64, _vp]),
    "hexb_rope": (_i, [_i, _vp, _vp, _i64, _i64, _i64, _i64, C.POINTER(_i64), C.POINTER(_i64), _f, _vp]),
    "hexb_decoder_workspace_bytes": (C.c_size_t, [C.POINTER(DecoderConfig)]),
    "hexb_decoder_forward_f16": (_i, [C.POINTER(DecoderConfig), C.POINTER(DecoderWeights), _vp, _vp, _vp, C.c_size_t, _vp]),
    "hexb_decoder_forward_f16_noalloc": (_i, [C.POINTER(DecoderConfig), C.POINTER(DecoderWeights), _vp, _vp, _vp]),
    "hexb_softmax_host": (_i, [_i, _vp, _vp, _i64, _i64]),
    "hexb_layer_norm_host": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _f]),
    "hexb_rms_norm_host": (_i, [_i, _vp, _vp, _vp, _i64, _i64, _f]),
    "hexb_matmul_f16_host": (_i, [_vp, _vp, _vp, _i64, _i64, _i64, _i]),
    "hexb_attention_fwd_host": (_i, [_i, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _f, _i]),
    "hexb_host_staging_release": (_i, []),
    "hexb_set_option": (_i, [C.c_char_p, _i]),
    "hexb_get_option": (_i, [C.c_char_p, C.POINTER(_i)]),
}

_lib = None


def load() -> C.CDLL:
    """Loads libhexb200.so once and attaches the prototypes.  No fallback: a missing library is an error."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python hexagon-mlir_b200/build.py` "
                "(there is no CPU or PyTorch fallback)"
            )
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(status: int, what: str = "") -> None:
    if status != HEXB_OK:
        lib = load()
        name = lib.hexb_status_string(status).decode()
        detail = lib.hexb_last_cuda_error().decode() if name == "HEXB_ERR_CUDA" else ""
        raise HexbError(status, name, (what + " " + detail).strip())


def set_option(key: str, value: int) -> None:
    check(load().hexb_set_option(key.encode(), int(value)), f"set_option({key})")


def device_status() -> int:
    out = C.c_int(0)
    check(load().hexb_device_status(C.byref(out)), "device_status")
    return out.value
