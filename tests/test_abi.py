"""CPU: the C-ABI library loads without a GPU, exports every symbol include/hexb.h declares, and
its host-side entry logic (status strings, option store, workspace query, argument checks that run
before any device call) behaves.  No compute call is made."""
import ctypes as C
import os
import re

import pytest

import hexb200
from hexb200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "hexb.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b((?:hexb|hexkl)_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    for must in ("hexb_softmax_f32", "hexb_layer_norm_f16", "hexb_rms_norm_f16", "hexb_matmul_f16",
                 "hexkl_matmul_f16f16_f32", "hexb_attention_fwd_f16", "hexb_decoder_forward_f16",
                 "hexb_layer_norm_host"):
        assert must in names


def test_library_exports_every_declared_symbol():
    lib = hexb200.load()
    for name in declared_functions():
        assert hasattr(lib, name), f"libhexb200.so lacks {name}"


def test_binding_covers_every_declared_symbol():
    assert sorted(_lib.PROTOTYPES) == declared_functions()


def test_status_strings_and_version():
    lib = hexb200.load()
    assert lib.hexb_version() >= 100
    names = {0: "HEXB_OK", -1: "HEXB_ERR_BAD_ARG", -2: "HEXB_ERR_UNSUPPORTED", -3: "HEXB_ERR_MISALIGNED",
             -4: "HEXB_ERR_CUDA", -5: "HEXB_ERR_TIMEOUT", -6: "HEXB_ERR_WORKSPACE", -7: "HEXB_ERR_NO_DEVICE"}
    for code, name in names.items():
        assert lib.hexb_status_string(code).decode() == name
    assert lib.hexb_status_string(-99).decode() == "HEXB_ERR_UNKNOWN"


def test_option_store():
    lib = hexb200.load()
    assert lib.hexb_set_option(b"norm_vpt_max", 4) == 0
    v = C.c_int(0)
    assert lib.hexb_get_option(b"norm_vpt_max", C.byref(v)) == 0 and v.value == 4
    assert lib.hexb_set_option(b"not_an_option", 1) == -1
    assert lib.hexb_set_option(None, 1) == -1
    assert lib.hexb_get_option(b"never_set_gemm_bn_like", C.byref(v)) == -1
    assert lib.hexb_get_option(b"gemm_bn", C.byref(v)) == -1          # a known key that was never set
    # switches that could make a kernel skip work or mis-describe an operand are not in the shipped table
    for dev_only in (b"ring_dbg", b"gemm_b_lbo", b"gemm_b_sbo", b"attn_v_lbo", b"attn_v_sbo"):
        assert lib.hexb_set_option(dev_only, 1) == -1
    with pytest.raises(hexb200.HexbError):
        hexb200.set_option("nope", 1)


def test_argument_checks_that_need_no_device():
    lib = hexb200.load()
    # negative sizes and null pointers are rejected before anything touches CUDA
    assert lib.hexb_softmax_f32(None, None, -1, 4, 4, 4, None) == -1
    assert lib.hexb_softmax_f32(None, None, 0, 4, 4, 4, None) == 0          # empty: nothing to do
    assert lib.hexb_softmax_f32(None, None, 4, 4, 4, 4, None) == -1
    assert lib.hexb_layer_norm_f16(None, None, None, None, None, None, 2, 0, 0, 0, 1e-5, None) == 0
    assert lib.hexb_matmul_f16(None, None, None, None, 4, 4, 4, 4, 4, 4, 99, None) == -2
    assert lib.hexb_matmul_f16(None, None, None, None, 0, 4, 4, 4, 4, 4, 1, None) == 0
    assert lib.hexb_matmul_f16(None, None, None, None, 4, 4, 4, 4, 4, 4, 1, None) == -1
    assert lib.hexb_attention_fwd_f16(None, None, None, None, 1, 1, 0, 64, None, 1.0, 0, None) == 0
    assert lib.hexb_attention_fwd_f16(None, None, None, None, 1, 1, 8, 64, None, 1.0, 0, None) == -1
    assert lib.hexb_swiglu_f16(None, None, 4, 12, None) == -1
    assert lib.hexb_softmax_host(7, None, None, 4, 4) == -2                  # unknown dtype id


def test_decoder_workspace_query():
    lib = hexb200.load()
    cfg = _lib.DecoderConfig(4, 2048, 16, 128, 8192, 8, 1024, 1e-6)
    need = lib.hexb_decoder_workspace_bytes(C.byref(cfg))
    T = 8 * 1024
    assert need >= T * (7 * 2048 + 3 * 8192) * 2
    assert need % 256 == 0
    bad = _lib.DecoderConfig(4, 2048, 15, 128, 8192, 8, 1024, 1e-6)          # heads * head_dim != d_model
    assert lib.hexb_decoder_workspace_bytes(C.byref(bad)) == 0
    assert lib.hexb_decoder_forward_f16(C.byref(bad), None, None, None, None, 0, None) == -1


def test_missing_library_is_an_error(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "libhexb200.so")
    with pytest.raises(ImportError):
        _lib.load()
