"""hexb200: the hexagon-mlir kernel set (row softmax, LayerNorm, RMSNorm, fp16 matmul,
flash-attention forward, decoder block stack) as hand-written sm_100a CUDA kernels behind a C ABI.

    import hexb200
    hexb200.kernels.softmax_kernel[(4,)](x, out, NUM_ROWS=r, NUM_COLS=c, BLOCK_SIZE=b)   # reference signature
    hexb200.ops.softmax(x, out)                                                        # tensor-level

The arithmetic lives in libhexb200.so (include/hexb.h); importing this package does not load it,
the first call does, and a missing library is an error (there is no CPU or PyTorch fallback).
"""
from . import _lib, gpt2, kernels, ops, options, report  # noqa: F401
from ._lib import HexbError, device_status, load, set_option  # noqa: F401

__all__ = ["gpt2", "kernels", "ops", "options", "report", "HexbError", "load", "set_option", "device_status"]
