"""GPU: the allocation-free decoder entry point (hexb_decoder_forward_f16_noalloc).

Some hosts cannot call cudaMalloc when they need a forward pass: they gave all device memory to
their own pool at start-up, or they run a serving loop whose latency bound leaves no room for an
allocation.  For them the library carries its intermediate activations in a fixed 64 MiB array
inside the library image.  This test calls that entry point through the C ABI twice in a row with
different inputs (the array is shared and keeps the first call's contents, so the second call shows
that stale contents do not leak into the result) and compares each output with the workspace-taking
entry point on the same inputs -- bit for bit, since both run the same kernels on the same data -- and
with the CPU oracle within the fp16 tolerance of the other GPU tests.  The second call must leave
the amount of free device memory unchanged (the first call on a device is where the driver
instantiates the library's image, so only later calls are held to that).  It also checks that a
configuration beyond the fixed array is refused with HEXB_ERR_WORKSPACE.
The file name sorts last so that a run stopping at the first failure has already run every other test.
"""
import ctypes as C
import os
import re

import pytest
import torch

import hexb200
from hexb200 import _lib, ops
from oracle import oracle as O

pytestmark = pytest.mark.gpu

REL_F16 = 2e-2


def static_scratch_bytes() -> int:
    """HEXB_DECODER_STATIC_SCRATCH_BYTES as the header states it."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    text = open(os.path.join(root, "include", "hexb.h")).read()
    m = re.search(r"#define\s+HEXB_DECODER_STATIC_SCRATCH_BYTES\s+\((\d+)u\s*<<\s*(\d+)\)", text)
    assert m, "the header no longer states the size of the fixed array"
    return int(m.group(1)) << int(m.group(2))


def test_noalloc_decoder_matches_workspace_entry_point_twice():
    assert torch.cuda.is_available()
    lib = hexb200.load()
    dev = torch.device("cuda:0")
    L, d, H, f, B, S = 2, 256, 2, 512, 2, 128
    x1, ws = O.make_decoder_inputs(L, d, H, f, B, S, seed=2001)
    x2, _ = O.make_decoder_inputs(L, d, H, f, B, S, seed=2002)
    wd = [{k: v.to(dev) for k, v in w.items()} for w in ws]
    stack = ops.DecoderStack(wd, H, d // H, f, B, S, 1e-6)          # owns the weight pointer tables
    assert stack.ws_bytes <= static_scratch_bytes()
    stream = torch.cuda.current_stream().cuda_stream
    for call, x in enumerate((x1, x2)):                             # two calls in a row, shared array
        xd = x.to(dev)
        want = torch.empty_like(xd)
        stack.forward(xd, want)                                     # existing entry point, explicit workspace
        got = torch.full_like(xd, float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]
        st = lib.hexb_decoder_forward_f16_noalloc(C.byref(stack.cfg), C.byref(stack.cweights), xd.data_ptr(),
                                                  got.data_ptr(), stream)
        assert st == 0, lib.hexb_status_string(st)
        torch.cuda.synchronize()
        if call > 0:                                                # nothing was allocated on the device
            assert torch.cuda.mem_get_info(dev)[0] == free_before
        assert hexb200.device_status() == 0
        assert torch.isfinite(got).all()
        assert torch.equal(got, want)                               # same kernels, same data: same bits
        assert O.max_rel_err(got.cpu(), O.torch_decoder(x, ws, H, d // H, f, B, S, 1e-6)) < REL_F16


def test_noalloc_decoder_refuses_sizes_beyond_the_fixed_array():
    lib = hexb200.load()
    big = _lib.DecoderConfig(4, 2048, 16, 128, 8192, 8, 1024, 1e-6)   # needs ~608 MiB of intermediates
    assert lib.hexb_decoder_workspace_bytes(C.byref(big)) > static_scratch_bytes()
    st = lib.hexb_decoder_forward_f16_noalloc(C.byref(big), None, None, None, None)
    assert lib.hexb_status_string(st).decode() == "HEXB_ERR_WORKSPACE"
