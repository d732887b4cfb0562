"""GPU parity for the elementwise row: GELU, cos/sin/rsqrt, add/sub/mul/div, whole-vector sum, RoPE.
Golden fixtures from the reference's Triton kernels, the oracle on seeded inputs, the reference
tests' own tolerances (gelu 1e-5 / 1e-2, rope 1e-3 / 1e-2, sum 1e-2, div 1e-6, cos/sin/rsqrt 1e-5),
odd sizes, unaligned views and empty inputs."""
import os

import numpy as np
import pytest
import torch

import hexb200
from hexb200 import kernels, ops
from oracle import oracle as O

pytestmark = pytest.mark.gpu
dev = torch.device("cuda:0")


def load(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    return {k: torch.from_numpy(z[k]) for k in z.files}


def run_unary(op, x):
    xd = x.to(dev)
    y = torch.empty_like(xd)
    ops.unary(op, xd, y)
    return y.cpu()


@pytest.mark.parametrize("tag,atol", [("f32", 1e-5), ("f16", 1e-2)])
def test_gelu_golden(golden_dir, tag, atol):
    g = load(golden_dir, f"gelu_16384_{tag}")
    y = run_unary("gelu_tanh", g["in0"])
    assert torch.allclose(y, g["output"], atol=atol)
    assert torch.allclose(y, g["expected"], atol=atol)
    assert torch.allclose(y, O.c_gelu(g["in0"]), atol=atol)


@pytest.mark.parametrize("n", [1, 7, 1001, 16384, (1 << 22) + 3])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_unary_vs_oracle(n, dtype):
    g = torch.Generator().manual_seed(n)
    x = (torch.randn(n, generator=g) * 2).to(dtype)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert torch.allclose(run_unary("gelu_tanh", x), O.torch_gelu(x), atol=tol)
    assert torch.allclose(run_unary("cos", x), torch.cos(x.float()).to(dtype), atol=tol)
    assert torch.allclose(run_unary("sin", x), torch.sin(x.float()).to(dtype), atol=tol)
    xp = (torch.rand(n, generator=g) + 0.05).to(dtype)
    assert torch.allclose(run_unary("rsqrt", xp), torch.rsqrt(xp.float()).to(dtype), atol=tol, rtol=1e-3)


def test_math_ops_golden(golden_dir):
    g = load(golden_dir, "math_ops_cos_sin_f32")
    assert torch.allclose(run_unary("cos", g["in0"]), g["output0"], atol=1e-5)
    assert torch.allclose(run_unary("sin", g["in0"]), g["output1"], atol=1e-5)


def test_binary_golden_and_odd(golden_dir):
    g = load(golden_dir, "vec_add_f32")
    a, b = g["in0"].to(dev), g["in1"].to(dev)
    out = torch.empty_like(a)
    ops.binary("add", a, b, out)
    assert torch.allclose(out.cpu(), g["output"])
    g = load(golden_dir, "vec_div_2d_f32")
    a, b = g["in0"].to(dev), g["in1"].to(dev)
    out = torch.empty_like(a)
    ops.binary("div", a, b, out)
    assert torch.allclose(out.cpu(), g["output"], atol=1e-6)
    gen = torch.Generator().manual_seed(3)
    for n, dtype in ((1, torch.float32), (1003, torch.float16), (65537, torch.float32)):
        a = torch.randn(n, generator=gen).to(dtype)
        b = (torch.rand(n, generator=gen) + 0.5).to(dtype)
        for op, ref in (("add", a.float() + b.float()), ("sub", a.float() - b.float()),
                        ("mul", a.float() * b.float()), ("div", a.float() / b.float())):
            out = torch.empty(n, dtype=dtype, device=dev)
            ops.binary(op, a.to(dev), b.to(dev), out)
            assert torch.equal(out.cpu(), ref.to(dtype)), op            # exact: one rounding of the fp32 result
    # unaligned views take the scalar path
    big = torch.randn(4099, generator=gen)
    a, b = big[1:4098].to(dev), big[2:4099].to(dev)
    base = torch.empty(4100, device=dev)
    out = base[3:4100]
    ops.binary("add", a.contiguous(), b.contiguous(), out)
    assert torch.equal(out.cpu(), big[1:4098] + big[2:4099])
    e = torch.empty(0, device=dev)
    ops.binary("add", e, e, torch.empty_like(e))


def test_sum(golden_dir):
    g = load(golden_dir, "sum_16384_f32")
    x = g["in0"].to(dev)
    out = torch.empty(1, device=dev)
    ops.vec_sum(x, out)
    assert torch.allclose(out.cpu(), g["output"], atol=1e-2)
    assert torch.allclose(out.cpu(), g["expected"], atol=1e-2)
    gen = torch.Generator().manual_seed(42)                         # the reference's shape and seed
    for dtype in (torch.float16, torch.float32):
        x = torch.randn(1024 * 1024, dtype=dtype, generator=gen)
        out = torch.empty(1, dtype=dtype, device=dev)
        ops.vec_sum(x.to(dev), out)
        assert abs(float(out) - O.c_sum(x)) < (1e-2 if dtype == torch.float32 else 0.5)
        out2 = torch.empty(1, dtype=dtype, device=dev)
        ops.vec_sum(x.to(dev), out2)
        assert torch.equal(out, out2)                               # fixed order: deterministic
    for n in (0, 1, 5, 1023, 1025, 4097):
        x = torch.arange(n, dtype=torch.float32)
        out = torch.full((1,), -1.0, device=dev)
        ops.vec_sum(x.to(dev), out)
        assert float(out) == float(x.sum())


@pytest.mark.parametrize("tag,atol", [("f32", 1e-3), ("f16", 1e-2)])
def test_rope_golden(golden_dir, tag, atol):
    g = load(golden_dir, f"rope_4x8x16x32_{tag}")
    x = g["in0"].to(dev)
    out = torch.empty_like(x)
    ops.rope(x, out, theta=10000.0)
    assert torch.allclose(out.cpu(), g["output"], atol=atol, rtol=0)
    assert torch.allclose(out.cpu(), g["expected"], atol=atol, rtol=0)
    assert torch.allclose(out.cpu(), O.c_rope(g["in0"]), atol=atol, rtol=0)


def test_rope_shapes_and_strides():
    gen = torch.Generator().manual_seed(9)
    for (B, L, H, D) in ((1, 1, 1, 2), (2, 1024, 16, 128), (3, 77, 5, 64)):
        x = torch.randn(B, L, H, D, generator=gen)
        out = torch.empty(B, L, H, D, device=dev)
        ops.rope(x.to(dev), out, theta=10000.0)
        assert torch.allclose(out.cpu(), O.torch_rope(x), atol=2e-3, rtol=0)   # large angles: fp32 sin/cos
        # rotation preserves the norm of every (even, odd) pair
        assert torch.allclose(out.cpu().pow(2).sum(-1), x.pow(2).sum(-1), rtol=1e-4)
    # heads selected by strides (q inside a packed qkv tensor)
    qkv = torch.randn(2, 64, 3, 4, 32, generator=gen).to(dev)
    q = qkv[:, :, 0]
    out = torch.empty(2, 64, 4, 32, device=dev)
    ops.rope(q, out)
    assert torch.allclose(out.cpu(), O.torch_rope(q.cpu().contiguous()), atol=1e-3, rtol=0)


def test_reference_style_launchers():
    # the launch forms of test_gelu.py, test_vec_add_with_scalar.py, test_sum.py, test_rope.py (CPU tensors)
    x = torch.rand(16384)
    out = torch.empty_like(x)
    kernels.lookup("gelu_kernel_float32")[(4,)](x, out, BLOCK_SIZE=4096, enableMultiThreading=False,
                                                enableVTCMTiling=False)
    assert torch.allclose(out, torch.nn.functional.gelu(x, approximate="tanh"), atol=1e-5)
    y = torch.rand(16384)
    kernels.add_kernel_scalar[(4,)](x, y, out, 16384, BLOCK_SIZE=4096, enableVTCMTiling=True)
    assert torch.allclose(out, x + y, atol=1e-2)
    s = torch.empty(1)
    kernels.sum_kernel[1, ](x, s, BLOCK_SIZE=16384, enableSplitReduction=True)
    assert torch.allclose(s, torch.sum(x), atol=1e-2)
    xr = torch.rand(4, 8, 16, 32, dtype=torch.float16)
    outr = torch.empty_like(xr)
    kernels.lookup("rope_kernel_float16")[(4,)](
        xr, outr, BATCH_SIZE=4, BATCH_SIZE_STRIDE=8 * 16 * 32, SEQ_LEN=8, SEQ_LEN_STRIDE=16 * 32, N_HEADS=16,
        N_HEADS_STRIDE=32, N_FEATURES=32, N_FEATURES_STRIDE=1, BLOCK_SIZE=1, THETA=10000.0,
        enableMultiThreading=False)
    torch.testing.assert_close(outr, O.torch_rope(xr), atol=1e-2, rtol=0)
    xm = torch.linspace(0, 3.14, 1024)
    ym = torch.empty_like(xm)
    kernels.cos_kernel[(1,)](xm, ym, BLOCK_SIZE=1024)
    assert torch.allclose(ym, torch.cos(xm), atol=1e-5)
    kernels.rsqrt_kernel[(1,)](x[:1024].contiguous() + 0.1, ym, BLOCK_SIZE=1024)
    assert torch.allclose(ym, torch.rsqrt(x[:1024] + 0.1), atol=1e-5)
    a2, b2 = torch.rand(64, 256), torch.rand(64, 256) + 0.5
    o2 = torch.empty_like(a2)
    kernels.div_kernel[(1,)](a2, b2, o2, 64, 256)
    assert torch.allclose(o2, a2 / b2, atol=1e-6)
    kernels.add_2d_kernel[(1,)](a2, b2, o2, NUM_ROWS=64, NUM_COLS=256, enableMultiThreading=True)
    assert torch.allclose(o2, a2 + b2)
    assert hexb200.device_status() == 0


# ------------------------------------------------------------------ cumulative sum (ttx.cumsum / additive ttx.scan)
@pytest.mark.parametrize("shape,axis", [((16, 32), 1), ((256,), 0), ((1000, 4096), 1), ((3, 100003), 1),
                                        ((1, 5_000_000), 1), ((7, 333, 5), 1), ((64, 128, 96), 0), ((4097,), 0),
                                        ((2, 3000, 40), 1), ((16384, 2048), 1)])
@pytest.mark.parametrize("reverse", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.int32])
def test_cumsum_vs_oracle(shape, axis, reverse, dtype):
    g = torch.Generator().manual_seed(sum(shape) + axis)
    if dtype == torch.int32:
        x = torch.randint(-2 ** 30, 2 ** 30, shape, generator=g, dtype=torch.int32)
    else:
        x = torch.rand(*shape, generator=g) - 0.25                     # positive drift: sums grow, no cancellation
        if dtype == torch.float16:
            x = x * min(1.0, 2000.0 / shape[axis])                     # keeps the running sum inside fp16's range
        x = x.to(dtype)
    out = torch.empty_like(x, device=dev)
    ops.cumsum(x.to(dev), out, axis=axis, reverse=reverse)
    ref = O.c_cumsum(x, axis, reverse)
    if dtype == torch.int32:
        assert torch.equal(out.cpu(), ref)                            # bit-exact, wrapping
    else:
        scale = ref.abs().max().item()
        tol = 1e-3 if dtype == torch.float32 else 2e-2 / 8            # fp16: half an ulp of the output
        assert (out.cpu().float() - ref).abs().max().item() <= tol * scale


def test_cumsum_segmented_rows_match_single_segment():
    """A row cut into segments (three launches) gives the sums of the one-CTA-per-row walk."""
    g = torch.Generator().manual_seed(8)
    x = torch.randint(-1000, 1000, (2, 1_000_000), generator=g, dtype=torch.int32).to(dev)
    a = torch.empty_like(x)
    b = torch.empty_like(x)
    ops.cumsum(x, a)
    hexb200.set_option("scan_segments", 1)
    try:
        ops.cumsum(x, b)
    finally:
        hexb200.set_option("scan_segments", 0)
    assert torch.equal(a, b)
    assert torch.equal(a.cpu(), x.cpu().cumsum(1).to(torch.int32))
