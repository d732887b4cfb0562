"""GPU parity tests: the CUDA kernels, called through the C ABI (ctypes over libhexb200.so), against
the CPU oracle on the same seeded inputs, against the golden fixtures made from the reference's own
Triton kernels, and -- at the benchmark's full sizes -- through size-independent properties.

Tolerances: the benchmark's (1e-3 relative for fp32 kernels, 2e-2 for fp16 with fp32 accumulation)
and, on the reference's own shapes, the reference tests' own (softmax atol 1e-5/1e-3, layer norm
1e-5, rms norm 1e-2, matmul 0.2 and rtol 1e-2, flash attention allclose defaults widened to the
fp32 round-off of a different summation order, silu 1e-2)."""
import ctypes as C
import math
import os

import numpy as np
import pytest
import torch

import hexb200
from hexb200 import ops
from oracle import oracle as O

pytestmark = pytest.mark.gpu

REL_F32 = 1e-3
REL_F16 = 2e-2


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    hexb200.load()
    return torch.device("cuda:0")


def load(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    return {k: torch.from_numpy(z[k]) for k in z.files}


def gpu_softmax(x, dev):
    xd = x.to(dev)
    yd = torch.empty_like(xd)
    ops.softmax(xd, yd)
    return yd.cpu()


# ------------------------------------------------------------------ softmax
@pytest.mark.parametrize("tag,atol", [("f32", 1e-5), ("f16", 1e-3)])
def test_softmax_golden(dev, golden_dir, tag, atol):
    g = load(golden_dir, f"softmax_128x128_{tag}")
    got = gpu_softmax(g["in0"], dev)
    assert torch.allclose(got, g["output"], atol=atol)      # what the reference kernel produced
    assert torch.allclose(got, g["expected"], atol=atol)    # what the reference test asserts against


def test_online_softmax_golden(dev, golden_dir):
    g = load(golden_dir, "online_softmax_128x128_f32")
    got = gpu_softmax(g["in0"], dev)
    assert torch.allclose(got, g["output"], atol=1e-5)


@pytest.mark.parametrize("rows,cols,dtype", [
    (8192, 1024, torch.float32),      # benchmark configuration 1
    (128, 128, torch.float32), (128, 128, torch.float16),
    (4, 65536, torch.float16),        # the reference's wide-row case
    (27, 8192, torch.float32), (127, 513, torch.float32), (127, 513, torch.float16),
    (1, 1, torch.float32), (3, 7, torch.float16), (5, 1000, torch.float32), (2, 40000, torch.float32),
    (9, 131072, torch.float16),       # beyond the register-resident path
    (1000, 8, torch.float32), (300, 2048, torch.float16), (70, 4096, torch.float32),
])
def test_softmax_vs_oracle(dev, rows, cols, dtype):
    x = O.make_softmax_inputs(rows, cols, dtype, seed=rows * 131 + cols)
    got = gpu_softmax(x, dev)
    ref = O.torch_softmax(x)
    tol = REL_F32 if dtype == torch.float32 else REL_F16
    assert O.max_rel_err(got, ref) < tol
    if rows * cols <= 1 << 20:
        assert O.max_rel_err(got, O.c_softmax(x)) < tol
    s = got.float().sum(dim=1)
    assert torch.allclose(s, torch.ones_like(s), atol=1e-4 if dtype == torch.float32 else 2e-2)
    assert (got >= 0).all()


def test_softmax_strided_and_empty(dev):
    x = O.make_softmax_inputs(64, 256).to(dev)
    big = torch.zeros(64, 512, device=dev)
    big[:, :256] = x
    out = torch.full((64, 384), -1.0, device=dev)
    ops.softmax(big[:, :256], out[:, :256])
    assert O.max_rel_err(out[:, :256].cpu(), O.torch_softmax(x.cpu())) < REL_F32
    assert (out[:, 256:] == -1).all()                      # nothing written past the row
    e = torch.empty(0, 16, device=dev)
    ops.softmax(e, torch.empty_like(e))                    # empty input is a no-op
    e = torch.empty(4, 0, device=dev)
    ops.softmax(e, torch.empty_like(e))


def test_softmax_shift_invariance_full_size(dev):
    x = O.make_softmax_inputs().to(dev)
    y1, y2 = torch.empty_like(x), torch.empty_like(x)
    ops.softmax(x, y1)
    ops.softmax(x + 3.0, y2)
    assert (y1 - y2).abs().max().item() < 1e-6
    ops.softmax(x, y2)
    assert torch.equal(y1, y2)                             # deterministic


# ------------------------------------------------------------------ LayerNorm / RMSNorm
def gpu_layer_norm(x, w, b, eps, dev, stats=True):
    xd, wd, bd = x.to(dev), w.to(dev), b.to(dev)
    yd = torch.empty_like(xd)
    mean = torch.empty(x.shape[0], dtype=torch.float32, device=dev) if stats else None
    rstd = torch.empty(x.shape[0], dtype=torch.float32, device=dev) if stats else None
    ops.layer_norm(xd, yd, wd, bd, mean, rstd, eps=eps)
    return yd.cpu(), (mean.cpu() if stats else None), (rstd.cpu() if stats else None)


def test_layer_norm_golden(dev, golden_dir):
    g = load(golden_dir, "layer_norm_27x1024_f32")
    y, mean, rstd = gpu_layer_norm(g["in0"], g["in1"], g["in2"], 1e-5, dev)
    assert torch.allclose(y, g["output"], atol=1e-5)
    assert torch.allclose(y, g["expected"], atol=1e-5)


@pytest.mark.parametrize("rows,cols,dtype", [
    (16384, 4096, torch.float16),     # benchmark configuration 2
    (27, 8192, torch.float32),        # the reference's shape
    (27, 8192, torch.float16), (127, 513, torch.float32), (127, 513, torch.float16), (1, 8, torch.float16),
    (3, 5, torch.float32), (33, 2048, torch.float16), (17, 16384, torch.float32), (5, 65536, torch.float16),
    (9, 100000, torch.float32), (8192, 2048, torch.float16),
])
def test_layer_norm_vs_oracle(dev, rows, cols, dtype):
    x, w, b = O.make_layer_norm_inputs(rows, cols, dtype, seed=rows * 7 + cols)
    y, mean, rstd = gpu_layer_norm(x, w, b, 1e-5, dev)
    ref = O.torch_layer_norm(x, w, b, 1e-5)
    tol = REL_F32 if dtype == torch.float32 else REL_F16
    assert O.max_rel_err(y, ref) < tol
    if dtype == torch.float32 and rows * cols <= 1 << 20:
        assert torch.allclose(y, ref, atol=1e-5 * max(1.0, float(ref.abs().max())))
    if rows * cols <= 1 << 22:
        yc, mc, rc = O.c_layer_norm(x, w, b, 1e-5)
        assert O.max_rel_err(y, yc) < tol
        assert torch.allclose(mean, mc, atol=1e-5)
        assert torch.allclose(rstd, rc, rtol=1e-4)
    xf = x.float()
    assert torch.allclose(mean, xf.mean(dim=1), atol=1e-4)
    assert torch.allclose(rstd, 1.0 / torch.sqrt(xf.var(dim=1, unbiased=False) + 1e-5), rtol=1e-3)


def ulp_distance_f16(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance between two fp16 tensors in units in the last place (ordered-integer view of the bits)."""
    def ordered(t):
        i = t.contiguous().view(torch.int16).to(torch.int32)
        return torch.where(i >= 0, i, -(i & 0x7FFF))
    return (ordered(a) - ordered(b)).abs()


def assert_within_ulps(got, ref, max_ulps, max_mismatch_fraction, tiny):
    """Every element within max_ulps fp16 ulps of ref, or -- for results so close to zero that an ulp
    is smaller than the fp32 round-off of the inputs to the final rounding -- within `tiny` absolutely."""
    d = ulp_distance_f16(got, ref)
    bad = (d > max_ulps) & ((got.float() - ref.float()).abs() > tiny)
    assert int(bad.sum()) == 0, f"{int(bad.sum())} elements beyond {max_ulps} ulp, worst {int(d.max())}"
    assert float((d > 0).float().mean()) < max_mismatch_fraction


@pytest.mark.parametrize("affine_f32", [1, 0])
def test_layer_norm_config2_within_one_ulp_of_the_oracle(dev, affine_f32):
    """Configuration 2 at full size, element by element against the C oracle (fp32 arithmetic from the
    fp16 inputs, one rounding): the kernel that does the affine step in fp32 differs by at most one
    fp16 ulp anywhere (a different summation order can move a value across a rounding boundary), and
    in few places.  The packed-fp16 affine variant rounds (x - mean) * rstd to fp16 before the gain and
    bias are applied: where gain * normalised value and bias nearly cancel, that first rounding is many
    ulps of the small result, so it is held to an absolute bar only (half an fp16 ulp of the largest
    normalised value, 4 * 2^-11 * 1.5)."""
    x, w, b = O.make_layer_norm_inputs()                           # [16384 x 4096] fp16
    hexb200.set_option("norm_affine_f32", affine_f32)
    try:
        y, mean, rstd = gpu_layer_norm(x, w, b, 1e-5, dev)
    finally:
        hexb200.set_option("norm_affine_f32", 1)
    yc, mc, rc = O.c_layer_norm(x, w, b, 1e-5)
    if affine_f32:
        assert_within_ulps(y, yc, 1, 0.01, tiny=5e-7)
    else:
        assert float((y.float() - yc.float()).abs().max()) < 6e-3
    assert torch.allclose(mean, mc, atol=1e-6) and torch.allclose(rstd, rc, rtol=1e-5)


@pytest.mark.parametrize("affine_f32", [1, 0])
def test_rms_norm_decoder_shape_within_one_ulp_of_the_oracle(dev, affine_f32):
    """The decoder's RMSNorm shape [8192 x 2048] fp16 (eight launches per forward pass), same bar."""
    g = torch.Generator().manual_seed(4242)
    x = torch.randn(8192, 2048, generator=g).half()
    gain = (0.5 + torch.rand(2048, generator=g)).half()
    xd, y = x.to(dev), torch.empty(8192, 2048, dtype=torch.float16, device=dev)
    hexb200.set_option("norm_affine_f32", affine_f32)
    try:
        ops.rms_norm(xd, y, gain.to(dev), eps=1e-6)
    finally:
        hexb200.set_option("norm_affine_f32", 1)
    assert_within_ulps(y.cpu(), O.c_rms_norm(x, gain, 1e-6), 1 if affine_f32 else 2, 0.01 if affine_f32 else 0.5, tiny=5e-7)


def test_layer_norm_without_stats_and_reference_dtype_stats(dev):
    x, w, b = O.make_layer_norm_inputs(64, 1024, torch.float16)
    y0, _, _ = gpu_layer_norm(x, w, b, 1e-5, dev, stats=False)
    y1, _, _ = gpu_layer_norm(x, w, b, 1e-5, dev, stats=True)
    assert torch.equal(y0, y1)
    xd, wd, bd = x.to(dev), w.to(dev), b.to(dev)
    m16 = torch.empty(64, dtype=torch.float16, device=dev)   # the reference allocates stats in x's dtype
    r16 = torch.empty(64, dtype=torch.float16, device=dev)
    ops.layer_norm(xd, torch.empty_like(xd), wd, bd, m16, r16)
    assert torch.allclose(m16.float().cpu(), x.float().mean(dim=1), atol=1e-3)


@pytest.mark.parametrize("tag", ["f32", "f16"])
def test_rms_norm_golden(dev, golden_dir, tag):
    g = load(golden_dir, f"rms_norm_127x513_{tag}")
    x, w = g["in0"].to(dev), g["in1"].to(dev)
    y = torch.empty_like(x)
    ops.rms_norm(x, y, w, eps=1e-5)
    assert torch.allclose(y.cpu(), g["output"], atol=1e-2)
    assert torch.allclose(y.cpu(), g["expected"], atol=1e-2)


@pytest.mark.parametrize("rows,cols,dtype", [
    (8192, 2048, torch.float16),      # the decoder's shape
    (127, 513, torch.float32), (127, 513, torch.float16), (4, 8192, torch.float32), (3, 50000, torch.float16),
])
def test_rms_norm_vs_oracle(dev, rows, cols, dtype):
    x, w, _ = O.make_layer_norm_inputs(rows, cols, dtype, seed=rows + cols)
    xd, wd = x.to(dev), w.to(dev)
    y = torch.empty_like(xd)
    ops.rms_norm(xd, y, wd, eps=1e-6)
    tol = REL_F32 if dtype == torch.float32 else REL_F16
    assert O.max_rel_err(y.cpu(), O.torch_rms_norm(x, w, 1e-6)) < tol
    if rows * cols <= 1 << 22:
        assert O.max_rel_err(y.cpu(), O.c_rms_norm(x, w, 1e-6)) < tol


def test_layer_norm_scale_invariance_full_size(dev):
    x, w, b = O.make_layer_norm_inputs()
    xd, wd, bd = x.to(dev), w.to(dev), b.to(dev)
    y1, y2 = torch.empty_like(xd), torch.empty_like(xd)
    ops.layer_norm(xd, y1, wd, bd)
    ops.layer_norm(xd * 2, y2, wd, bd)                     # exact in fp16; eps makes the difference tiny
    assert (y1.float() - y2.float()).abs().max().item() < 2e-2
    ones, zeros = torch.ones_like(wd), torch.zeros_like(bd)
    ops.layer_norm(xd, y1, ones, zeros)
    yf = y1.float()
    assert yf.mean(dim=1).abs().max().item() < 2e-3        # normalised rows: mean 0, variance 1
    assert (yf.var(dim=1, unbiased=False) - 1).abs().max().item() < 5e-3


# ------------------------------------------------------------------ matmul
def gpu_matmul(a, b, dev, out_dtype=torch.float16, residual=None):
    ad, bd = a.to(dev), b.to(dev)
    c = torch.empty(a.shape[0], b.shape[1], dtype=out_dtype, device=dev)
    ops.matmul(ad, bd, c, None if residual is None else residual.to(dev))
    torch.cuda.synchronize()
    assert hexb200.device_status() == 0
    return c.cpu()


def test_matmul_golden(dev, golden_dir):
    g = load(golden_dir, "matmul_256x128x64_f16")
    c = gpu_matmul(g["in0"], g["in1"], dev)
    assert torch.allclose(c, g["output"], atol=2e-1)
    assert torch.allclose(c, g["expected"], atol=2e-1)
    assert O.max_rel_err(c, g["output"]) < 2e-3


@pytest.mark.parametrize("M,N,K", [
    (128, 128, 64), (128, 256, 64), (128, 64, 64), (128, 256, 256), (256, 512, 128),
    (1024, 512, 64),                  # the reference's shape
    (1024, 1024, 1024), (100, 72, 40), (129, 264, 136), (1, 8, 8), (300, 1000, 520), (2048, 6144, 2048),
    (512, 4096, 4096),                # one 8-GPU shard of configuration 3
])
@pytest.mark.parametrize("out_dtype", [torch.float16, torch.float32])
def test_matmul_vs_oracle(dev, M, N, K, out_dtype):
    if out_dtype == torch.float32 and M * N * K > 1 << 28:
        pytest.skip("fp32-output variant is covered at the smaller shapes")
    a, b = O.make_matmul_inputs(M, N, K, seed=M + 3 * N + 7 * K)
    c = gpu_matmul(a, b, dev, out_dtype)
    ref = O.torch_matmul(a, b, out_dtype)
    assert O.max_rel_err(c, ref) < (REL_F16 if out_dtype == torch.float16 else REL_F32)
    if out_dtype == torch.float32:
        assert torch.allclose(c, ref, rtol=1e-2, atol=1e-2)        # the HexKL check: MAX_DIFF 1e-2
    if M * N * K <= 1 << 24:
        assert O.max_rel_err(c, O.c_matmul(a, b, out_dtype)) < (REL_F16 if out_dtype == torch.float16 else REL_F32)


def test_matmul_unaligned_and_residual(dev):
    a, b = O.make_matmul_inputs(37, 29, 13, seed=5)               # breaks the 16-byte rule: CUDA-core path
    c = gpu_matmul(a, b, dev)
    assert O.max_rel_err(c, O.torch_matmul(a, b)) < REL_F16
    a, b = O.make_matmul_inputs(256, 384, 192, seed=6)
    r = (torch.randn(256, 384, generator=torch.Generator().manual_seed(1))).half()
    c = gpu_matmul(a, b, dev, residual=r)
    assert O.max_rel_err(c, O.torch_matmul(a, b, residual=r)) < REL_F16
    assert O.max_rel_err(c, O.c_matmul(a, b, residual=r)) < REL_F16


def test_hexkl_symbol(dev):
    a, b = O.make_matmul_inputs(1024, 512, 64, seed=9)
    ad, bd = a.to(dev), b.to(dev)
    out = torch.zeros(1024, 512, dtype=torch.float32, device=dev)
    ops.hexkl_matmul_f16f16_f32(1024, 512, 64, out, ad, bd)         # rows, cols, inner; out first
    ref = O.c_matmul(a, b, torch.float32)
    diff = (out.cpu() - ref).abs().max().item()
    assert diff < 1e-2                                             # MAX_DIFF of the reference's wrapper check


def test_matmul_full_size_properties(dev):
    a, b = O.make_matmul_inputs()                                  # 4096^3, configuration 3
    ad, bd = a.to(dev), b.to(dev)
    c = torch.empty(4096, 4096, dtype=torch.float16, device=dev)
    ops.matmul(ad, bd, c)
    c2 = torch.empty_like(c)
    ops.matmul(ad, bd, c2)
    assert torch.equal(c, c2)                                      # deterministic
    # linearity in A: (2A) B == 2 (A B) up to the last fp16 bit (power-of-two scaling)
    ops.matmul(ad * 2, bd, c2)
    assert O.max_rel_err(c2.float(), c.float() * 2) < 1e-3
    # the whole 4096 x 4096 output against torch CPU (fp32 arithmetic from the fp16 inputs, one rounding)
    ref = O.torch_matmul(a, b)
    assert O.max_rel_err(c.cpu(), ref) < REL_F16
    # fp32 accumulation of 4096 products in another order: ~1e-4 of round-off on either side, which is
    # below one fp16 ulp wherever |c| >= 1 and is allowed absolutely below that
    assert_within_ulps(c.cpu(), ref, 1, 0.05, tiny=1e-3)
    # checksum: column sums of C == (column sums of A) B
    colsum = c.float().sum(dim=0).cpu()
    ref_sum = (a.float().sum(dim=0, keepdim=True) @ b.float()).squeeze(0)
    assert O.max_rel_err(colsum, ref_sum) < 5e-3
    assert hexb200.device_status() == 0


# ------------------------------------------------------------------ attention
def gpu_attention(q, k, v, scale, causal, dev):
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    o = torch.empty_like(qd)
    ops.attention(qd, kd, vd, o, sm_scale=scale, causal=causal)
    torch.cuda.synchronize()
    assert hexb200.device_status() == 0
    return o.cpu()


def test_flash_attention_golden(dev, golden_dir):
    g = load(golden_dir, "flash_attention_1x1x256x64_f32")
    o = gpu_attention(g["in0"], g["in1"], g["in2"], 0.5, False, dev)
    assert torch.allclose(o, g["output"], rtol=1e-4, atol=1e-5)
    assert torch.allclose(o, g["expected"], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("Z,H,N,D,causal", [
    (1, 1, 128, 128, False), (1, 1, 128, 128, True), (1, 1, 256, 128, True), (1, 2, 512, 128, False),
    (2, 3, 384, 128, True), (1, 1, 1024, 64, False),   # the reference's shape (its fp16 MLIR form)
    (1, 2, 1024, 64, True), (1, 1, 200, 128, True), (1, 1, 77, 64, False), (2, 2, 1000, 128, True),
    (1, 16, 1024, 128, True),                          # one sequence of the decoder
])
def test_attention_f16_vs_oracle(dev, Z, H, N, D, causal):
    q, k, v = O.make_attention_inputs(Z, H, N, D, seed=Z + H + N + D)
    scale = D ** -0.5
    o = gpu_attention(q, k, v, scale, causal, dev)
    ref = O.torch_attention(q, k, v, scale, causal)
    assert O.max_rel_err(o, ref) < REL_F16
    if Z * H * N * N * D <= 1 << 28:
        assert O.max_rel_err(o, O.c_attention(q, k, v, scale, causal)) < REL_F16


def test_attention_reference_scale_and_unfused_check(dev):
    # the fp16 MLIR test: [1,1,1024,64], inputs ~ N(0, 0.5), scale 0.5, checked against an unfused chain
    g = torch.Generator().manual_seed(3)
    q, k, v = ((torch.randn(1, 1, 1024, 64, generator=g) * 0.5).half() for _ in range(3))
    o = gpu_attention(q, k, v, 0.5, False, dev)
    ref = O.c_attention_unfused(q, k, v, 0.5, False)
    assert (o.float() - ref).abs().max().item() < 2e-3            # MAX_DIFF 1e-3 plus fp16 output rounding


@pytest.mark.parametrize("D,causal", [(64, False), (64, True), (32, True), (128, False)])
def test_attention_f32(dev, D, causal):
    q, k, v = O.make_attention_inputs(1, 2, 256, D, torch.float32, seed=D)
    o = gpu_attention(q, k, v, 0.5, causal, dev)
    assert torch.allclose(o, O.torch_attention(q, k, v, 0.5, causal), rtol=1e-4, atol=1e-5)
    assert torch.allclose(o, O.c_attention(q, k, v, 0.5, causal), rtol=1e-4, atol=1e-5)


def test_attention_strided_heads(dev):
    # q|k|v packed per token, heads split by strides (the decoder's layout)
    B, S, H, D = 2, 256, 4, 128
    g = torch.Generator().manual_seed(8)
    qkv = (torch.randn(B, S, 3, H, D, generator=g) * D ** -0.5).half().to(dev)
    q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))      # [B, H, S, D] views
    out = torch.empty(B, S, H, D, dtype=torch.float16, device=dev)
    ops.attention(q, k, v, out.permute(0, 2, 1, 3), causal=True)
    ref = O.torch_attention(q.cpu().contiguous(), k.cpu().contiguous(), v.cpu().contiguous(), D ** -0.5, True)
    assert O.max_rel_err(out.permute(0, 2, 1, 3).cpu(), ref) < REL_F16
    assert hexb200.device_status() == 0


def test_attention_full_size_properties(dev):
    q, k, v = O.make_attention_inputs()                            # [4, 32, 4096, 128], configuration 4
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    o = torch.empty_like(qd)
    ops.attention(qd, kd, vd, o, causal=True)
    o2 = torch.empty_like(qd)
    ops.attention(qd, kd, vd, o2, causal=True)
    assert torch.equal(o, o2)
    # row 0 of a causal head attends to key 0 only
    assert torch.allclose(o[:, :, 0].float(), vd[:, :, 0].float(), atol=1e-3)
    # rows of softmax sum to one: with V = ones the output is ones
    ones = torch.ones_like(vd)
    ops.attention(qd, kd, ones, o2, causal=True)
    assert (o2.float() - 1).abs().max().item() < 2e-3
    # heads spread over every batch index and the head range against the oracle
    for (z, h) in ((0, 0), (0, 13), (1, 17), (1, 30), (2, 5), (2, 22), (3, 9), (3, 31)):
        ref = O.torch_attention(q[z:z + 1, h:h + 1], k[z:z + 1, h:h + 1], v[z:z + 1, h:h + 1], 128 ** -0.5, True)
        assert O.max_rel_err(o[z:z + 1, h:h + 1].cpu(), ref) < REL_F16
    assert hexb200.device_status() == 0


# ------------------------------------------------------------------ SiLU / SwiGLU
@pytest.mark.parametrize("tag", ["f32", "f16"])
def test_silu_golden(dev, golden_dir, tag):
    g = load(golden_dir, f"silu_16384_{tag}")
    x = g["in0"].to(dev)
    y = torch.empty_like(x)
    ops.silu(x, y)
    assert torch.allclose(y.cpu(), g["output"], atol=1e-2)
    assert torch.allclose(y.cpu(), g["expected"], atol=1e-2)


def test_swiglu_and_silu_odd(dev):
    g = torch.Generator().manual_seed(4)
    gu = torch.randn(300, 2 * 264, generator=g).half()
    out = torch.empty(300, 264, dtype=torch.float16, device=dev)
    ops.swiglu(gu.to(dev), out)
    assert O.max_rel_err(out.cpu(), O.c_swiglu(gu)) < REL_F16
    x = torch.randn(1001, generator=g)
    y = torch.empty(1001, device=dev)
    ops.silu(x.to(dev), y)
    assert torch.allclose(y.cpu(), O.c_silu(x), atol=1e-5)


# ------------------------------------------------------------------ decoder block stack
def test_decoder_small_vs_oracle(dev):
    L, d, H, f, B, S = 2, 256, 2, 512, 2, 128
    x, ws = O.make_decoder_inputs(L, d, H, f, B, S)
    wd = [{k: v.to(dev) for k, v in w.items()} for w in ws]
    stack = ops.DecoderStack(wd, H, d // H, f, B, S, 1e-6)
    out = torch.empty(B, S, d, dtype=torch.float16, device=dev)
    stack.forward(x.to(dev), out)
    torch.cuda.synchronize()
    assert hexb200.device_status() == 0
    ref_c = O.c_decoder(x.reshape(-1, d), ws, H, d // H, f, B, S, 1e-6).reshape(B, S, d)
    ref_t = O.torch_decoder(x, ws, H, d // H, f, B, S, 1e-6)
    assert O.max_rel_err(out.cpu(), ref_c) < REL_F16
    assert O.max_rel_err(out.cpu(), ref_t) < REL_F16


def test_decoder_config5_one_sequence(dev):
    # configuration 5 (4 layers, d 2048, 16 x 128 heads, SwiGLU 8192) on one sequence of 1024 tokens:
    # the oracle (torch CPU, fp32 arithmetic, fp16 storage) finishes in seconds at this size.
    x, ws = O.make_decoder_inputs(4, 2048, 16, 8192, 1, 1024)
    wd = [{k: v.to(dev) for k, v in w.items()} for w in ws]
    stack = ops.DecoderStack(wd, 16, 128, 8192, 1, 1024, 1e-6)
    out = torch.empty(1, 1024, 2048, dtype=torch.float16, device=dev)
    stack.forward(x.to(dev), out)
    torch.cuda.synchronize()
    assert hexb200.device_status() == 0
    ref = O.torch_decoder(x, ws, 16, 128, 8192, 1, 1024, 1e-6)
    assert O.max_rel_err(out.cpu(), ref) < REL_F16
    # batch independence: the same sequence twice in a batch of 2 gives the same rows twice
    stack2 = ops.DecoderStack(wd, 16, 128, 8192, 2, 1024, 1e-6)
    x2 = torch.cat([x, x], dim=0).to(dev)
    out2 = torch.empty(2, 1024, 2048, dtype=torch.float16, device=dev)
    stack2.forward(x2, out2)
    assert torch.equal(out2[0], out2[1])
    assert torch.equal(out2[0], out[0])


def test_decoder_config5_batch8_three_sequences(dev):
    """Configuration 5 as benchmarked (batch 8 x 1024 tokens): the first, a middle and the last
    sequence of the output against the torch CPU oracle run on those sequences alone."""
    x, ws = O.make_decoder_inputs(4, 2048, 16, 8192, 8, 1024)
    wd = [{k: v.to(dev) for k, v in w.items()} for w in ws]
    stack = ops.DecoderStack(wd, 16, 128, 8192, 8, 1024, 1e-6)
    out = torch.empty(8, 1024, 2048, dtype=torch.float16, device=dev)
    stack.forward(x.to(dev), out)
    torch.cuda.synchronize()
    assert hexb200.device_status() == 0
    got = out.cpu()
    for b in (0, 3, 7):
        ref = O.torch_decoder(x[b:b + 1].contiguous(), ws, 16, 128, 8192, 1, 1024, 1e-6)
        assert O.max_rel_err(got[b:b + 1], ref) < REL_F16, b


# ------------------------------------------------------------------ bounded waits
def test_bounded_wait_runs_out_and_the_context_stays_usable(dev):
    """A device-side wait that nothing satisfies gives up after its limit: the call returns, the status
    word reports HEXB_ERR_TIMEOUT exactly once, and a tensor-core matmul afterwards is still right."""
    import time
    lib = hexb200.load()
    assert hexb200.device_status() == 0
    assert lib.hexb_selftest_bounded_wait(0, None) == -1            # limit out of range: nothing is launched
    t = time.perf_counter()
    assert lib.hexb_selftest_bounded_wait(1000, torch.cuda.current_stream().cuda_stream) == 0   # 1 ms
    assert lib.hexb_status_string(hexb200.device_status()).decode() == "HEXB_ERR_TIMEOUT"
    assert time.perf_counter() - t < 1.0                            # far below the kernels' 2 s default
    assert hexb200.device_status() == 0                             # reported once, then clear
    a, b = O.make_matmul_inputs(512, 512, 256, seed=5)
    c = torch.empty(512, 512, dtype=torch.float16, device=dev)
    ops.matmul(a.to(dev), b.to(dev), c)
    assert O.max_rel_err(c.cpu(), O.torch_matmul(a, b)) < REL_F16
    assert hexb200.device_status() == 0


# ------------------------------------------------------------------ host-buffer entry points and errors
def test_host_entry_points(dev):
    x, w, b = O.make_layer_norm_inputs(2048, 4096)
    y = torch.empty_like(x)
    mean = torch.empty(2048)
    rstd = torch.empty(2048)
    ops.layer_norm(x.pin_memory(), y, w, b, mean, rstd)            # CPU tensors: staged inside the call
    assert O.max_rel_err(y, O.torch_layer_norm(x, w, b, 1e-5)) < REL_F16
    assert torch.allclose(mean, x.float().mean(dim=1), atol=1e-4)
    xs = O.make_softmax_inputs(3000, 1024)
    ys = torch.empty_like(xs)
    ops.softmax(xs, ys)
    assert O.max_rel_err(ys, O.torch_softmax(xs)) < REL_F32
    a, bm = O.make_matmul_inputs(256, 128, 64)
    c = torch.empty(256, 128, dtype=torch.float16)
    ops.matmul(a, bm, c)
    assert O.max_rel_err(c, O.torch_matmul(a, bm)) < REL_F16
    q, k, v = O.make_attention_inputs(2, 2, 256, 128)
    o = torch.empty_like(q)
    ops.attention(q, k, v, o, causal=True)
    assert O.max_rel_err(o, O.torch_attention(q, k, v, 128 ** -0.5, True)) < REL_F16
    xr = torch.rand(127, 513)
    yr = torch.empty_like(xr)
    ops.rms_norm(xr, yr, torch.rand(513).fill_(1.0), eps=1e-5)
    assert torch.allclose(yr, O.torch_rms_norm(xr, torch.ones(513), 1e-5), atol=1e-5)


@pytest.mark.parametrize("chunks,taper", [(1, 0), (3, 0), (8, 0), (8, 1), (64, 1)])
def test_host_entry_points_in_pieces(dev, chunks, taper):
    """The `_host` entry points cut their operands into pieces that flow through upload, kernel and download
    streams.  Rows, row blocks of A and (batch, head) pairs are independent, so whatever the number and the
    sizes of the pieces (equal or tapered, ragged last piece, pinned or pageable memory) the result is the one
    the device entry point gives for the whole tensor -- for the row operators to one fp16 ulp rather than bit
    for bit, because a small piece may run the register form of the kernel where the whole matrix runs the
    ring form, and the two sum in different orders."""
    hexb200.set_option("host_chunks", chunks)
    hexb200.set_option("host_taper", taper)
    try:
        g = torch.Generator().manual_seed(40 + chunks)
        # LayerNorm: 4099 rows (ragged pieces), 8 MiB
        x = torch.randn(4099, 1024, generator=g).half()
        w, b = torch.randn(1024, generator=g).half(), torch.randn(1024, generator=g).half()
        y_dev = torch.empty_like(x, device=dev)
        ops.layer_norm(x.to(dev), y_dev, w.to(dev), b.to(dev))
        for xin in (x.pin_memory(), x):
            y, mean, rstd = torch.empty_like(x), torch.empty(4099), torch.empty(4099)
            ops.layer_norm(xin, y, w, b, mean, rstd)
            assert_within_ulps(y, y_dev.cpu(), 1, 0.1, 1e-3)
            assert_within_ulps(y, O.torch_layer_norm(x, w, b, 1e-5), 1, 0.1, 1e-3)
            assert torch.allclose(mean, x.float().mean(dim=1), atol=1e-4)
        # matmul: 2100 rows of A (pieces are multiples of 256 rows), B whole
        a = (torch.randn(2100, 1024, generator=g) * 0.5).half()
        bm = (torch.randn(1024, 520, generator=g) * 0.05).half()
        c_dev = torch.empty(2100, 520, dtype=torch.float16, device=dev)
        ops.matmul(a.to(dev), bm.to(dev), c_dev)
        c = torch.empty(2100, 520, dtype=torch.float16)
        ops.matmul(a.pin_memory(), bm.pin_memory(), c)
        assert O.max_rel_err(c, c_dev.cpu()) < 1e-3
        assert O.max_rel_err(c, O.torch_matmul(a, bm)) < REL_F16
        # attention: 15 (batch, head) pairs of 512 KiB each
        q, k, v = ((torch.randn(3, 5, 2048, 128, generator=g) * 0.3).half() for _ in range(3))
        o_dev = torch.empty_like(q, device=dev)
        ops.attention(q.to(dev), k.to(dev), v.to(dev), o_dev, causal=True)
        o = torch.empty_like(q)
        ops.attention(q.pin_memory(), k.pin_memory(), v.pin_memory(), o, causal=True)
        assert torch.equal(o, o_dev.cpu())
        assert hexb200.device_status() == 0
    finally:
        hexb200.set_option("host_chunks", 8)
        hexb200.set_option("host_taper", -1)


def test_error_codes(dev):
    lib = hexb200.load()
    x = torch.zeros(4, 8, device=dev)
    assert lib.hexb_softmax_f32(None, x.data_ptr(), 4, 8, 8, 8, None) == -1          # HEXB_ERR_BAD_ARG
    assert lib.hexb_softmax_f32(x.data_ptr(), x.data_ptr(), -1, 8, 8, 8, None) == -1
    assert lib.hexb_softmax_f32(x.data_ptr(), x.data_ptr(), 4, 8, 4, 8, None) == -1   # stride < cols
    assert lib.hexb_matmul_f16(x.data_ptr(), x.data_ptr(), x.data_ptr(), None, 4, 4, 4, 4, 4, 4, 7, None) == -2
    assert lib.hexb_set_option(b"no_such_option", 1) == -1
    with pytest.raises(hexb200.HexbError) as e:
        hexb200._lib.check(lib.hexb_softmax_f32(None, x.data_ptr(), 4, 8, 8, 8, None), "softmax")
    assert e.value.status_name == "HEXB_ERR_BAD_ARG"
    with pytest.raises(ValueError):
        ops.softmax(x, torch.zeros(4, 16, device=dev))


# ------------------------------------------------------------------ gate/up projection with fused SwiGLU
@pytest.mark.parametrize("M,F,K", [(128, 128, 64), (256, 384, 192), (300, 264, 136), (1000, 72, 40), (2048, 8192, 2048)])
def test_matmul_swiglu_vs_oracle(dev, M, F, K):
    g = torch.Generator().manual_seed(M + F + K)
    a = (torch.randn(M, K, generator=g) * 0.5).half()
    b = (torch.randn(K, 2 * F, generator=g) * K ** -0.5).half()
    out = torch.empty(M, F, dtype=torch.float16, device=dev)
    ops.matmul_swiglu(a.to(dev), b.to(dev), out)
    torch.cuda.synchronize()
    assert hexb200.device_status() == 0
    rows = torch.arange(M) if M * F * K <= 1 << 26 else torch.tensor([0, 1, 127, 128, M // 2, M - 1])
    gu = a[rows].float() @ b.float()
    ref = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    assert O.max_rel_err(out.cpu()[rows], ref) < REL_F16
    if M * F * K <= 1 << 24:
        unfused = O.c_swiglu(O.c_matmul(a, b))                       # gate|up rounded to fp16 in between
        assert O.max_rel_err(out.cpu(), unfused) < REL_F16


def test_decoder_fused_and_unfused_gating_agree(dev):
    L, d, H, f, B, S = 2, 256, 2, 512, 2, 128
    x, ws = O.make_decoder_inputs(L, d, H, f, B, S, seed=77)
    wd = [{k: v.to(dev) for k, v in w.items()} for w in ws]
    stack = ops.DecoderStack(wd, H, d // H, f, B, S, 1e-6)
    outs = []
    try:
        for fused in (1, 0):
            hexb200.set_option("decoder_fused_swiglu", fused)
            out = torch.empty(B, S, d, dtype=torch.float16, device=dev)
            stack.forward(x.to(dev), out)
            outs.append(out.cpu())
    finally:
        hexb200.set_option("decoder_fused_swiglu", 1)
    assert O.max_rel_err(outs[0], outs[1]) < 5e-3
    ref = O.torch_decoder(x, ws, H, d // H, f, B, S, 1e-6)
    assert O.max_rel_err(outs[0], ref) < REL_F16 and O.max_rel_err(outs[1], ref) < REL_F16


# ------------------------------------------------------------------ matmul with the weight stored transposed
@pytest.mark.parametrize("M,N,K", [(1024, 256, 512),          # the reference's transposed case
                                   (128, 128, 64), (256, 512, 128), (100, 72, 40), (129, 264, 136),
                                   (37, 29, 13), (4096, 4096, 1024), (2560, 2560, 256)])
@pytest.mark.parametrize("out_dtype", [torch.float16, torch.float32])
def test_matmul_nt_vs_oracle(dev, M, N, K, out_dtype):
    g = torch.Generator().manual_seed(M * 3 + N * 5 + K)
    a = torch.randn(M, K, generator=g).half()
    w = (torch.randn(N, K, generator=g) * K ** -0.5).half()           # weight [N, K]; the product uses w.T
    c = torch.empty(M, N, dtype=out_dtype, device=dev)
    ops.matmul_nt(a.to(dev), w.to(dev), c)
    torch.cuda.synchronize()
    assert hexb200.device_status() == 0
    ref = torch.matmul(a.float(), w.float().T)
    assert O.max_rel_err(c.cpu(), ref) < (REL_F16 if out_dtype == torch.float16 else REL_F32)
    if out_dtype == torch.float16:
        assert torch.allclose(c.cpu().float(), ref, rtol=1e-2, atol=1e-2)   # the reference test's tolerance
    # same numbers as the non-transposed entry point on a materialised w.T
    c2 = torch.empty(M, N, dtype=out_dtype, device=dev)
    ops.matmul(a.to(dev), w.T.contiguous().to(dev), c2)
    assert O.max_rel_err(c.cpu(), c2.cpu()) < 1e-3


# ------------------------------------------------------------------ generalised attention: mask, fp32 out, N_Q != N_KV
def _sdpa_ref(q, k, v, mask, scale, causal=False):
    """fp32 torch reference on the (already rounded) inputs."""
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * scale
    if mask is not None:
        s = s + mask.float()
    if causal:
        nq, nkv = s.shape[-2:]
        s = s.masked_fill(torch.ones(nq, nkv, dtype=torch.bool).triu(1), float("-inf"))
    return torch.matmul(torch.softmax(s, dim=-1), v.float())


def test_attention_f16_in_f32_out_reference_case(dev):
    """The fp16-in / fp32-out attention of the reference's MLIR test: 1x1x1024x64, scale 0.5, inputs
    N(0, 0.5) rounded to 4 decimals, |diff| <= 1e-3 against its unfused CPU check."""
    g = torch.Generator().manual_seed(11)
    q, k, v = ((torch.randn(1, 1, 1024, 64, generator=g) * 0.5 * 1e4).round() / 1e4 for _ in range(3))
    q, k, v = q.half(), k.half(), v.half()
    out = torch.empty(1, 1, 1024, 64, dtype=torch.float32, device=dev)
    ops.attention_ex(q.to(dev), k.to(dev), v.to(dev), out, sm_scale=0.5)
    ref = O.c_attention_unfused(q, k, v, 0.5)
    assert (out.cpu() - ref).abs().max() <= 1e-3
    assert hexb200.device_status() == 0


@pytest.mark.parametrize("Z,H,NQ,NKV,D", [(2, 3, 256, 256, 64), (1, 2, 384, 640, 128), (2, 2, 100, 77, 64),
                                          (1, 1, 130, 200, 128), (1, 2, 64, 1024, 64)])
@pytest.mark.parametrize("mask_dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("out_dtype", [torch.float16, torch.float32])
def test_attention_masked_f16(dev, Z, H, NQ, NKV, D, mask_dtype, out_dtype):
    g = torch.Generator().manual_seed(Z + 3 * H + NQ + NKV)
    q = torch.randn(Z, H, NQ, D, generator=g).half()
    k, v = (torch.randn(Z, H, NKV, D, generator=g).half() for _ in range(2))
    mask = torch.randn(Z, H, NQ, NKV, generator=g).to(mask_dtype)
    out = torch.empty(Z, H, NQ, D, dtype=out_dtype, device=dev)
    ops.attention_ex(q.to(dev), k.to(dev), v.to(dev), out, mask=mask.to(dev))
    ref = _sdpa_ref(q, k, v, mask, 1.0 / math.sqrt(D))
    assert O.max_rel_err(out.cpu(), ref) < REL_F16
    assert hexb200.device_status() == 0


@pytest.mark.parametrize("mask_dtype", [torch.float16, torch.float32])
def test_attention_mask_shared_by_the_batches_of_a_head(dev, mask_dtype):
    """A mask of shape [1, H, N_Q, N_KV] broadcast over the batch: the kernel then orders its CTAs head-major
    (the batches of a head next to each other, so that they find the head's mask tiles in L2); the (batch,
    head) a CTA works on must still be the right one."""
    g = torch.Generator().manual_seed(91)
    Z, H, NQ, NKV, D = 3, 5, 256, 320, 128
    q = torch.randn(Z, H, NQ, D, generator=g).half()
    k, v = (torch.randn(Z, H, NKV, D, generator=g).half() for _ in range(2))
    mask = torch.randn(1, H, NQ, NKV, generator=g).to(mask_dtype)
    out = torch.empty(Z, H, NQ, D, dtype=torch.float16, device=dev)
    ops.attention_ex(q.to(dev), k.to(dev), v.to(dev), out, mask=mask.to(dev).expand(Z, H, NQ, NKV))
    ref = _sdpa_ref(q, k, v, mask.expand(Z, H, NQ, NKV), 1.0 / math.sqrt(D))
    assert O.max_rel_err(out.cpu(), ref) < REL_F16
    assert hexb200.device_status() == 0


def test_attention_masked_matches_oracle_rank3(dev):
    """tm_tensor.attention form: rank-3 operands, mask [batch, seq_q, seq_kv], checked against the C oracle."""
    g = torch.Generator().manual_seed(77)
    B, SQ, SKV, D = 4, 192, 320, 64
    q = torch.randn(B, SQ, D, generator=g).half()
    k, v = (torch.randn(B, SKV, D, generator=g).half() for _ in range(2))
    mask = torch.randn(B, SQ, SKV, generator=g).half()
    out = torch.empty(B, SQ, D, dtype=torch.float16, device=dev)
    ops.sdpa_masked(q.to(dev), k.to(dev), v.to(dev), mask.to(dev), out)
    ref = O.c_sdpa_masked(q, k, v, mask)
    assert O.max_rel_err(out.cpu(), ref) < REL_F16
    # the same in fp32 end to end (CUDA-core path)
    out32 = torch.empty(B, SQ, D, dtype=torch.float32, device=dev)
    ops.sdpa_masked(q.float().to(dev), k.float().to(dev), v.float().to(dev), mask.float().to(dev), out32)
    assert O.max_rel_err(out32.cpu(), ref) < REL_F32


@pytest.mark.parametrize("D", [64, 128])
def test_attention_additive_causal_mask_equals_causal_flag(dev, D):
    """-inf above the diagonal as an additive mask gives the causal kernel's result, including key
    blocks that are masked out entirely."""
    g = torch.Generator().manual_seed(3)
    Z, H, N = 1, 2, 512
    q, k, v = (torch.randn(Z, H, N, D, generator=g).half().to(dev) for _ in range(3))
    mask = torch.full((N, N), float("-inf")).triu(1).half().to(dev)          # broadcast over Z and H
    a = torch.empty_like(q)
    b = torch.empty_like(q)
    ops.attention_ex(q, k, v, a, mask=mask)
    ops.attention(q, k, v, b, causal=True)
    assert O.max_rel_err(a.cpu(), b.cpu()) < 2e-3
    c = torch.empty_like(q)
    ops.attention_ex(q, k, v, c, causal=True)                                # flag through the general entry
    assert torch.equal(c, b)
    # a leading block fully masked for every row: keys [0, 128) get -inf
    mask2 = torch.zeros(N, N)
    mask2[:, :128] = float("-inf")
    ops.attention_ex(q, k, v, a, mask=mask2.to(dev))
    ref = _sdpa_ref(q.cpu(), k.cpu(), v.cpu(), mask2, 1.0 / math.sqrt(D))
    assert O.max_rel_err(a.cpu(), ref) < REL_F16
    assert hexb200.device_status() == 0


@pytest.mark.parametrize("D,force_simt", [(64, 0), (128, 0), (64, 1), (48, 0)])
def test_attention_fully_masked_row_is_nan_like_the_reference(dev, D, force_simt):
    """A row whose keys are all masked to -inf is NaN (exp(-inf - -inf)), on the tensor-core kernel and on
    the CUDA-core kernel alike (D = 48 and the forced case take the latter); a row whose FIRST key blocks
    are masked out but later ones are not is finite and right; every other row matches the oracle."""
    g = torch.Generator().manual_seed(4)
    q, k, v = (torch.randn(1, 1, 192, D, generator=g).half() for _ in range(3))
    mask = torch.zeros(192, 192)
    mask[5, :] = float("-inf")
    mask[9, :130] = float("-inf")                # two whole 64-key blocks and a bit: weights 0 there, not NaN
    out = torch.empty(1, 1, 192, D, dtype=torch.float32, device=dev)
    hexb200.set_option("attn_force_simt", force_simt)
    try:
        ops.attention_ex(q.to(dev), k.to(dev), v.to(dev), out, mask=mask.to(dev))
    finally:
        hexb200.set_option("attn_force_simt", 0)
    o = out.cpu()[0, 0]
    assert torch.isnan(o[5]).all()
    keep = torch.ones(192, dtype=torch.bool)
    keep[5] = False
    assert torch.isfinite(o[keep]).all()
    ref = _sdpa_ref(q, k, v, mask.view(1, 1, 192, 192), 1.0 / math.sqrt(D))[0, 0]
    assert O.max_rel_err(o[keep], ref[keep]) < REL_F16


def test_attention_masked_odd_strides_and_broadcast(dev):
    """A mask row stride that is not a multiple of 16 bytes (scalar loads) and a [1, 1, 1, N_KV] key bias."""
    g = torch.Generator().manual_seed(9)
    Z, H, NQ, NKV, D = 1, 2, 128, 203, 64
    q = torch.randn(Z, H, NQ, D, generator=g).half()
    k, v = (torch.randn(Z, H, NKV, D, generator=g).half() for _ in range(2))
    mask = torch.randn(Z, H, NQ, NKV, generator=g)
    out = torch.empty(Z, H, NQ, D, dtype=torch.float16, device=dev)
    ops.attention_ex(q.to(dev), k.to(dev), v.to(dev), out, mask=mask.to(dev))
    assert O.max_rel_err(out.cpu(), _sdpa_ref(q, k, v, mask, 1.0 / math.sqrt(D))) < REL_F16
    bias = torch.randn(NKV, generator=g)
    ops.attention_ex(q.to(dev), k.to(dev), v.to(dev), out, mask=bias.to(dev))
    assert O.max_rel_err(out.cpu(), _sdpa_ref(q, k, v, bias.view(1, 1, 1, NKV), 1.0 / math.sqrt(D))) < REL_F16
    assert hexb200.device_status() == 0


def test_attention_masked_f32_and_odd_head_dim(dev):
    g = torch.Generator().manual_seed(10)
    Z, H, NQ, NKV, D = 2, 2, 75, 131, 40
    q = torch.randn(Z, H, NQ, D, generator=g)
    k, v = (torch.randn(Z, H, NKV, D, generator=g) for _ in range(2))
    mask = torch.randn(Z, H, NQ, NKV, generator=g)
    out = torch.empty(Z, H, NQ, D, dtype=torch.float32, device=dev)
    ops.attention_ex(q.to(dev), k.to(dev), v.to(dev), out, mask=mask.to(dev), causal=True)
    assert O.max_rel_err(out.cpu(), _sdpa_ref(q, k, v, mask, 1.0 / math.sqrt(D), causal=True)) < REL_F32
    # fp16 tensors of the same odd shape take the CUDA-core path too, with an fp32 result
    ops.attention_ex(q.half().to(dev), k.half().to(dev), v.half().to(dev), out, mask=mask.half().to(dev))
    assert O.max_rel_err(out.cpu(), _sdpa_ref(q.half(), k.half(), v.half(), mask.half(), 1.0 / math.sqrt(D))) < REL_F16


@pytest.mark.parametrize("which", [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11])
@pytest.mark.parametrize("causal", [False, True])
def test_attention_selectable_kernels_agree_with_default(dev, which, causal):
    """Every tensor-core kernel stays selectable -- 128-key single-buffer (1), 64-key two-buffer (2), two
    query tiles per CTA with one (3) or two (4) softmax threads per row, 128-key two-buffer (5), 128-key two-buffer with two (6) or four (7) softmax
    threads per row, two warpgroups taking turns (8), 64-key two-buffer with two threads per row (9) or with P handed over through shared memory (10) or with three K stages (11) -- and must give the result of the kernel the library picks by itself, to rounding, on
    full, ragged and odd-tile-count shapes."""
    for Z, H, N, D in [(1, 2, 512, 128), (2, 1, 300, 64), (1, 1, 640, 128)]:
        g = torch.Generator().manual_seed(N + D + which)
        q, k, v = (torch.randn(Z, H, N, D, generator=g).half().to(dev) for _ in range(3))
        a, b = torch.empty_like(q), torch.empty_like(q)
        ops.attention(q, k, v, a, causal=causal)
        hexb200.set_option("attn_kernel", which)
        try:
            ops.attention(q, k, v, b, causal=causal)
        finally:
            hexb200.set_option("attn_kernel", 0)
        assert hexb200.device_status() == 0
        assert O.max_rel_err(b.cpu(), a.cpu()) < 2e-3


@pytest.mark.parametrize("Z,H,N,D,causal", [
    (2, 3, 1024, 128, True), (2, 3, 1024, 128, False), (1, 4, 1000, 64, True), (1, 2, 129, 128, True),
    (3, 2, 384, 64, False), (1, 1, 2048, 128, True), (1, 2, 100, 128, False), (1, 1, 257, 64, True)])
@pytest.mark.parametrize("which", [3, 4, 6, 7, 8, 9, 10, 11])
def test_attention_persistent_kernels_vs_oracle(dev, Z, H, N, D, causal, which):
    """The kernels that exchange values between softmax warps or walk several tiles (forced: two query
    tiles per CTA = 3, 4, several softmax threads per row = 4, 6, 7, 9, alternating warpgroups = 8) against the oracle: even and odd tile counts, ragged lengths, a tile that lies wholly past the last
    row, fp16 and fp32 output, and the decoder's strided [tokens, 3 * d_model] layout."""
    g = torch.Generator().manual_seed(Z * 1000 + N + D)
    qkv = (torch.randn(Z, N, 3, H, D, generator=g) * D ** -0.25).half()
    q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))          # [Z, H, N, D] views of one buffer
    ref = O.torch_attention(q.contiguous(), k.contiguous(), v.contiguous(), D ** -0.5, causal)
    qd = qkv.to(dev)
    qv, kv_, vv = (qd[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    out16 = torch.empty(Z, N, H, D, dtype=torch.float16, device=dev).permute(0, 2, 1, 3)   # heads merged by strides
    out32 = torch.empty(Z, H, N, D, dtype=torch.float32, device=dev)
    hexb200.set_option("attn_kernel", which)
    try:
        ops.attention(qv, kv_, vv, out16, causal=causal)
        ops.attention_ex(qv, kv_, vv, out32, causal=causal)
    finally:
        hexb200.set_option("attn_kernel", 0)
    assert hexb200.device_status() == 0
    assert O.max_rel_err(out16.cpu(), ref) < REL_F16
    assert O.max_rel_err(out32.cpu(), ref) < REL_F16
    assert O.max_rel_err(out32.cpu(), out16.float().cpu()) < 2e-3


@pytest.mark.parametrize("tiles_per_cta", [1, 2])
@pytest.mark.parametrize("Z,H,N,D", [(2, 3, 1024, 128), (1, 2, 512, 64), (1, 1, 2048, 128), (1, 5, 300, 128)])
def test_attention_causal_tile_pairing(dev, Z, H, N, D, tiles_per_cta):
    """Causal calls walk one query tile per CTA or a long and a short one; the library pairs them only when the
    pairs cover the SMs, so both forms are forced here on shapes of either kind (an odd tile count falls
    back to one tile per CTA by itself) and held to the oracle."""
    q, k, v = O.make_attention_inputs(Z, H, N, D)
    ref = O.torch_attention(q, k, v, D ** -0.5, True)
    out = torch.empty_like(q, device=dev)
    hexb200.set_option("attn_tiles_per_cta", tiles_per_cta)
    try:
        ops.attention(q.to(dev), k.to(dev), v.to(dev), out, causal=True)
    finally:
        hexb200.set_option("attn_tiles_per_cta", 0)
    assert hexb200.device_status() == 0
    assert O.max_rel_err(out.cpu(), ref) < REL_F16


@pytest.mark.parametrize("Z,H,NQ,NKV,D,causal", [
    (1, 1, 1024, 1024, 64, False),        # the reference test's shape (scale 0.5 below)
    (2, 3, 512, 512, 128, True), (1, 2, 300, 300, 64, True), (2, 2, 256, 640, 128, False), (1, 4, 129, 77, 64, False),
    (1, 2, 2048, 2048, 128, True)])
def test_attention_f32_on_tensor_cores(dev, Z, H, NQ, NKV, D, causal):
    """fp32 tensors through the kind::tf32 kernel (forced; by default only problems of 2^30 multiply-adds and
    more take it): the tensor cores read the operands as tf32, so the bar is the benchmark's 1e-3 relative for
    fp32 kernels (met at unit logit spread), not the exact kernel's round-off; at the reference test's own
    scale 0.5 on N(0, 1) inputs (logit spread 4) the tf32 scores cost up to 3e-3.  The default path at the
    reference's test shape stays the exact kernel."""
    g = torch.Generator().manual_seed(NQ + NKV + D)
    q = torch.randn(Z, H, NQ, D, generator=g)
    k, v = (torch.randn(Z, H, NKV, D, generator=g) for _ in range(2))
    scale = 0.5 if (NQ, D) == (1024, 64) else D ** -0.5
    ref = _sdpa_ref(q, k, v, None, scale, causal=causal and NQ == NKV)
    out = torch.empty(Z, H, NQ, D, device=dev)
    hexb200.set_option("attn_f32_tensor", 2)
    try:
        ops.attention_ex(q.to(dev), k.to(dev), v.to(dev), out, sm_scale=scale, causal=causal and NQ == NKV)
    finally:
        hexb200.set_option("attn_f32_tensor", 0)
    assert hexb200.device_status() == 0
    err_tc = O.max_rel_err(out.cpu(), ref)
    assert err_tc < (3e-3 if scale == 0.5 else REL_F32), err_tc
    exact = torch.empty_like(out)
    hexb200.set_option("attn_f32_tensor", 1)
    try:
        ops.attention_ex(q.to(dev), k.to(dev), v.to(dev), exact, sm_scale=scale, causal=causal and NQ == NKV)
    finally:
        hexb200.set_option("attn_f32_tensor", 0)
    err_exact = O.max_rel_err(exact.cpu(), ref)
    assert err_exact < 2e-5 and err_exact < err_tc          # the CUDA-core kernel is the exact one
    if (NQ, D) == (1024, 64):                                # what the library picks by itself at the reference's shape
        auto = torch.empty_like(out)
        ops.attention_ex(q.to(dev), k.to(dev), v.to(dev), auto, sm_scale=scale)
        assert torch.equal(auto, exact)


def test_entry_points_are_thread_safe_and_stream_ordered(dev):
    """Two host threads drive the library on their own streams at the same time (ctypes releases the GIL
    for the duration of a call); every result must equal the single-threaded one."""
    import threading

    g = torch.Generator().manual_seed(21)
    a = torch.randn(512, 256, generator=g).half().to(dev)
    b = torch.randn(256, 384, generator=g).half().to(dev)
    x = torch.randn(1024, 1024, generator=g).to(dev)
    ref_c = torch.empty(512, 384, dtype=torch.float16, device=dev)
    ref_y = torch.empty_like(x)
    ops.matmul(a, b, ref_c)
    ops.softmax(x, ref_y)
    torch.cuda.synchronize()
    errors = []

    def worker(seed):
        try:
            s = torch.cuda.Stream(device=dev)
            with torch.cuda.stream(s):
                c = torch.empty_like(ref_c)
                y = torch.empty_like(ref_y)
                for _ in range(40):
                    ops.matmul(a, b, c)
                    ops.softmax(x, y)
                s.synchronize()
                if not (torch.equal(c, ref_c) and torch.equal(y, ref_y)):
                    errors.append(f"thread {seed}: result differs")
        except Exception as e:  # noqa: BLE001
            errors.append(repr(e))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(3)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert hexb200.device_status() == 0
