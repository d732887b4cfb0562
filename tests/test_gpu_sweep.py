"""GPU: seeded random sweeps over shapes, leading dimensions and options of every kernel family, against
fp32 torch on the same (rounded) inputs.  The fixed-shape parity tests pin the reference's own cases;
these look for the shape nobody thought of (ragged tiles, padded leading dimensions, tiny and odd sizes,
every epilogue combination)."""
import math
import random

import pytest
import torch

import hexb200
from hexb200 import ops
from oracle import oracle as O

pytestmark = pytest.mark.gpu
dev = torch.device("cuda:0")


def _randn(g, *shape, scale=1.0):
    return torch.randn(*shape, generator=g) * scale


@pytest.mark.parametrize("seed", range(24))
def test_linear_random_shapes(seed):
    rnd = random.Random(seed)
    g = torch.Generator().manual_seed(seed)
    big = seed % 4 == 0
    M = rnd.choice([1, 7, 128, 129, 255, 256, 300]) if not big else rnd.choice([1024, 2304, 4096])
    N = rnd.choice([1, 8, 24, 64, 72, 200, 256, 520]) if not big else rnd.choice([768, 2048, 2304 + 8])
    K = rnd.choice([8, 16, 40, 64, 136, 512]) if not big else rnd.choice([256, 768, 1024])
    transposed = rnd.random() < 0.5
    out_dtype = rnd.choice([torch.float16, torch.float32])
    pad_a, pad_w, pad_c = (rnd.choice([0, 8, 16]) for _ in range(3))
    use_bias, use_res, act = rnd.random() < 0.5, rnd.random() < 0.5, rnd.choice(["none", "gelu_tanh"])
    a_full = _randn(g, M, K + pad_a).half().to(dev)
    a = a_full[:, :K]
    w_ref = _randn(g, K, N, scale=K ** -0.5).half()
    if transposed:
        w_full = torch.zeros(N, K + pad_w, dtype=torch.float16)
        w_full[:, :K] = w_ref.T
        w = w_full.to(dev)[:, :K]
    else:
        w_full = torch.zeros(K, N + pad_w, dtype=torch.float16)
        w_full[:, :N] = w_ref
        w = w_full.to(dev)[:, :N]
    c_full = torch.full((M, N + pad_c), float("nan"), dtype=out_dtype, device=dev)
    c = c_full[:, :N]
    bias = _randn(g, N).half() if use_bias else None
    res_full = _randn(g, M, N + pad_c).half().to(dev) if use_res else None
    res = res_full[:, :N] if use_res else None
    ops.linear(a, w, c, bias=None if bias is None else bias.to(dev), residual=res, act=act, w_transposed=transposed)
    ref = a.cpu().float() @ w_ref.float()
    if bias is not None:
        ref = ref + bias.float()
    if act == "gelu_tanh":
        ref = 0.5 * ref * (1.0 + torch.tanh(0.797885 * ref + 0.035677 * ref ** 3))
    if use_res:
        ref = ref + res.cpu().float()
    assert hexb200.device_status() == 0
    tol = 2e-2 if out_dtype == torch.float16 else 2e-3
    assert O.max_rel_err(c.cpu(), ref) < tol, (M, N, K, transposed, out_dtype, pad_a, pad_w, pad_c, use_bias, use_res, act)
    if pad_c:
        assert torch.isnan(c_full[:, N:].float()).all()      # nothing written past column N


@pytest.mark.parametrize("seed", range(20))
def test_attention_random_shapes(seed):
    rnd = random.Random(1000 + seed)
    g = torch.Generator().manual_seed(1000 + seed)
    Z, H = rnd.choice([1, 2]), rnd.choice([1, 3])
    D = rnd.choice([64, 128, 128, 64, 32, 80])
    NQ = rnd.choice([1, 17, 128, 130, 256, 333, 512])
    NKV = NQ if rnd.random() < 0.5 else rnd.choice([1, 64, 65, 200, 384, 700])
    causal = rnd.random() < 0.5
    mask_kind = rnd.choice(["none", "none", "f16", "f32", "bcast"])
    out_dtype = rnd.choice([torch.float16, torch.float32])
    q = _randn(g, Z, H, NQ, D).half()
    k, v = _randn(g, Z, H, NKV, D).half(), _randn(g, Z, H, NKV, D).half()
    mask = None
    if mask_kind == "f16":
        mask = _randn(g, Z, H, NQ, NKV).half()
    elif mask_kind == "f32":
        mask = _randn(g, Z, H, NQ, NKV)
    elif mask_kind == "bcast":
        mask = _randn(g, NQ, NKV).half()
    out = torch.empty(Z, H, NQ, D, dtype=out_dtype, device=dev)
    ops.attention_ex(q.to(dev), k.to(dev), v.to(dev), out, mask=None if mask is None else mask.to(dev), causal=causal)
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) / math.sqrt(D)
    if mask is not None:
        s = s + mask.float()
    if causal:
        s = s.masked_fill(torch.ones(NQ, NKV, dtype=torch.bool).triu(1), float("-inf"))
    ref = torch.matmul(torch.softmax(s, dim=-1), v.float())
    assert hexb200.device_status() == 0
    assert O.max_rel_err(out.cpu(), ref) < 2e-2, (Z, H, NQ, NKV, D, causal, mask_kind, out_dtype)


@pytest.mark.parametrize("seed", range(16))
def test_row_kernels_random_shapes(seed):
    rnd = random.Random(2000 + seed)
    g = torch.Generator().manual_seed(2000 + seed)
    rows = rnd.choice([1, 3, 27, 128, 1000, 4097])
    cols = rnd.choice([1, 5, 64, 513, 768, 1000, 1024, 4096, 8192, 10000])
    dtype = rnd.choice([torch.float16, torch.float32])
    pad = rnd.choice([0, 8])
    x_full = _randn(g, rows, cols + pad).to(dtype).to(dev)
    x = x_full[:, :cols]
    tol = 2e-2 if dtype == torch.float16 else 1e-3
    y = torch.empty(rows, cols, dtype=dtype, device=dev)
    ops.softmax(x, y)
    assert O.max_rel_err(y.cpu(), torch.softmax(x.cpu().float(), dim=1)) < tol, ("softmax", rows, cols, dtype, pad)
    w, b = _randn(g, cols).to(dtype), _randn(g, cols).to(dtype)
    mean = torch.empty(rows, dtype=torch.float32, device=dev)
    rstd = torch.empty(rows, dtype=torch.float32, device=dev)
    ops.layer_norm(x, y, w.to(dev), b.to(dev), mean, rstd, eps=1e-5)
    ref = torch.nn.functional.layer_norm(x.cpu().float(), (cols,), w.float(), b.float(), 1e-5)
    assert O.max_rel_err(y.cpu(), ref) < tol, ("layer_norm", rows, cols, dtype, pad)
    assert torch.allclose(mean.cpu(), x.cpu().float().mean(1), atol=1e-3)
    ops.rms_norm(x, y, w.to(dev), eps=1e-6)
    xf = x.cpu().float()
    ref = xf / torch.sqrt((xf * xf).mean(1, keepdim=True) + 1e-6) * w.float()
    assert O.max_rel_err(y.cpu(), ref) < tol, ("rms_norm", rows, cols, dtype, pad)
    assert hexb200.device_status() == 0


@pytest.mark.parametrize("seed", range(12))
def test_cumsum_random_shapes(seed):
    rnd = random.Random(3000 + seed)
    g = torch.Generator().manual_seed(3000 + seed)
    shape = tuple(rnd.choice([1, 2, 5, 33, 257, 1025]) for _ in range(rnd.choice([1, 2, 3])))
    axis = rnd.randrange(len(shape))
    reverse = rnd.random() < 0.5
    x = torch.randint(-1000, 1000, shape, generator=g, dtype=torch.int32)
    out = torch.empty_like(x, device=dev)
    ops.cumsum(x.to(dev), out, axis=axis, reverse=reverse)
    ref = x.flip(axis).cumsum(axis).flip(axis) if reverse else x.cumsum(axis)
    assert torch.equal(out.cpu(), ref.to(torch.int32)), (shape, axis, reverse)
    xf = torch.rand(shape, generator=g)
    outf = torch.empty_like(xf, device=dev)
    ops.cumsum(xf.to(dev), outf, axis=axis, reverse=reverse)
    reff = xf.double().flip(axis).cumsum(axis).flip(axis) if reverse else xf.double().cumsum(axis)
    assert (outf.cpu().double() - reff).abs().max() <= 1e-3 * max(1.0, reff.abs().max().item()), (shape, axis, reverse)


def test_empty_and_degenerate_inputs_of_the_newer_entry_points():
    """Zero-sized problems return without launching; impossible ones are refused with a status, not a fault."""
    lib = hexb200.load()
    h = torch.float16
    # linear: M == 0 / N == 0 are no-ops, K == 0 gives bias (+ residual)
    a0 = torch.empty(0, 16, dtype=h, device=dev)
    w = torch.randn(16, 8, device=dev).half()
    ops.linear(a0, w, torch.empty(0, 8, dtype=h, device=dev))
    ak = torch.empty(4, 0, dtype=h, device=dev)
    wk = torch.empty(0, 8, dtype=h, device=dev)
    bias = torch.randn(8, device=dev).half()
    c = torch.full((4, 8), float("nan"), dtype=h, device=dev)
    ops.linear(ak, wk, c, bias=bias)
    assert torch.equal(c, bias.expand(4, 8))
    # cumsum: any zero extent is a no-op; a length-1 axis copies
    for shape in [(0, 5), (5, 0), (3, 0, 2)]:
        x = torch.empty(shape, device=dev)
        ops.cumsum(x, torch.empty_like(x), axis=1)
    x1 = torch.randn(7, 1, 3, device=dev)
    y1 = torch.empty_like(x1)
    ops.cumsum(x1, y1, axis=1)
    assert torch.equal(x1, y1)
    # embedding: no tokens
    wte, wpe = torch.randn(10, 8, device=dev).half(), torch.randn(4, 8, device=dev).half()
    ops.embedding(wte, wpe, torch.empty(0, 3, dtype=torch.int64, device=dev), torch.empty(0, 3, 8, dtype=h, device=dev))
    # attention: no keys cannot be normalised -> refused; no queries is a no-op
    q = torch.randn(1, 1, 4, 64, device=dev).half()
    k0 = torch.empty(1, 1, 0, 64, dtype=h, device=dev)
    with pytest.raises(hexb200.HexbError):
        ops.attention_ex(q, k0, k0, torch.empty_like(q))
    q0 = torch.empty(1, 1, 0, 64, dtype=h, device=dev)
    kk = torch.randn(1, 1, 5, 64, device=dev).half()
    ops.attention_ex(q0, kk, kk, torch.empty_like(q0))
    # iota: nothing to fill
    ops.iota(torch.empty(0, device=dev))
    assert hexb200.device_status() == 0
    assert lib.hexb_cumsum(99, None, None, 1, 1, 1, 0, None) != 0          # unknown dtype


def test_newer_ops_accept_host_tensors():
    """CPU tensors are staged through the device and the results written back in place, as the reference's
    launchers take CPU tensors (backend/triton_hexagon_launcher.py:716-728)."""
    g = torch.Generator().manual_seed(5)
    a = torch.randn(64, 32, generator=g).half()
    w = torch.randn(32, 48, generator=g).half()
    bias = torch.randn(48, generator=g).half()
    c = torch.empty(64, 48, dtype=torch.float16)
    ops.linear(a, w, c, bias=bias, act="gelu_tanh")
    ref = a.float() @ w.float() + bias.float()
    ref = 0.5 * ref * (1 + torch.tanh(0.797885 * ref + 0.035677 * ref ** 3))
    assert O.max_rel_err(c, ref) < 2e-2
    c2 = torch.empty(64, 48, dtype=torch.float32)
    ops.matmul_nt(a, w.T.contiguous(), c2)
    assert O.max_rel_err(c2, a.float() @ w.float()) < 2e-3
    x = torch.randint(-50, 50, (5, 1000), generator=g, dtype=torch.int32)
    y = torch.empty_like(x)
    ops.cumsum(x, y, axis=1)
    assert torch.equal(y, x.cumsum(1).to(torch.int32))
    q, k, v = (torch.randn(1, 2, 96, 64, generator=g).half() for _ in range(3))
    mask = torch.randn(96, 96, generator=g).half()
    o = torch.empty_like(q)
    ops.attention_ex(q, k, v, o, mask=mask)
    s = q.float() @ k.float().transpose(-1, -2) / 8.0 + mask.float()
    assert O.max_rel_err(o, torch.softmax(s, -1) @ v.float()) < 2e-2
