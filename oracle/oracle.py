"""TEST INFRASTRUCTURE, not product code: the CPU oracle of the kernel set.

Two layers, both CPU-only:
  * ``c_*``   -- ctypes calls into liboracle.so, the plain-C restatement in oracle.c of the
                 reference's operator definitions (each C function cites the reference lines);
  * ``torch_*`` -- the exact PyTorch CPU eager calls the reference's tests compare against
                 (test/python/triton/test_softmax.py:93, test_layer_norm.py:111-113,
                 test_rms_norm.py:85-87, test_matmul.py:90, test_flash_attention.py:212), computed in
                 fp32 from the fp16 inputs where the data is fp16, so that a tolerance measures the
                 kernel and not the comparator.
Only tests/, the smoke check and the CPU legs of bench.py (cpu_baseline, the reference arm, and the
untimed comparison of gathered multi-GPU output) import this module.

Parity status: pinned against torch CPU and against outputs of the reference's own Triton kernels
executed in Triton's interpreter (tests/golden/*.npz, made by tests/golden/make_golden.py).  Parity
with the Hexagon NPU's own approximations is unpinned (no Hexagon toolchain or device output).
"""
from __future__ import annotations

import ctypes as C
import math
import subprocess
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent
_LIB = None


def build() -> Path:
    """Compiles oracle.c into liboracle.so with the committed Makefile."""
    subprocess.run(["make", "-C", str(HERE), "liboracle.so"], check=True, capture_output=True)
    return HERE / "liboracle.so"


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        path = HERE / "liboracle.so"
        if not path.exists():
            build()
        _LIB = C.CDLL(str(path))
    return _LIB


def _p(t: torch.Tensor):
    assert t.device.type == "cpu" and t.is_contiguous()
    return C.c_void_p(t.data_ptr())


_i64 = C.c_int64


# ------------------------------------------------------------------ C restatement
def c_softmax(x: torch.Tensor) -> torch.Tensor:
    y = torch.empty_like(x)
    fn = lib().oracle_softmax_f16 if x.dtype == torch.float16 else lib().oracle_softmax_f32
    fn(_p(x), _p(y), _i64(x.shape[0]), _i64(x.shape[1]))
    return y


def c_online_softmax(x: torch.Tensor, block_cols: int) -> torch.Tensor:
    y = torch.empty_like(x)
    lib().oracle_online_softmax_f32(_p(x), _p(y), _i64(x.shape[0]), _i64(x.shape[1]), _i64(block_cols))
    return y


def c_layer_norm(x, w, b, eps):
    y = torch.empty_like(x)
    mean = torch.empty(x.shape[0], dtype=torch.float32)
    rstd = torch.empty(x.shape[0], dtype=torch.float32)
    fn = lib().oracle_layer_norm_f16 if x.dtype == torch.float16 else lib().oracle_layer_norm_f32
    fn(_p(x), _p(y), _p(w), _p(b), _p(mean), _p(rstd), _i64(x.shape[0]), _i64(x.shape[1]), C.c_float(eps))
    return y, mean, rstd


def c_rms_norm(x, g, eps):
    y = torch.empty_like(x)
    fn = lib().oracle_rms_norm_f16 if x.dtype == torch.float16 else lib().oracle_rms_norm_f32
    fn(_p(x), _p(y), _p(g), _i64(x.shape[0]), _i64(x.shape[1]), C.c_float(eps))
    return y


def c_matmul(a, b, out_dtype=torch.float16, residual=None):
    M, K = a.shape
    N = b.shape[1]
    c = torch.empty(M, N, dtype=out_dtype)
    if out_dtype == torch.float32:
        assert residual is None
        lib().oracle_matmul_f16_f32(_p(a), _p(b), _p(c), _i64(M), _i64(N), _i64(K))
    else:
        lib().oracle_matmul_f16_f16(_p(a), _p(b), _p(c), _p(residual) if residual is not None else None,
                                    _i64(M), _i64(N), _i64(K))
    return c


def c_attention(q, k, v, sm_scale, causal=False, block_n=64):
    o = torch.empty_like(q)
    Z, H, N, D = q.shape
    fn = lib().oracle_attention_f16 if q.dtype == torch.float16 else lib().oracle_attention_f32
    fn(_p(q), _p(k), _p(v), _p(o), _i64(Z), _i64(H), _i64(N), _i64(D), C.c_float(sm_scale), C.c_int(int(causal)),
       _i64(block_n))
    return o


def c_attention_unfused(q, k, v, scale, causal=False):
    Z, H, N, D = q.shape
    o = torch.empty(q.shape, dtype=torch.float32)
    lib().oracle_attention_unfused_f16_f32(_p(q), _p(k), _p(v), _p(o), _i64(Z), _i64(H), _i64(N), _i64(D),
                                           C.c_float(scale), C.c_int(int(causal)))
    return o


def c_sdpa_masked(q, k, v, mask):
    """tm_tensor.attention on rank-3 operands (any float dtype; computed in fp32 from the given values)."""
    B, SQ, D = q.shape
    SKV = k.shape[1]
    qf, kf, vf = (t.float().contiguous() for t in (q, k, v))
    mf = mask.float().expand(B, SQ, SKV).contiguous()
    o = torch.zeros(B, SQ, D, dtype=torch.float32)
    lib().oracle_sdpa_masked_f32(_p(qf), _p(kf), _p(vf), _p(mf), _p(o), _i64(B), _i64(SQ), _i64(SKV), _i64(D))
    return o


def c_cumsum(x, axis=-1, reverse=False):
    """ttx.cumsum / additive ttx.scan along `axis`; float inputs are summed in fp32 and returned as fp32."""
    axis = axis % x.dim()
    outer = int(np.prod(x.shape[:axis], dtype=np.int64))
    inner = int(np.prod(x.shape[axis + 1:], dtype=np.int64))
    if x.dtype == torch.int32:
        xi = x.contiguous()
        y = torch.empty_like(xi)
        lib().oracle_cumsum_i32(_p(xi), _p(y), _i64(outer), _i64(x.shape[axis]), _i64(inner), C.c_int(int(reverse)))
        return y
    xf = x.float().contiguous()
    y = torch.empty_like(xf)
    lib().oracle_cumsum_f32(_p(xf), _p(y), _i64(outer), _i64(x.shape[axis]), _i64(inner), C.c_int(int(reverse)))
    return y


def c_silu(x):
    y = torch.empty_like(x)
    fn = lib().oracle_silu_f16 if x.dtype == torch.float16 else lib().oracle_silu_f32
    fn(_p(x), _p(y), _i64(x.numel()))
    return y


def c_gelu(x):
    y = torch.empty_like(x)
    fn = lib().oracle_gelu_f16 if x.dtype == torch.float16 else lib().oracle_gelu_f32
    fn(_p(x), _p(y), _i64(x.numel()))
    return y


def c_rope(x, theta=10000.0):
    y = torch.empty_like(x)
    B, L, H, D = x.shape
    fn = lib().oracle_rope_f16 if x.dtype == torch.float16 else lib().oracle_rope_f32
    fn(_p(x), _p(y), _i64(B), _i64(L), _i64(H), _i64(D), C.c_float(theta))
    return y


def c_sum(x):
    fn = lib().oracle_sum_f16 if x.dtype == torch.float16 else lib().oracle_sum_f32
    fn.restype = C.c_float
    return float(fn(_p(x), _i64(x.numel())))


def torch_gelu(x):
    return F.gelu(x.float(), approximate="tanh").to(x.dtype)


def torch_rope(x, theta=10000.0):
    """The PyTorch restatement the reference ships with its test (test_rope.py:58-92), in fp32."""
    B, L, H, D = x.shape
    idx = torch.arange(D, dtype=torch.float32)
    steps = torch.where(idx % 2 == 0, idx, idx - 1)
    freqs = 1.0 / (theta ** (steps / D))
    ang = torch.arange(L, dtype=torch.float32)[:, None] * freqs[None, :]
    cos, sin = torch.cos(ang).reshape(1, L, 1, D), torch.sin(ang).reshape(1, L, 1, D)
    xf = x.float()
    fwd, bwd = torch.roll(xf, -1, 3), torch.roll(xf, 1, 3)
    even = (torch.arange(D) % 2 == 0).view(1, 1, 1, D)
    return torch.where(even, xf * cos - fwd * sin, bwd * sin + xf * cos).to(x.dtype)


def c_swiglu(gu):
    rows, c2 = gu.shape
    out = torch.empty(rows, c2 // 2, dtype=torch.float16)
    lib().oracle_swiglu_f16(_p(gu), _p(out), _i64(rows), _i64(c2 // 2))
    return out


def c_decoder(x, weights, n_heads, head_dim, d_ff, batch, seq, eps):
    n = len(weights)
    out = torch.empty_like(x)
    tabs = []
    for name in ("wqkv", "wo", "wgu", "wd", "g1", "g2"):
        tabs.append((C.c_void_p * max(n, 1))(*[w[name].data_ptr() for w in weights]))
    lib().oracle_decoder_f16(_p(x), _p(out), *tabs, C.c_int(n), C.c_int(n_heads * head_dim), C.c_int(n_heads),
                             C.c_int(head_dim), C.c_int(d_ff), C.c_int(batch), C.c_int(seq), C.c_float(eps))
    return out


# ------------------------------------------------------------------ torch CPU comparator
def torch_softmax(x):
    return F.softmax(x.float(), dim=1).to(x.dtype)


def torch_layer_norm(x, w, b, eps):
    return F.layer_norm(x.float(), (x.shape[1],), weight=w.float(), bias=b.float(), eps=eps).to(x.dtype)


def torch_rms_norm(x, g, eps):
    return F.rms_norm(x.float(), (x.shape[1],), weight=g.float(), eps=eps).to(x.dtype)


def torch_matmul(a, b, out_dtype=torch.float16, residual=None):
    c = torch.matmul(a.float(), b.float())
    if residual is not None:
        c = c + residual.float()
    return c.to(out_dtype)


def torch_attention(q, k, v, sm_scale, causal=False):
    return F.scaled_dot_product_attention(q.float(), k.float(), v.float(), scale=sm_scale,
                                          is_causal=causal).to(q.dtype)


def torch_silu(x):
    return F.silu(x.float()).to(x.dtype)


def torch_decoder(x, weights, n_heads, head_dim, d_ff, batch, seq, eps, store_dtype=torch.float16):
    """The block stack in plain PyTorch CPU; activations rounded to store_dtype between operators."""
    d = n_heads * head_dim
    rd = (lambda t: t.to(store_dtype).float()) if store_dtype is not None else (lambda t: t)
    cur = x.float().reshape(batch * seq, d)
    for w in weights:
        n = rd(F.rms_norm(cur, (d,), weight=w["g1"].float(), eps=eps))
        qkv = rd(n @ w["wqkv"].float())
        q, k, v = (qkv[:, i * d:(i + 1) * d].reshape(batch, seq, n_heads, head_dim).transpose(1, 2) for i in range(3))
        a = rd(F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=1.0 / math.sqrt(head_dim)))
        a = a.transpose(1, 2).reshape(batch * seq, d)
        h = rd(a @ w["wo"].float() + cur)
        n = rd(F.rms_norm(h, (d,), weight=w["g2"].float(), eps=eps))
        gu = rd(n @ w["wgu"].float())
        act = rd(F.silu(gu[:, :d_ff]) * gu[:, d_ff:])
        cur = rd(act @ w["wd"].float() + h)
    return cur.to(x.dtype).reshape(x.shape)


def torch_gpt2(sd, n_layer, n_head, eps, input_ids):
    """GPT2LMHeadModel forward in plain fp32 torch from a Hugging Face state dict: what the reference runs
    on x86 as its expected result (test/python/torch-mlir/gpt2lmheadmodel.py:30-33, 143-169).  Conv1D is
    x @ W + b with W [in, out]; GELU is the tanh form; attention is causal with scale 1/sqrt(head_dim);
    the LM head is tied to the token embedding."""
    f = {k: v.float() for k, v in sd.items()}
    B, S = input_ids.shape
    x = f["transformer.wte.weight"][input_ids] + f["transformer.wpe.weight"][:S]
    d = x.shape[-1]
    hd = d // n_head
    for i in range(n_layer):
        p = f"transformer.h.{i}."
        h = F.layer_norm(x, (d,), f[p + "ln_1.weight"], f[p + "ln_1.bias"], eps)
        qkv = h @ f[p + "attn.c_attn.weight"] + f[p + "attn.c_attn.bias"]
        q, k, v = (t.view(B, S, n_head, hd).transpose(1, 2) for t in qkv.split(d, dim=-1))
        s = (q @ k.transpose(-1, -2)) / math.sqrt(hd)
        s = s.masked_fill(torch.ones(S, S, dtype=torch.bool).triu(1), float("-inf"))
        a = (torch.softmax(s, dim=-1) @ v).transpose(1, 2).reshape(B, S, d)
        x = x + a @ f[p + "attn.c_proj.weight"] + f[p + "attn.c_proj.bias"]
        h = F.layer_norm(x, (d,), f[p + "ln_2.weight"], f[p + "ln_2.bias"], eps)
        h = h @ f[p + "mlp.c_fc.weight"] + f[p + "mlp.c_fc.bias"]
        h = 0.5 * h * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (h + 0.044715 * h ** 3)))
        x = x + h @ f[p + "mlp.c_proj.weight"] + f[p + "mlp.c_proj.bias"]
    x = F.layer_norm(x, (d,), f["transformer.ln_f.weight"], f["transformer.ln_f.bias"], eps)
    return x @ f["transformer.wte.weight"].T


# ------------------------------------------------------------------ seeded inputs of the five configurations
# The seeded generators live in the product package (hexb200.synth) so that the benchmark's GPU arm
# needs nothing from this directory; they are re-exported here for the tests.
from hexb200.synth import (make_attention_inputs, make_decoder_inputs, make_layer_norm_inputs,  # noqa: E402,F401
                           make_matmul_inputs, make_softmax_inputs)


def max_rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """max |got - ref| / max |ref|: the relative error the tolerances of the benchmark are stated in."""
    ref = ref.float()
    denom = ref.abs().max().clamp_min(1e-30)
    return float((got.float() - ref).abs().max() / denom)
