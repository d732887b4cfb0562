"""Seeded synthetic inputs of the five benchmark configurations.

The reference's tests draw unseeded ``torch.rand`` tensors (test/python/triton/test_softmax.py:86-88,
test_layer_norm.py:86-92, test_matmul.py:78-83, test_flash_attention.py:176-184); the benchmark fixes
the shapes and distributions and this module fixes the seeds, so that every process, rank and checker
draws bit-identical tensors: values are generated in fp32 on the CPU by a ``torch.Generator`` and
cast once.  No arithmetic of the hot path lives here.
"""
from __future__ import annotations

import torch


def _gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(seed)


def make_softmax_inputs(rows=8192, cols=1024, dtype=torch.float32, seed=1001):
    """x ~ N(0, 1), [rows, cols]."""
    return torch.randn(rows, cols, generator=_gen(seed)).to(dtype)


def make_layer_norm_inputs(rows=16384, cols=4096, dtype=torch.float16, seed=1002):
    """x ~ N(0, 1); gamma ~ U(0.5, 1.5); beta ~ U(-0.1, 0.1)."""
    g = _gen(seed)
    x = torch.randn(rows, cols, generator=g).to(dtype)
    w = (0.5 + torch.rand(cols, generator=g)).to(dtype)
    b = (-0.1 + 0.2 * torch.rand(cols, generator=g)).to(dtype)
    return x, w, b


def make_matmul_inputs(M=4096, N=4096, K=4096, seed=1003):
    """A [M, K], B [K, N] ~ U(-1, 1), fp16."""
    g = _gen(seed)
    a = (2 * torch.rand(M, K, generator=g) - 1).to(torch.float16)
    b = (2 * torch.rand(K, N, generator=g) - 1).to(torch.float16)
    return a, b


def make_attention_inputs(Z=4, H=32, N=4096, D=128, dtype=torch.float16, seed=1004):
    """Q, K, V ~ N(0, 1) / sqrt(D), [Z, H, N, D]."""
    g = _gen(seed)
    s = D ** -0.5
    return tuple((torch.randn(Z, H, N, D, generator=g) * s).to(dtype) for _ in range(3))


def make_decoder_inputs(n_layers=4, d_model=2048, n_heads=16, d_ff=8192, batch=8, seq=1024, seed=1005):
    """x ~ N(0, 0.02) [batch, seq, d_model]; per layer weights ~ N(0, 1/fan_in), RMSNorm gains 1."""
    g = _gen(seed)
    x = (0.02 * torch.randn(batch, seq, d_model, generator=g)).to(torch.float16)
    weights = []
    for layer in range(n_layers):
        gl = _gen(seed + 1 + layer)
        mk = lambda r, c: (torch.randn(r, c, generator=gl) * r ** -0.5).to(torch.float16)
        weights.append({
            "wqkv": mk(d_model, 3 * d_model), "wo": mk(d_model, d_model), "wgu": mk(d_model, 2 * d_ff),
            "wd": mk(d_ff, d_model), "g1": torch.ones(d_model, dtype=torch.float16),
            "g2": torch.ones(d_model, dtype=torch.float16),
        })
    return x, weights
