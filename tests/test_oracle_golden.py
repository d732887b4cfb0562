"""CPU: pins the oracle against the fixtures produced by the reference's own Triton kernels
(tests/golden/make_golden.py) and against the torch values the reference tests assert against.
Tolerances are the reference tests' own (softmax atol 1e-5 / 1e-3, layer norm 1e-5, rms norm 1e-2,
matmul 0.2, flash attention allclose defaults, silu 1e-2)."""
import math
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O


def load(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    return {k: torch.from_numpy(z[k]) for k in z.files}


@pytest.mark.parametrize("tag,atol", [("f32", 1e-5), ("f16", 1e-3)])
def test_softmax_golden(golden_dir, tag, atol):
    g = load(golden_dir, f"softmax_128x128_{tag}")
    x = g["in0"]
    for got in (O.c_softmax(x), O.torch_softmax(x)):
        assert torch.allclose(got, g["output"], atol=atol)
        assert torch.allclose(got, g["expected"], atol=atol)


def test_online_softmax_golden(golden_dir):
    g = load(golden_dir, "online_softmax_128x128_f32")
    got = O.c_online_softmax(g["in0"], 32)
    assert torch.allclose(got, g["output"], atol=1e-5)
    assert torch.allclose(got, g["expected"], atol=1e-5)


def test_layer_norm_golden(golden_dir):
    g = load(golden_dir, "layer_norm_27x1024_f32")
    x, w, b = g["in0"], g["in1"], g["in2"]
    y, mean, rstd = O.c_layer_norm(x, w, b, 1e-5)
    assert torch.allclose(y, g["output"], atol=1e-5)
    assert torch.allclose(y, g["expected"], atol=1e-5)
    assert torch.allclose(O.torch_layer_norm(x, w, b, 1e-5), g["output"], atol=1e-5)
    assert torch.allclose(mean, x.mean(dim=1), atol=1e-6)
    assert torch.allclose(rstd, 1.0 / torch.sqrt(x.var(dim=1, unbiased=False) + 1e-5), rtol=1e-5)


@pytest.mark.parametrize("tag", ["f32", "f16"])
def test_rms_norm_golden(golden_dir, tag):
    g = load(golden_dir, f"rms_norm_127x513_{tag}")
    x, w = g["in0"], g["in1"]
    eps = 1e-5
    for got in (O.c_rms_norm(x, w, eps), O.torch_rms_norm(x, w, eps)):
        assert torch.allclose(got, g["output"], atol=1e-2)
        assert torch.allclose(got, g["expected"], atol=1e-2)


def test_matmul_golden(golden_dir):
    g = load(golden_dir, "matmul_256x128x64_f16")
    a, b = g["in0"], g["in1"]
    for got in (O.c_matmul(a, b, torch.float16), O.torch_matmul(a, b, torch.float16)):
        assert torch.allclose(got, g["output"], atol=2e-1)
        assert torch.allclose(got, g["expected"], atol=2e-1)
        assert O.max_rel_err(got, g["output"]) < 2e-3  # one fp16 rounding apart at most
    c32 = O.c_matmul(a, b, torch.float32)
    assert torch.allclose(c32, a.float() @ b.float(), rtol=1e-5, atol=1e-5)


def test_flash_attention_golden(golden_dir):
    g = load(golden_dir, "flash_attention_1x1x256x64_f32")
    q, k, v = g["in0"], g["in1"], g["in2"]
    got = O.c_attention(q, k, v, 0.5, causal=False, block_n=64)
    assert torch.allclose(got, g["output"], rtol=1e-5, atol=1e-6)
    assert torch.allclose(got, g["expected"], rtol=1e-5, atol=1e-6)
    assert torch.allclose(O.torch_attention(q, k, v, 0.5), g["output"], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("tag", ["f32", "f16"])
def test_silu_golden(golden_dir, tag):
    g = load(golden_dir, f"silu_16384_{tag}")
    x = g["in0"]
    for got in (O.c_silu(x), O.torch_silu(x)):
        assert torch.allclose(got, g["output"], atol=1e-2)
        assert torch.allclose(got, g["expected"], atol=1e-2)


def test_known_constants():
    # constants the reference's lowered IR carries (SDPA.mlir:18, hexkl_attention/input.mlir:6)
    assert abs(8 ** -0.5 - 0.353553385) < 1e-8
    assert abs(0.5 * 1.44269504 - 0.72134751) < 1e-7


def test_c_oracle_matches_torch_on_config_shapes():
    torch.manual_seed(0)
    x = O.make_softmax_inputs(64, 1024)
    assert torch.allclose(O.c_softmax(x), O.torch_softmax(x), atol=1e-6)
    x, w, b = O.make_layer_norm_inputs(32, 4096)
    y, _, _ = O.c_layer_norm(x, w, b, 1e-5)
    assert O.max_rel_err(y, O.torch_layer_norm(x, w, b, 1e-5)) < 2e-3
    a, bm = O.make_matmul_inputs(64, 96, 128)
    assert O.max_rel_err(O.c_matmul(a, bm), O.torch_matmul(a, bm)) < 2e-3
    q, k, v = O.make_attention_inputs(1, 2, 256, 128)
    for causal in (False, True):
        got = O.c_attention(q, k, v, 128 ** -0.5, causal)
        assert O.max_rel_err(got, O.torch_attention(q, k, v, 128 ** -0.5, causal)) < 2e-2
        unf = O.c_attention_unfused(q, k, v, 128 ** -0.5, causal)
        assert O.max_rel_err(unf, O.torch_attention(q.float(), k.float(), v.float(), 128 ** -0.5, causal)) < 1e-4


def test_decoder_oracles_agree():
    x, ws = O.make_decoder_inputs(2, 256, 2, 512, 2, 128)
    c = O.c_decoder(x.reshape(-1, 256), ws, 2, 128, 512, 2, 128, 1e-6).reshape(x.shape)
    t = O.torch_decoder(x, ws, 2, 128, 512, 2, 128, 1e-6)
    assert O.max_rel_err(c, t) < 2e-2


# ------------------------------------------------------------------ elementwise row (gelu, rope, sum, add/div, cos/sin)
@pytest.mark.parametrize("tag,atol", [("f32", 1e-5), ("f16", 1e-2)])
def test_gelu_golden(golden_dir, tag, atol):
    g = load(golden_dir, f"gelu_16384_{tag}")
    for got in (O.c_gelu(g["in0"]), O.torch_gelu(g["in0"])):
        assert torch.allclose(got, g["output"], atol=atol)
        assert torch.allclose(got, g["expected"], atol=atol)


@pytest.mark.parametrize("tag,atol", [("f32", 1e-3), ("f16", 1e-2)])
def test_rope_golden(golden_dir, tag, atol):
    g = load(golden_dir, f"rope_4x8x16x32_{tag}")
    for got in (O.c_rope(g["in0"]), O.torch_rope(g["in0"])):
        assert torch.allclose(got, g["output"], atol=atol, rtol=0)
        assert torch.allclose(got, g["expected"], atol=atol, rtol=0)


def test_sum_golden(golden_dir):
    g = load(golden_dir, "sum_16384_f32")
    assert abs(O.c_sum(g["in0"]) - float(g["output"])) < 1e-2
    assert abs(O.c_sum(g["in0"]) - float(g["expected"])) < 1e-2


def test_binary_and_math_golden(golden_dir):
    g = load(golden_dir, "vec_add_f32")
    assert torch.allclose(g["in0"] + g["in1"], g["output"])
    g = load(golden_dir, "vec_div_2d_f32")
    assert torch.allclose(g["in0"] / g["in1"], g["output"], atol=1e-6)
    g = load(golden_dir, "math_ops_cos_sin_f32")
    assert torch.allclose(torch.cos(g["in0"]), g["output0"], atol=1e-5)
    assert torch.allclose(torch.sin(g["in0"]), g["output1"], atol=1e-5)


# ------------------------------------------------------------------ tm_tensor.attention (masked SDPA)
@pytest.mark.parametrize("B,SQ,SKV,D", [(2, 4, 4, 8),        # the operand shapes of the reference's SDPA.mlir lit test
                                        (3, 37, 53, 16), (2, 128, 128, 64)])
def test_sdpa_masked_oracle_vs_torch(B, SQ, SKV, D):
    g = torch.Generator().manual_seed(B * 7 + SQ)
    q, k, v = (torch.randn(B, n, D, generator=g) for n in (SQ, SKV, SKV))
    mask = torch.randn(B, SQ, SKV, generator=g)
    mask[:, :, ::3] = -1e4                      # a large negative bias: those keys get zero weight
    got = O.c_sdpa_masked(q, k, v, mask)
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=mask)
    assert torch.allclose(got, ref, rtol=1e-5, atol=1e-6)
    # the scale constant FileCheck expects for d = 8 (SDPA.mlir:17): 1/sqrt(8) as f32
    if D == 8:
        assert abs(np.float32(1.0 / math.sqrt(8)) - np.float32(0.353553385)) < 1e-9


def test_sdpa_masked_causal_mask_equals_causal_attention():
    g = torch.Generator().manual_seed(5)
    B, S, D = 2, 96, 32
    q, k, v = (torch.randn(B, S, D, generator=g) for _ in range(3))
    mask = torch.full((S, S), float("-inf")).triu(1).expand(B, S, S)
    got = O.c_sdpa_masked(q, k, v, mask)
    ref = O.c_attention(q.unsqueeze(1).contiguous(), k.unsqueeze(1).contiguous(), v.unsqueeze(1).contiguous(),
                        1.0 / math.sqrt(D), causal=True).squeeze(1)
    assert torch.allclose(got, ref, rtol=1e-5, atol=1e-6)


# ------------------------------------------------------------------ ttx.cumsum / additive ttx.scan
@pytest.mark.parametrize("shape,axis", [((16, 32), 1),      # cumsum_2D.mlir
                                        ((256,), 0),         # the 1-D lit tests
                                        ((5, 7, 9), 1), ((5, 7, 9), 0)])
@pytest.mark.parametrize("reverse", [False, True])
def test_cumsum_oracle_vs_torch(shape, axis, reverse):
    g = torch.Generator().manual_seed(len(shape) * 10 + axis)
    x = torch.randn(*shape, generator=g)
    xi = torch.randint(-2 ** 30, 2 ** 30, shape, generator=g, dtype=torch.int32)
    for t in (x, xi):
        got = O.c_cumsum(t, axis, reverse)
        ref = t.flip(axis).cumsum(axis).flip(axis) if reverse else t.cumsum(axis)
        if t.dtype == torch.int32:
            assert torch.equal(got, ref.to(torch.int32))      # wraps like two's complement
        else:
            assert torch.allclose(got, ref, rtol=1e-5, atol=1e-5)


# ------------------------------------------------------------------ GPT-2 (two layers, random weights)
def test_gpt2_oracle_matches_transformers():
    """Pins the plain-torch GPT-2 restatement on Hugging Face's GPT2LMHeadModel, the model the reference
    test instantiates (with pretrained weights, which need a network; random weights here)."""
    transformers = pytest.importorskip("transformers")
    import hexb200
    from hexb200 import gpt2
    cfg = gpt2.GPT2Config(n_layer=2, n_embd=64, n_head=4, n_positions=32, vocab_size=101)
    sd = gpt2.random_state_dict(cfg, seed=3, dtype=torch.float32)
    hf_cfg = transformers.GPT2Config(n_layer=cfg.n_layer, n_embd=cfg.n_embd, n_head=cfg.n_head,
                                     n_positions=cfg.n_positions, vocab_size=cfg.vocab_size)
    model = transformers.GPT2LMHeadModel(hf_cfg).eval()
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not unexpected and all(("attn.bias" in m or "masked_bias" in m or m == "lm_head.weight") for m in missing)
    ids = torch.randint(0, cfg.vocab_size, (2, 17), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = model(input_ids=ids).logits
    got = O.torch_gpt2(sd, cfg.n_layer, cfg.n_head, cfg.layer_norm_epsilon, ids)
    assert torch.allclose(got, ref, rtol=1e-4, atol=1e-5)
