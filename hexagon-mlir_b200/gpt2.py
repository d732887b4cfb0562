"""GPT-2 language-model forward on one B200, built from the library's kernels.

The reference's largest workload is `GPT2LMHeadModel` cut to two layers, exported through torch-mlir
to linalg, compiled, run on the device and compared with the PyTorch result on the top-5 tokens of the
last position (test/python/torch-mlir/gpt2lmheadmodel.py:143-169, comparison :74-95).  Here the same
network runs as hand-written kernels: per block

    LayerNorm -> linear(c_attn) + bias -> causal attention (heads read in place from the fused
    q|k|v buffer through strides) -> linear(c_proj) + bias + residual -> LayerNorm ->
    linear(c_fc) + bias + GELU(tanh) -> linear(c_proj) + bias + residual

seven launches per block, then the final LayerNorm and the tied LM head as a transposed-weight matmul
against the token-embedding table.  Weights follow the Hugging Face `GPT2LMHeadModel.state_dict()`
names (Conv1D weights are [in, out]); buffers are allocated once per (batch, seq).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import ops


@dataclass
class GPT2Config:
    """The fields of `transformers.GPT2Config` the forward pass reads (defaults: gpt2-small, two layers
    as in the reference's test)."""
    n_layer: int = 2
    n_embd: int = 768
    n_head: int = 12
    n_positions: int = 1024
    vocab_size: int = 50257
    layer_norm_epsilon: float = 1e-5


def random_state_dict(cfg: GPT2Config, seed: int = 0, dtype=torch.float16) -> dict:
    """Random weights under the Hugging Face names.  Matrices ~ N(0, 0.02) like GPT-2's initialiser; norm
    scales near 1 and biases ~ N(0, 0.02) rather than the initialiser's exact 1 / 0, so that every
    parameter matters to the result."""
    g = torch.Generator().manual_seed(seed)
    d = cfg.n_embd

    def n(*shape, std=0.02, mean=0.0):
        return (torch.randn(*shape, generator=g) * std + mean).to(dtype)

    sd = {"transformer.wte.weight": n(cfg.vocab_size, d), "transformer.wpe.weight": n(cfg.n_positions, d, std=0.01)}
    for i in range(cfg.n_layer):
        p = f"transformer.h.{i}."
        sd[p + "ln_1.weight"], sd[p + "ln_1.bias"] = n(d, std=0.1, mean=1.0), n(d)
        sd[p + "attn.c_attn.weight"], sd[p + "attn.c_attn.bias"] = n(d, 3 * d), n(3 * d)
        sd[p + "attn.c_proj.weight"], sd[p + "attn.c_proj.bias"] = n(d, d), n(d)
        sd[p + "ln_2.weight"], sd[p + "ln_2.bias"] = n(d, std=0.1, mean=1.0), n(d)
        sd[p + "mlp.c_fc.weight"], sd[p + "mlp.c_fc.bias"] = n(d, 4 * d), n(4 * d)
        sd[p + "mlp.c_proj.weight"], sd[p + "mlp.c_proj.bias"] = n(4 * d, d), n(d)
    sd["transformer.ln_f.weight"], sd["transformer.ln_f.bias"] = n(d, std=0.1, mean=1.0), n(d)
    return sd


class GPT2Runner:
    """Forward pass of GPT2LMHeadModel (no KV cache, no dropout: the reference runs inference on a prompt)."""

    LAUNCHES_PER_LAYER = 7

    def __init__(self, cfg: GPT2Config, state_dict: dict, device="cuda:0"):
        if cfg.n_embd % cfg.n_head:
            raise ValueError("n_embd must be a multiple of n_head")
        self.cfg = cfg
        self.device = torch.device(device)
        self.head_dim = cfg.n_embd // cfg.n_head
        self.w = {}
        for k, v in state_dict.items():
            if k.endswith(".attn.bias") or k.endswith(".attn.masked_bias") or k == "lm_head.weight":
                continue  # causal-mask buffers of older checkpoints; the LM head is tied to wte
            self.w[k] = v.detach().to(device=self.device, dtype=torch.float16).contiguous()
        need = ["transformer.wte.weight", "transformer.wpe.weight", "transformer.ln_f.weight", "transformer.ln_f.bias"]
        for i in range(cfg.n_layer):
            need += [f"transformer.h.{i}.{n}" for n in (
                "ln_1.weight", "ln_1.bias", "attn.c_attn.weight", "attn.c_attn.bias", "attn.c_proj.weight",
                "attn.c_proj.bias", "ln_2.weight", "ln_2.bias", "mlp.c_fc.weight", "mlp.c_fc.bias",
                "mlp.c_proj.weight", "mlp.c_proj.bias")]
        missing = [n for n in need if n not in self.w]
        if missing:
            raise KeyError(f"GPT2Runner: missing weights {missing[:4]}{'...' if len(missing) > 4 else ''}")
        self._bufs = {}
        self._graphs = {}

    def launches(self) -> int:
        """Kernel launches of one forward pass (embedding + blocks + final norm + LM head)."""
        return 1 + self.LAUNCHES_PER_LAYER * self.cfg.n_layer + 2

    def _buffers(self, B: int, S: int, logits_dtype, last_only: bool = False):
        key = (B, S, logits_dtype, last_only)
        if key not in self._bufs:
            d, dev, h = self.cfg.n_embd, self.device, torch.float16
            T = B * S
            self._bufs[key] = {
                "x": torch.empty(T, d, dtype=h, device=dev), "x2": torch.empty(T, d, dtype=h, device=dev),
                "ln": torch.empty(T, d, dtype=h, device=dev), "qkv": torch.empty(T, 3 * d, dtype=h, device=dev),
                "att": torch.empty(T, d, dtype=h, device=dev), "fc": torch.empty(T, 4 * d, dtype=h, device=dev),
                # rows padded to a multiple of 16 bytes so that the LM head stores whole vectors; one row per
                # sequence when only the last position is asked for
                "logits": torch.empty(B if last_only else T, (self.cfg.vocab_size + 7) // 8 * 8, dtype=logits_dtype,
                                      device=dev),
            }
        return self._bufs[key]

    def forward(self, input_ids: torch.Tensor, logits_dtype=torch.float32, graph: bool = False,
                last_only: bool = False, check_ids: bool = False) -> torch.Tensor:
        """input_ids: int64 [batch, seq] on the runner's device.  Returns logits [batch, seq, vocab]
        (a buffer owned by the runner, overwritten by the next call with the same shape).

        last_only=True computes the final LayerNorm and the LM head for the last position of every
        sequence only and returns [batch, 1, vocab]: what next-token prediction -- and the reference's
        top-5 comparison -- reads; the LM head is more than half of a full forward pass.

        graph=True replays the 17 launches as one CUDA graph captured on the first call with this
        (batch, seq, logits dtype): for short prompts the launches, not the kernels, set the latency.

        check_ids=True validates the token ids against the vocabulary before the launches (one device
        synchronisation) and raises IndexError for a bad one, as the torch model does.  Without it an
        out-of-range id embeds as a zero row and only the device status word records it: callers that
        replay graphs should poll hexb200.device_status() between requests."""
        cfg = self.cfg
        if input_ids.dim() != 2 or input_ids.dtype != torch.int64 or input_ids.device != self.device:
            raise ValueError("GPT2Runner: int64 [batch, seq] ids on the runner's device expected")
        B, S = input_ids.shape
        if S > cfg.n_positions:
            raise ValueError("GPT2Runner: sequence longer than n_positions")
        if check_ids and input_ids.numel():
            lo, hi = int(input_ids.min()), int(input_ids.max())
            if lo < 0 or hi >= cfg.vocab_size:
                raise IndexError(f"GPT2Runner: token id {lo if lo < 0 else hi} is outside [0, {cfg.vocab_size})")
        if not graph:
            return self._forward(input_ids.contiguous(), logits_dtype, last_only)
        key = (B, S, logits_dtype, last_only)
        if key not in self._graphs:
            static_ids = input_ids.clone()
            self._forward(static_ids, logits_dtype, last_only)   # first call outside capture: one-time set-up
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                out = self._forward(static_ids, logits_dtype, last_only)
            self._graphs[key] = (g, static_ids, out)
        g, static_ids, out = self._graphs[key]
        static_ids.copy_(input_ids)
        g.replay()
        return out

    def _forward(self, input_ids: torch.Tensor, logits_dtype, last_only: bool = False) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        B, S = input_ids.shape
        d, H, D = cfg.n_embd, cfg.n_head, self.head_dim
        b = self._buffers(B, S, logits_dtype, last_only)
        x, x2 = b["x"], b["x2"]
        ops.embedding(w["transformer.wte.weight"], w["transformer.wpe.weight"], input_ids, x.view(B, S, d))
        qkv4 = b["qkv"].view(B, S, 3, H, D)
        q, k, v = (qkv4[:, :, i].permute(0, 2, 1, 3) for i in range(3))      # [B, H, S, D] views of the fused buffer
        att4 = b["att"].view(B, S, H, D).permute(0, 2, 1, 3)
        for i in range(cfg.n_layer):
            p = f"transformer.h.{i}."
            ops.layer_norm(x, b["ln"], w[p + "ln_1.weight"], w[p + "ln_1.bias"], eps=cfg.layer_norm_epsilon)
            ops.linear(b["ln"], w[p + "attn.c_attn.weight"], b["qkv"], bias=w[p + "attn.c_attn.bias"])
            ops.attention(q, k, v, att4, causal=True)
            ops.linear(b["att"], w[p + "attn.c_proj.weight"], x2, bias=w[p + "attn.c_proj.bias"], residual=x)
            ops.layer_norm(x2, b["ln"], w[p + "ln_2.weight"], w[p + "ln_2.bias"], eps=cfg.layer_norm_epsilon)
            ops.linear(b["ln"], w[p + "mlp.c_fc.weight"], b["fc"], bias=w[p + "mlp.c_fc.bias"], act="gelu_tanh")
            ops.linear(b["fc"], w[p + "mlp.c_proj.weight"], x, bias=w[p + "mlp.c_proj.bias"], residual=x2)
        if last_only:
            last = x[S - 1::S]                               # the last position of every sequence: [B, d], row stride S * d
            ln = b["ln"][:B]
            ops.layer_norm(last, ln, w["transformer.ln_f.weight"], w["transformer.ln_f.bias"], eps=cfg.layer_norm_epsilon)
            logits = b["logits"][:B, :cfg.vocab_size]
            ops.matmul_nt(ln, w["transformer.wte.weight"], logits)
            return logits.unflatten(0, (B, 1))
        ops.layer_norm(x, b["ln"], w["transformer.ln_f.weight"], w["transformer.ln_f.bias"], eps=cfg.layer_norm_epsilon)
        logits = b["logits"][:, :cfg.vocab_size]
        ops.matmul_nt(b["ln"], w["transformer.wte.weight"], logits)
        return logits.unflatten(0, (B, S))

    def flops(self, B: int, S: int) -> float:
        """Matmul and attention FLOPs of one forward pass (causal attention counted at half the square)."""
        return self.flops_of(self.cfg, B, S)

    @staticmethod
    def flops_of(cfg: GPT2Config, B: int, S: int) -> float:
        d, L, V = cfg.n_embd, cfg.n_layer, cfg.vocab_size
        T = B * S
        per_layer = 2.0 * T * d * (3 * d + d + 4 * d + 4 * d) + 4.0 * B * S * S * d * 0.5
        return L * per_layer + 2.0 * T * d * V


def top5_match(logits_a: torch.Tensor, logits_b: torch.Tensor, rtol: float = 0.03):
    """The reference's acceptance test (gpt2lmheadmodel.py:52-95): the five most probable tokens of the
    last position of the first sequence agree, and their logits agree within rtol."""
    va, ia = torch.topk(logits_a[0, -1, :].float().cpu(), 5)
    vb, ib = torch.topk(logits_b[0, -1, :].float().cpu(), 5)
    return bool(torch.equal(ia, ib)), bool(torch.allclose(va, vb, rtol))
