"""Launchers with the operator signatures of the reference's Triton kernels.

``kernels.softmax_kernel[grid](x, output, NUM_ROWS=..., NUM_COLS=..., BLOCK_SIZE=..., enableX=...)``
takes exactly the positional/keyword list of the reference kernel of that name
(test/python/triton/*.py of qualcomm/hexagon-mlir), accepts torch tensors on the CPU (as the
reference does: its driver works on host tensors, backend/driver.py:146-149) or on a CUDA device,
writes the result into the output tensor that was passed, and returns None.  ``grid`` is advisory:
the CUDA grid is chosen by the library.  Block-size constexprs are accepted and ignored.
"""
from __future__ import annotations

import inspect

import torch

from . import ops
from .options import split_options


def _as_rows(t: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    if t.dim() == 2 and tuple(t.shape) == (rows, cols):
        return t
    if not t.is_contiguous() or t.numel() < rows * cols:
        raise ValueError("tensor does not hold NUM_ROWS x NUM_COLS contiguous elements")
    return t.view(-1)[: rows * cols].view(rows, cols)


def _softmax_kernel(x_ptr, output_ptr, NUM_ROWS, NUM_COLS, BLOCK_SIZE=None):
    ops.softmax(_as_rows(x_ptr, NUM_ROWS, NUM_COLS), _as_rows(output_ptr, NUM_ROWS, NUM_COLS))


def _online_softmax(x_ptr, output_ptr, NUM_ROWS, NUM_COLS, BLOCK_ROW_SIZE=None, BLOCK_COL_SIZE=None):
    ops.softmax(_as_rows(x_ptr, NUM_ROWS, NUM_COLS), _as_rows(output_ptr, NUM_ROWS, NUM_COLS))


def _layer_norm_fwd_kernel(x_ptr, y_ptr, weights_ptr, biases_ptr, mean_ptr, rstd_ptr, BLOCK_SIZE=None,
                           EPSILON=1e-5, NUM_COLS=None, NUM_ROWS=None):
    ops.layer_norm(_as_rows(x_ptr, NUM_ROWS, NUM_COLS), _as_rows(y_ptr, NUM_ROWS, NUM_COLS), weights_ptr,
                   biases_ptr, mean_ptr, rstd_ptr, eps=EPSILON)


def _rms_norm_fwd_kernel(x_ptr, y_ptr, weights_ptr, BLOCK_SIZE=None, EPSILON=1e-6, NUM_COLS=None,
                         NUM_ROWS=None):
    ops.rms_norm(_as_rows(x_ptr, NUM_ROWS, NUM_COLS), _as_rows(y_ptr, NUM_ROWS, NUM_COLS), weights_ptr,
                 eps=EPSILON)


def _matmul(A, B, C, N_ROWS, N_COLUMNS, N_INNER):
    ops.matmul(_as_rows(A, N_ROWS, N_INNER), _as_rows(B, N_INNER, N_COLUMNS), _as_rows(C, N_ROWS, N_COLUMNS))


def _attention_fwd_kernel(pid1, Q, K, V, sm_scale, Out, H, N_CTX, BLOCK_M=None, BLOCK_DMODEL=None,
                          BLOCK_N=None, STAGE=1, stride_0=None, stride_1=None, stride_2=None, stride_3=1):
    """One launch covers the (batch, head) pair ``pid1`` like the reference kernel (off_z = pid1 // H,
    off_h = pid1 % H, test_flash_attention.py:88-92).  STAGE == 3 selects the causal mask (the
    convention named in the reference's comment, test_flash_attention.py:152-154); STAGE == 1 is the
    unmasked form the reference implements."""
    if stride_3 != 1:
        raise ValueError("attention_fwd_kernel: stride_3 must be 1")
    D = BLOCK_DMODEL if BLOCK_DMODEL is not None else Q.shape[-1]
    z, h = divmod(int(pid1), int(H))

    def head_view(t):
        base = z * stride_0 + h * stride_1
        return torch.as_strided(t, (1, 1, N_CTX, D), (stride_0, stride_1, stride_2, 1), t.storage_offset() + base)

    q, k, v, o = (head_view(t) for t in (Q, K, V, Out))
    if Q.device.type != "cuda":
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        tmp = torch.empty_like(q)
        ops.attention(q, k, v, tmp, sm_scale=sm_scale, causal=(STAGE == 3))
        o.copy_(tmp)
    else:
        ops.attention(q, k, v, o, sm_scale=sm_scale, causal=(STAGE == 3))


def _silu_kernel(x_ptr, output_ptr, BLOCK_SIZE=None):
    ops.silu(x_ptr, output_ptr)


class KernelLauncher:
    """``launcher[grid](*args, **kwargs)``: binds arguments by the reference kernel's parameter names."""

    def __init__(self, name: str, impl):
        self.name = name
        self.__name__ = name
        self._impl = impl
        self._sig = inspect.signature(impl)
        self._params = list(self._sig.parameters)

    def __getitem__(self, grid):
        def run(*args, **kwargs):
            kargs, _opts = split_options(kwargs, self._params)
            bound = self._sig.bind(*args, **kargs)
            self._impl(*bound.args, **bound.kwargs)
            return None

        return run


_REGISTRY = {
    "softmax_kernel": _softmax_kernel,
    "online_softmax": _online_softmax,
    "layer_norm_fwd_kernel": _layer_norm_fwd_kernel,
    "rms_norm_fwd_kernel": _rms_norm_fwd_kernel,
    "matmul": _matmul,
    "matmul_hexkl": _matmul,
    "attention_fwd_kernel": _attention_fwd_kernel,
    "silu_kernel": _silu_kernel,
}

_DTYPE_SUFFIXES = ("_float16", "_float32", "_float64", "_int8", "_int16", "_int32", "_int64", "_uint8",
                   "_uint16", "_uint32", "_uint64", "_bool")


def lookup(name: str) -> KernelLauncher:
    """Finds the launcher for a kernel function name; a trailing dtype suffix added by the reference's
    ``parameterize_func_name`` (test/python/utils.py:13-51) is ignored."""
    base = name
    for suf in _DTYPE_SUFFIXES:
        if base.endswith(suf):
            base = base[: -len(suf)]
            break
    if base not in _REGISTRY:
        raise NotImplementedError(f"no B200 kernel is registered for '{name}'")
    return KernelLauncher(base, _REGISTRY[base])


softmax_kernel = KernelLauncher("softmax_kernel", _softmax_kernel)
online_softmax = KernelLauncher("online_softmax", _online_softmax)
layer_norm_fwd_kernel = KernelLauncher("layer_norm_fwd_kernel", _layer_norm_fwd_kernel)
rms_norm_fwd_kernel = KernelLauncher("rms_norm_fwd_kernel", _rms_norm_fwd_kernel)
matmul = KernelLauncher("matmul", _matmul)
matmul_hexkl = KernelLauncher("matmul_hexkl", _matmul)
attention_fwd_kernel = KernelLauncher("attention_fwd_kernel", _attention_fwd_kernel)
silu_kernel = KernelLauncher("silu_kernel", _silu_kernel)
