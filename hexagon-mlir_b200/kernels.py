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


def _flat(t, n):
    if not t.is_contiguous() or t.numel() < n:
        raise ValueError("tensor does not hold the elements the launch covers")
    return t.view(-1)[:n]


def _covered(x, BLOCK_SIZE, _grid):
    """Elements one launch touches: programs * BLOCK_SIZE, as the reference kernels index them."""
    progs = 1
    for g in (_grid if isinstance(_grid, (tuple, list)) else (_grid,)):
        progs *= int(g)
    return min(x.numel(), progs * int(BLOCK_SIZE))


def _gelu_kernel(x_ptr, output_ptr, BLOCK_SIZE, _grid=(1,)):
    n = _covered(x_ptr, BLOCK_SIZE, _grid)
    ops.unary("gelu_tanh", _flat(x_ptr, n), _flat(output_ptr, n))


def _cos_kernel(x_ptr, output_ptr, BLOCK_SIZE, _grid=(1,)):
    n = _covered(x_ptr, BLOCK_SIZE, _grid)
    ops.unary("cos", _flat(x_ptr, n), _flat(output_ptr, n))


def _sin_kernel(x_ptr, output_ptr, BLOCK_SIZE, _grid=(1,)):
    n = _covered(x_ptr, BLOCK_SIZE, _grid)
    ops.unary("sin", _flat(x_ptr, n), _flat(output_ptr, n))


def _rsqrt_kernel(x_ptr, output_ptr, BLOCK_SIZE, _grid=(1,)):
    n = _covered(x_ptr, BLOCK_SIZE, _grid)
    ops.unary("rsqrt", _flat(x_ptr, n), _flat(output_ptr, n))


def _add_kernel(x_ptr, y_ptr, output_ptr, *rest, BLOCK_SIZE=None, n_elements=None, block_size=None, _grid=(1,)):
    """Two reference kernels share this name: add_kernel(x, y, out, BLOCK_SIZE) (test_vec_add.py:19-25) and
    add_kernel(x, y, out, n_elements, block_size) with a bounds mask (test_static_allocator_vadd.py:27-35)."""
    rest = list(rest)
    if BLOCK_SIZE is None and block_size is None and len(rest) == 1:
        BLOCK_SIZE = rest.pop(0)                      # add_kernel(x, y, out, BLOCK_SIZE)
    if rest:
        n_elements = rest.pop(0)                      # add_kernel(x, y, out, n_elements, block_size[=...])
    if rest:
        block_size = rest.pop(0)
    if rest:
        raise TypeError("add_kernel: too many positional arguments")
    bs = BLOCK_SIZE if BLOCK_SIZE is not None else block_size
    if bs is None:
        raise TypeError("add_kernel: BLOCK_SIZE (or block_size) is required")
    n = _covered(x_ptr, bs, _grid)
    if n_elements is not None:
        n = min(n, int(n_elements))
    ops.binary("add", _flat(x_ptr, n), _flat(y_ptr, n), _flat(output_ptr, n))


def _gelu_bptr_kernel(x_ptr, output_ptr, N, H, W, C):
    """Whole-tensor GELU through block pointers over an [N, H, W, C] tensor (test_gelu_block_ptr.py:31-60)."""
    n = int(N) * int(H) * int(W) * int(C)
    ops.unary("gelu_tanh", _flat(x_ptr, n), _flat(output_ptr, n))


def _flatten_pid(ptr, _grid=(1,)):
    """Every program of a 1-, 2- or 3-D grid stores its flattened id at that index (test_multidim_grid.py:21-37):
    the result is 0, 1, ..., prod(grid) - 1."""
    progs = 1
    for g in (_grid if isinstance(_grid, (tuple, list)) else (_grid,)):
        progs *= int(g)
    ops.iota(_flat(ptr, progs))


def _add_kernel_scalar(x_ptr, y_ptr, output_ptr, n_elements, BLOCK_SIZE, _grid=(1,)):
    n = min(int(n_elements), _covered(x_ptr, BLOCK_SIZE, _grid))
    ops.binary("add", _flat(x_ptr, n), _flat(y_ptr, n), _flat(output_ptr, n))


def _add_2d_kernel(x_ptr, y_ptr, output_ptr, NUM_ROWS, NUM_COLS):
    n = NUM_ROWS * NUM_COLS
    ops.binary("add", _flat(x_ptr, n), _flat(y_ptr, n), _flat(output_ptr, n))


def _div_kernel(x_ptr, y_ptr, output_ptr, NUM_ROWS, NUM_COLS):
    n = NUM_ROWS * NUM_COLS
    ops.binary("div", _flat(x_ptr, n), _flat(y_ptr, n), _flat(output_ptr, n))


def _sum_kernel(x_ptr, output_ptr, BLOCK_SIZE, _grid=(1,)):
    """Program pid writes the sum of its BLOCK_SIZE elements to output[pid] (test_sum.py:31-36)."""
    progs = int(_grid[0]) if isinstance(_grid, (tuple, list)) else int(_grid)
    flat = x_ptr.view(-1)
    for pid in range(progs):
        ops.vec_sum(flat[pid * BLOCK_SIZE:(pid + 1) * BLOCK_SIZE], output_ptr.view(-1)[pid:pid + 1])


def _rope_kernel(x_ptr, output_ptr, BATCH_SIZE, BATCH_SIZE_STRIDE, SEQ_LEN, SEQ_LEN_STRIDE, N_HEADS, N_HEADS_STRIDE,
                 N_FEATURES, N_FEATURES_STRIDE, BLOCK_SIZE=None, THETA=10000.0):
    if N_FEATURES_STRIDE != 1:
        raise ValueError("rope_kernel: N_FEATURES_STRIDE must be 1")
    shape = (BATCH_SIZE, SEQ_LEN, N_HEADS, N_FEATURES)
    strides = (BATCH_SIZE_STRIDE, SEQ_LEN_STRIDE, N_HEADS_STRIDE, 1)
    xv = torch.as_strided(x_ptr, shape, strides, x_ptr.storage_offset())
    ov = torch.as_strided(output_ptr, shape, strides, output_ptr.storage_offset())
    if x_ptr.device.type != "cuda":
        tmp = torch.empty(shape, dtype=x_ptr.dtype)
        ops.rope(xv.contiguous(), tmp, theta=THETA)
        ov.copy_(tmp)
    else:
        ops.rope(xv, ov, theta=THETA)


class KernelLauncher:
    """``launcher[grid](*args, **kwargs)``: binds arguments by the reference kernel's parameter names."""

    def __init__(self, name: str, impl):
        self.name = name
        self.__name__ = name
        self._impl = impl
        self._params = frozenset(inspect.signature(impl).parameters)
        self._wants_grid = "_grid" in self._params

    def __getitem__(self, grid):
        impl, params, wants_grid = self._impl, self._params, self._wants_grid

        def run(*args, **kwargs):
            kargs, _opts = split_options(kwargs, params)
            if wants_grid:
                kargs["_grid"] = grid
            impl(*args, **kargs)      # Python's own binding raises TypeError for a wrong argument list
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
    "gelu_kernel": _gelu_kernel,
    "libd_gelu_kernel": _gelu_kernel,          # the same formula with libdevice.tanh (test_libd_gelu.py:35-49)
    "gelu_bptr_kernel": _gelu_bptr_kernel,
    "add_kernel_mulithreaded": _add_kernel,    # (sic) test_vec_add_multithread.py:23
    "flatten_pid": _flatten_pid,
    "cos_kernel": _cos_kernel,
    "sin_kernel": _sin_kernel,
    "rsqrt_kernel": _rsqrt_kernel,
    "add_kernel": _add_kernel,
    "add_kernel_scalar": _add_kernel_scalar,
    "add_2d_kernel": _add_2d_kernel,
    "div_kernel": _div_kernel,
    "sum_kernel": _sum_kernel,
    "rope_kernel": _rope_kernel,
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
gelu_kernel = KernelLauncher("gelu_kernel", _gelu_kernel)
cos_kernel = KernelLauncher("cos_kernel", _cos_kernel)
sin_kernel = KernelLauncher("sin_kernel", _sin_kernel)
rsqrt_kernel = KernelLauncher("rsqrt_kernel", _rsqrt_kernel)
add_kernel = KernelLauncher("add_kernel", _add_kernel)
add_kernel_scalar = KernelLauncher("add_kernel_scalar", _add_kernel_scalar)
add_2d_kernel = KernelLauncher("add_2d_kernel", _add_2d_kernel)
div_kernel = KernelLauncher("div_kernel", _div_kernel)
sum_kernel = KernelLauncher("sum_kernel", _sum_kernel)
rope_kernel = KernelLauncher("rope_kernel", _rope_kernel)
