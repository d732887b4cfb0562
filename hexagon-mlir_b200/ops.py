"""Tensor-level entry points over the C ABI.

Every function writes into caller-provided output tensors (the reference launcher copies results
back into the tensors the test passed, qcom_hexagon_backend/backend/triton_hexagon_launcher.py:716-728)
and returns nothing useful.  CUDA tensors are used in place on the current stream; CPU tensors go
through the `_host` entry points, which stage them across PCIe inside the call.  PyTorch is used
for memory and streams only; all arithmetic happens in libhexb200.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import _lib
from ._lib import HEXB_DT_F16, HEXB_DT_F32, HEXB_DT_I32, check

_DT = {torch.float16: HEXB_DT_F16, torch.float32: HEXB_DT_F32}


def _dt(t: torch.Tensor) -> int:
    if t.dtype not in _DT:
        raise TypeError(f"unsupported dtype {t.dtype}: the kernels take float16 and float32")
    return _DT[t.dtype]


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(t: torch.Tensor) -> int:
    """The raw cudaStream_t of torch's current stream on the tensor's device."""
    if _raw_stream is not None:
        idx = t.device.index
        return _raw_stream(torch.cuda.current_device() if idx is None else idx)
    return torch.cuda.current_stream(t.device).cuda_stream


class _guard:
    """Makes `dev` the current CUDA device for the duration of a call; costs one query when it already is
    (the usual case), where torch.cuda.device() always pays a set/restore pair."""
    __slots__ = ("idx", "prev")

    def __init__(self, dev: torch.device):
        self.idx = dev.index
        self.prev = -1

    def __enter__(self):
        if self.idx is not None:
            cur = torch.cuda.current_device()
            if cur != self.idx:
                self.prev = cur
                torch.cuda.set_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


def _ptr(t):
    return None if t is None else t.data_ptr()


def _same_place(*ts):
    ts = [t for t in ts if t is not None]
    dev = ts[0].device
    for t in ts:
        if t.device != dev:
            raise ValueError("all tensors of one call must live on the same device")
    return dev


def _rows2d(t: torch.Tensor, what: str):
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise ValueError(f"{what}: expected a 2-D tensor with unit inner stride")
    return t.shape[0], t.shape[1], (t.stride(0) if t.shape[0] > 1 else max(t.shape[1], t.stride(0)))


def softmax(x: torch.Tensor, out: torch.Tensor) -> None:
    """out[r, :] = softmax(x[r, :]) (reference: test/python/triton/test_softmax.py:44-72)."""
    lib = _lib.load()
    dev = _same_place(x, out)
    rows, cols, xs = _rows2d(x, "x")
    r2, c2, ys = _rows2d(out, "out")
    if (rows, cols) != (r2, c2) or x.dtype != out.dtype:
        raise ValueError("softmax: x and out differ in shape or dtype")
    if dev.type == "cuda":
        with _guard(dev):
            fn = lib.hexb_softmax_f16 if x.dtype == torch.float16 else lib.hexb_softmax_f32
            _dt(x)
            check(fn(_ptr(x), _ptr(out), rows, cols, xs, ys, _stream(x)), "softmax")
    else:
        if not (x.is_contiguous() and out.is_contiguous()):
            raise ValueError("softmax: host tensors must be contiguous")
        check(lib.hexb_softmax_host(_dt(x), _ptr(x), _ptr(out), rows, cols), "softmax_host")


def layer_norm(x, out, weight, bias, mean=None, rstd=None, eps: float = 1e-5) -> None:
    """LayerNorm forward (reference: test/python/triton/test_layer_norm.py:42-82).

    mean / rstd, when given, receive the per-row statistics.  They may be float32 or x's dtype (the
    reference allocates them in x's dtype); the kernel produces float32.
    """
    lib = _lib.load()
    dev = _same_place(x, out, weight, bias, mean, rstd)
    rows, cols, xs = _rows2d(x, "x")
    r2, c2, ys = _rows2d(out, "out")
    if (rows, cols) != (r2, c2) or not (x.dtype == out.dtype == weight.dtype == bias.dtype):
        raise ValueError("layer_norm: shape or dtype mismatch")
    if weight.numel() != cols or bias.numel() != cols:
        raise ValueError("layer_norm: weight/bias must have NUM_COLS elements")
    stats = []
    for s in (mean, rstd):
        if s is None:
            stats.append((None, None))
        elif s.dtype == torch.float32 and s.is_contiguous():
            stats.append((s, None))
        else:
            stats.append((torch.empty(rows, dtype=torch.float32, device=dev), s))
    m32, r32 = stats[0][0], stats[1][0]
    if dev.type == "cuda":
        with _guard(dev):
            fn = lib.hexb_layer_norm_f16 if x.dtype == torch.float16 else lib.hexb_layer_norm_f32
            _dt(x)
            check(fn(_ptr(x), _ptr(out), _ptr(weight.contiguous()), _ptr(bias.contiguous()), _ptr(m32),
                     _ptr(r32), rows, cols, xs, ys, float(eps), _stream(x)), "layer_norm")
    else:
        if not (x.is_contiguous() and out.is_contiguous()):
            raise ValueError("layer_norm: host tensors must be contiguous")
        check(lib.hexb_layer_norm_host(_dt(x), _ptr(x), _ptr(out), _ptr(weight.contiguous()),
                                       _ptr(bias.contiguous()), _ptr(m32), _ptr(r32), rows, cols,
                                       float(eps)), "layer_norm_host")
    for tmp, dst in stats:
        if dst is not None:
            dst.copy_(tmp.to(dst.dtype).reshape(dst.shape))


def rms_norm(x, out, weight, eps: float = 1e-6) -> None:
    """RMSNorm forward (reference: test/python/triton/test_rms_norm.py:37-63)."""
    lib = _lib.load()
    dev = _same_place(x, out, weight)
    rows, cols, xs = _rows2d(x, "x")
    r2, c2, ys = _rows2d(out, "out")
    if (rows, cols) != (r2, c2) or not (x.dtype == out.dtype == weight.dtype):
        raise ValueError("rms_norm: shape or dtype mismatch")
    if weight.numel() != cols:
        raise ValueError("rms_norm: weight must have NUM_COLS elements")
    if dev.type == "cuda":
        with _guard(dev):
            fn = lib.hexb_rms_norm_f16 if x.dtype == torch.float16 else lib.hexb_rms_norm_f32
            _dt(x)
            check(fn(_ptr(x), _ptr(out), _ptr(weight.contiguous()), rows, cols, xs, ys, float(eps),
                     _stream(x)), "rms_norm")
    else:
        if not (x.is_contiguous() and out.is_contiguous()):
            raise ValueError("rms_norm: host tensors must be contiguous")
        check(lib.hexb_rms_norm_host(_dt(x), _ptr(x), _ptr(out), _ptr(weight.contiguous()), rows, cols,
                                     float(eps)), "rms_norm_host")


def matmul(a, b, c, residual=None) -> None:
    """c = a @ b (+ residual); a, b float16 row-major, c float16 or float32, fp32 accumulation.

    Reference: test/python/triton/test_matmul.py:35-70, docs/tutorials/triton/matmul_hexkl.md:61-97.
    """
    lib = _lib.load()
    dev = _same_place(a, b, c, residual)
    if a.dtype != torch.float16 or b.dtype != torch.float16:
        raise TypeError("matmul: A and B must be float16")
    M, K, lda = _rows2d(a, "A")
    K2, N, ldb = _rows2d(b, "B")
    M2, N2, ldc = _rows2d(c, "C")
    if K != K2 or M != M2 or N != N2:
        raise ValueError("matmul: shapes do not agree")
    if dev.type == "cuda":
        if residual is not None:
            if residual.dtype != torch.float16 or residual.shape != c.shape or residual.stride(0) != c.stride(0):
                raise ValueError("matmul: residual must be float16 with C's shape and leading dimension")
        with _guard(dev):
            check(lib.hexb_matmul_f16(_ptr(a), _ptr(b), _ptr(c), _ptr(residual), M, N, K, lda, ldb, ldc,
                                      _dt(c), _stream(a)), "matmul")
    else:
        if residual is not None:
            raise ValueError("matmul: residual is a device-path feature")
        if not (a.is_contiguous() and b.is_contiguous() and c.is_contiguous()):
            raise ValueError("matmul: host tensors must be contiguous")
        check(lib.hexb_matmul_f16_host(_ptr(a), _ptr(b), _ptr(c), M, N, K, _dt(c)), "matmul_host")


def matmul_nt(a, bt, c, residual=None) -> None:
    """c = a @ bt.T for a [M, K], bt [N, K] (a weight stored transposed), float16 CUDA tensors; c float16 or
    float32.  Reference: test/python/torch-mlir/test_hexkl_macro_matmul.py:24-28,51-69."""
    lib = _lib.load()
    if any(t is not None and t.device.type != "cuda" for t in (a, bt, c, residual)):
        return _stage(lambda a, bt, c, residual: matmul_nt(a, bt, c, residual), dict(a=a, bt=bt, c=c, residual=residual), ("c",))
    _same_place(a, bt, c, residual)
    if a.dtype != torch.float16 or bt.dtype != torch.float16:
        raise TypeError("matmul_nt: A and Bt must be float16")
    M, K, lda = _rows2d(a, "A")
    N, K2, ldb = _rows2d(bt, "Bt")
    M2, N2, ldc = _rows2d(c, "C")
    if K != K2 or M != M2 or N != N2:
        raise ValueError("matmul_nt: shapes do not agree")
    if residual is not None and (residual.dtype != torch.float16 or residual.shape != c.shape
                                 or residual.stride(0) != c.stride(0)):
        raise ValueError("matmul_nt: residual must be float16 with C's shape and leading dimension")
    with _guard(a.device):
        check(lib.hexb_matmul_f16_nt(_ptr(a), _ptr(bt), _ptr(c), _ptr(residual), M, N, K, lda, ldb, ldc, _dt(c),
                                     _stream(a)), "matmul_nt")


def linear(a, w, c, bias=None, residual=None, act: str = "none", w_transposed: bool = False) -> None:
    """c = act(a @ w + bias) + residual in one launch; w is [K, N], or [N, K] with w_transposed.
    act: "none" or "gelu_tanh".  Reference: the addmm / gelu / add chains of the GPT-2 graph,
    test/python/torch-mlir/gpt2lmheadmodel.py:143-169."""
    lib = _lib.load()
    if any(t is not None and t.device.type != "cuda" for t in (a, w, c, bias, residual)):
        res_is_c = residual is c
        tensors = dict(a=a, w=w, c=c, bias=bias, residual=None if res_is_c else residual)
        return _stage(lambda a, w, c, bias, residual: linear(a, w, c, bias, c if res_is_c else residual, act, w_transposed),
                      tensors, ("c",))
    _same_place(a, w, c, bias, residual)
    if a.dtype != torch.float16 or w.dtype != torch.float16:
        raise TypeError("linear: A and W must be float16")
    M, K, lda = _rows2d(a, "A")
    if w_transposed:
        N, K2, ldw = _rows2d(w, "W")
    else:
        K2, N, ldw = _rows2d(w, "W")
    M2, N2, ldc = _rows2d(c, "C")
    if K != K2 or M != M2 or N != N2:
        raise ValueError("linear: shapes do not agree")
    if bias is not None and (bias.dtype != torch.float16 or bias.shape != (N,) or not bias.is_contiguous()):
        raise ValueError("linear: bias must be a contiguous float16 [N] vector")
    if residual is not None and (residual.dtype != torch.float16 or residual.shape != c.shape
                                 or residual.stride(0) != c.stride(0)):
        raise ValueError("linear: residual must be float16 with C's shape and leading dimension")
    acts = {"none": 0, "gelu_tanh": 1}
    if act not in acts:
        raise ValueError(f"linear: unknown activation {act!r}")
    with _guard(a.device):
        check(lib.hexb_linear_f16(_ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(c), M, N, K, lda, ldw, ldc,
                                  int(bool(w_transposed)), acts[act], _dt(c), _stream(a)), "linear")


def embedding(wte, wpe, ids, out, check_ids: bool = False) -> None:
    """out[b, s, :] = wte[ids[b, s], :] + wpe[s, :] for float16 tables and int64 ids [batch, seq].

    The kernel writes a zero row for an id outside [0, vocab) and records HEXB_ERR_BAD_ARG in the
    device status word (read it with ``hexb200.device_status()``; a CUDA-graph replay has no other
    way to report it).  ``check_ids=True`` validates the ids first -- one device synchronisation --
    and raises IndexError as torch's own embedding lookup does."""
    lib = _lib.load()
    if check_ids and ids.numel():
        lo, hi = int(ids.min()), int(ids.max())
        if lo < 0 or hi >= wte.shape[0]:
            raise IndexError(f"embedding: token id {lo if lo < 0 else hi} is outside [0, {wte.shape[0]})")
    if any(t.device.type != "cuda" for t in (wte, wpe, ids, out)):
        return _stage(lambda wte, wpe, ids, out: embedding(wte, wpe, ids, out), dict(wte=wte, wpe=wpe, ids=ids, out=out),
                      ("out",))
    _same_place(wte, wpe, ids, out)
    if wte.dtype != torch.float16 or wpe.dtype != torch.float16 or out.dtype != torch.float16:
        raise TypeError("embedding: tables and output must be float16")
    if ids.dtype != torch.int64 or ids.dim() != 2:
        raise TypeError("embedding: ids must be an int64 [batch, seq] tensor")
    B, S = ids.shape
    V, Dm = wte.shape
    if wpe.shape[1] != Dm or out.shape != (B, S, Dm) or wpe.shape[0] < S:
        raise ValueError("embedding: shapes do not agree")
    if not all(t.is_contiguous() for t in (wte, wpe, ids, out)):
        raise ValueError("embedding: contiguous tensors expected")
    with _guard(wte.device):
        check(lib.hexb_embedding_f16(_ptr(wte), _ptr(wpe), _ptr(ids), _ptr(out), B * S, S, Dm, V, wpe.shape[0],
                                     _stream(wte)), "embedding")


def matmul_swiglu(a, b_gate_up, out) -> None:
    """out = silu(a @ b[:, :F]) * (a @ b[:, F:]) for a [M, K], b [K, 2F], out [M, F]; float16 CUDA tensors."""
    lib = _lib.load()
    _same_place(a, b_gate_up, out)
    if not (a.dtype == b_gate_up.dtype == out.dtype == torch.float16):
        raise TypeError("matmul_swiglu: float16 tensors expected")
    M, K, lda = _rows2d(a, "A")
    K2, F2, ldb = _rows2d(b_gate_up, "B")
    M2, Fo, ldo = _rows2d(out, "out")
    if K != K2 or M != M2 or F2 != 2 * Fo:
        raise ValueError("matmul_swiglu: shapes do not agree")
    with _guard(a.device):
        check(lib.hexb_matmul_swiglu_f16(_ptr(a), _ptr(b_gate_up), _ptr(out), M, Fo, K, lda, ldb, ldo, _stream(a)),
              "matmul_swiglu")


def hexkl_matmul_f16f16_f32(n_row, n_col, n_inner, out, act, w) -> None:
    """The HexKL runtime symbol, same argument order (bin/runtime/include/HexKLAPI.h:16-21); device tensors."""
    lib = _lib.load()
    with _guard(out.device):
        torch.cuda.current_stream().synchronize()  # the symbol runs on the legacy default stream
        check(lib.hexkl_matmul_f16f16_f32(n_row, n_col, n_inner, _ptr(out), _ptr(act), _ptr(w)), "hexkl_matmul")
        torch.cuda.synchronize()


def attention(q, k, v, out, sm_scale=None, causal: bool = False) -> None:
    """out = softmax(q k^T * sm_scale [+ causal mask]) v for [Z, H, N_CTX, D] tensors.

    Reference: test/python/triton/test_flash_attention.py:37-168.  Any strides with a unit
    innermost stride are accepted on the device path.
    """
    lib = _lib.load()
    dev = _same_place(q, k, v, out)
    if not (q.dim() == k.dim() == v.dim() == out.dim() == 4):
        raise ValueError("attention: expected [Z, H, N_CTX, D] tensors")
    if not (q.shape == k.shape == v.shape == out.shape) or not (q.dtype == k.dtype == v.dtype == out.dtype):
        raise ValueError("attention: q, k, v, out must agree in shape and dtype")
    Z, H, N, D = q.shape
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    dt = _dt(q)
    if dev.type == "cuda":
        strides = []
        for t in (q, k, v, out):
            if D > 1 and t.stride(3) != 1:
                raise ValueError("attention: innermost stride must be 1")
            strides += [t.stride(0), t.stride(1), t.stride(2)]
        arr = (C.c_int64 * 12)(*strides)
        with _guard(dev):
            fn = lib.hexb_attention_fwd_f16 if dt == HEXB_DT_F16 else lib.hexb_attention_fwd_f32
            check(fn(_ptr(q), _ptr(k), _ptr(v), _ptr(out), Z, H, N, D, arr, float(sm_scale), int(bool(causal)),
                     _stream(q)), "attention")
    else:
        if not all(t.is_contiguous() for t in (q, k, v, out)):
            raise ValueError("attention: host tensors must be contiguous")
        check(lib.hexb_attention_fwd_host(dt, _ptr(q), _ptr(k), _ptr(v), _ptr(out), Z, H, N, D,
                                          float(sm_scale), int(bool(causal))), "attention_host")


def attention_ex(q, k, v, out, mask=None, sm_scale=None, causal: bool = False) -> None:
    """out = softmax(q k^T * sm_scale + mask) v on CUDA tensors.

    q, out: [Z, H, N_Q, D]; k, v: [Z, H, N_KV, D]; float16 inputs with a float16 or float32 `out`
    (the fp16-in / fp32-out form of test/python/mlir/hexkl_attention/input.mlir:5), or all float32.
    `mask` is additive, float16 or float32, and broadcastable to [Z, H, N_Q, N_KV] with a unit
    innermost stride; it enters before the row maximum as in the lowering of tm_tensor.attention
    (qcom_hexagon_backend/lib/Transforms/LowerTmTensor.cpp:126-160).
    """
    lib = _lib.load()
    if any(t is not None and t.device.type != "cuda" for t in (q, k, v, out, mask)):
        return _stage(lambda q, k, v, out, mask: attention_ex(q, k, v, out, mask, sm_scale, causal),
                      dict(q=q, k=k, v=v, out=out, mask=mask), ("out",))
    dev = _same_place(q, k, v, out, mask)
    if not (q.dim() == k.dim() == v.dim() == out.dim() == 4):
        raise ValueError("attention_ex: expected [Z, H, N, D] tensors")
    Z, H, NQ, D = q.shape
    NKV = k.shape[2]
    if k.shape != (Z, H, NKV, D) or v.shape != k.shape or out.shape != q.shape:
        raise ValueError("attention_ex: shapes do not agree")
    if not (q.dtype == k.dtype == v.dtype):
        raise TypeError("attention_ex: q, k, v must share a dtype")
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    d = _lib.AttentionDesc()
    d.Q, d.K, d.V, d.Out = _ptr(q), _ptr(k), _ptr(v), _ptr(out)
    d.Z, d.H, d.N_Q, d.N_KV, d.D = Z, H, NQ, NKV, D
    strides = []
    for t in (q, k, v, out):
        if D > 1 and t.stride(3) != 1:
            raise ValueError("attention_ex: innermost stride must be 1")
        strides += [t.stride(0), t.stride(1), t.stride(2)]
    d.strides = (C.c_int64 * 12)(*strides)
    d.in_dtype, d.out_dtype = _dt(q), _dt(out)
    if mask is not None:
        m = mask
        while m.dim() < 4:
            m = m.unsqueeze(0)
        if m.shape[3] != NKV or (NKV > 1 and m.stride(3) != 1):
            raise ValueError("attention_ex: the mask's last dimension must be N_KV with stride 1")
        m = m.expand(Z, H, NQ, NKV)
        d.mask = _ptr(m)
        d.mask_strides = (C.c_int64 * 3)(m.stride(0), m.stride(1), m.stride(2))
        d.mask_dtype = _dt(m)
    else:
        d.mask = None
        d.mask_dtype = 0
    d.sm_scale = float(sm_scale)
    d.causal = int(bool(causal))
    with _guard(dev):
        check(lib.hexb_attention_fwd_ex(C.byref(d), _stream(q)), "attention_ex")


def sdpa_masked(query, key, value, mask, out) -> None:
    """tm_tensor.attention ins(Q, K, V, mask) outs(out): rank-3 operands [batch, seq, d], additive mask
    [batch, seq_q, seq_kv], scale 1/sqrt(d)
    (qcom_hexagon_backend/include/hexagon/Dialect/TmTensor/IR/TmTensorOps.td:27-55)."""
    if not (query.dim() == key.dim() == value.dim() == out.dim() == mask.dim() == 3):
        raise ValueError("sdpa_masked: rank-3 operands expected")
    attention_ex(query.unsqueeze(1), key.unsqueeze(1), value.unsqueeze(1), out.unsqueeze(1), mask=mask.unsqueeze(1))


def silu(x, out) -> None:
    """out = x / (1 + exp(-x)) (reference: test/python/triton/test_silu.py:38-52)."""
    lib = _lib.load()
    dev = _same_place(x, out)
    if x.shape != out.shape or x.dtype != out.dtype or not (x.is_contiguous() and out.is_contiguous()):
        raise ValueError("silu: x and out must be contiguous with equal shape and dtype")
    host = dev.type != "cuda"
    xd, od = (x.cuda(), torch.empty_like(x, device="cuda")) if host else (x, out)
    with _guard(xd.device):
        fn = lib.hexb_silu_f16 if _dt(x) == HEXB_DT_F16 else lib.hexb_silu_f32
        check(fn(_ptr(xd), _ptr(od), x.numel(), _stream(xd)), "silu")
    if host:
        out.copy_(od)


def swiglu(gate_up, out) -> None:
    """out[r, c] = silu(gate_up[r, c]) * gate_up[r, cols + c]; float16 device tensors."""
    lib = _lib.load()
    _same_place(gate_up, out)
    rows, cols2 = gate_up.shape
    if gate_up.dtype != torch.float16 or out.dtype != torch.float16 or out.shape != (rows, cols2 // 2):
        raise ValueError("swiglu: expected float16 [rows, 2*cols] -> [rows, cols]")
    if not (gate_up.is_contiguous() and out.is_contiguous()):
        raise ValueError("swiglu: tensors must be contiguous")
    with _guard(gate_up.device):
        check(lib.hexb_swiglu_f16(_ptr(gate_up), _ptr(out), rows, cols2 // 2, _stream(gate_up)), "swiglu")


UNARY_OPS = {"gelu_tanh": 1, "cos": 2, "sin": 3, "rsqrt": 4}
BINARY_OPS = {"add": 1, "sub": 2, "mul": 3, "div": 4}


def _on_device(*ts):
    """CUDA tensors pass through; CPU tensors are staged (torch moves the bytes, nothing else)."""
    host = ts[0].device.type != "cuda"
    return host, [t.cuda() if host else t for t in ts]


def _stage(fn, tensors: dict, outputs: tuple):
    """Runs fn(**tensors) with every CPU tensor staged through the current CUDA device (torch moves the
    bytes, nothing else) and copies the tensors named in `outputs` back; CUDA tensors pass through."""
    host = any(t is not None and t.device.type != "cuda" for t in tensors.values())
    if not host:
        return fn(**tensors)
    staged = {k: (None if t is None else (t.cuda() if t.device.type != "cuda" else t)) for k, t in tensors.items()}
    fn(**staged)
    for k in outputs:
        if tensors[k].device.type != "cuda":
            tensors[k].copy_(staged[k])


def unary(op: str, x, out) -> None:
    """out = op(x), op in gelu_tanh / cos / sin / rsqrt (reference: test_gelu.py:25-54,
    test_math_ops.py:24-37, test_rsqrt.py:19-24)."""
    lib = _lib.load()
    _same_place(x, out)
    if x.shape != out.shape or x.dtype != out.dtype or not (x.is_contiguous() and out.is_contiguous()):
        raise ValueError("unary: x and out must be contiguous with equal shape and dtype")
    host, (xd,) = _on_device(x)
    od = torch.empty_like(xd) if host else out
    with _guard(xd.device):
        check(lib.hexb_unary(UNARY_OPS[op], _dt(x), _ptr(xd), _ptr(od), x.numel(), _stream(xd)), op)
    if host:
        out.copy_(od)


def binary(op: str, a, b, out) -> None:
    """out = a op b, op in add / sub / mul / div (reference: test_vec_add.py:19-25,
    test_vec_add_2d.py:21-56, test_vec_div_2d.py:20-55)."""
    lib = _lib.load()
    _same_place(a, b, out)
    if not (a.shape == b.shape == out.shape) or not (a.dtype == b.dtype == out.dtype):
        raise ValueError("binary: a, b and out must agree in shape and dtype")
    if not (a.is_contiguous() and b.is_contiguous() and out.is_contiguous()):
        raise ValueError("binary: tensors must be contiguous")
    host, (ad, bd) = _on_device(a, b)
    od = torch.empty_like(ad) if host else out
    with _guard(ad.device):
        check(lib.hexb_binary(BINARY_OPS[op], _dt(a), _ptr(ad), _ptr(bd), _ptr(od), a.numel(), _stream(ad)), op)
    if host:
        out.copy_(od)


def iota(out) -> None:
    """out[i] = i (reference: flatten_pid over a multi-dimensional grid, test_multidim_grid.py:21-37)."""
    lib = _lib.load()
    if not out.is_contiguous():
        raise ValueError("iota: contiguous tensor expected")
    host = out.device.type != "cuda"
    od = torch.empty(out.shape, dtype=out.dtype, device="cuda") if host else out
    with _guard(od.device):
        check(lib.hexb_iota(_dt(out), _ptr(od), out.numel(), _stream(od)), "iota")
    if host:
        out.copy_(od)


def vec_sum(x, out) -> None:
    """out[0] = sum(x) with fp32 accumulation in a fixed order (reference: test_sum.py:31-36)."""
    lib = _lib.load()
    _same_place(x, out)
    if x.dtype != out.dtype or out.numel() < 1 or not x.is_contiguous():
        raise ValueError("sum: out must hold one element of x's dtype, x contiguous")
    host, (xd,) = _on_device(x)
    od = torch.empty(1, dtype=x.dtype, device=xd.device) if host else out
    with _guard(xd.device):
        check(lib.hexb_sum(_dt(x), _ptr(xd), _ptr(od), x.numel(), _stream(xd)), "sum")
    if host:
        out.view(-1)[:1].copy_(od)


def cumsum(x, out, axis: int = -1, reverse: bool = False) -> None:
    """out = inclusive prefix sum of x along `axis` (from the far end when `reverse`), contiguous CUDA tensors
    of float32, float16 (fp32 accumulation) or int32.  Reference: ttx.cumsum / ttx.scan with an addition body
    (qcom_hexagon_backend/include/hexagon/Dialect/TTX/IR/TTXOps.td:25-75, lib/Transforms/LowerTTX.cpp:75-300)."""
    lib = _lib.load()
    if x.device.type != "cuda" or out.device.type != "cuda":
        return _stage(lambda x, out: cumsum(x, out, axis, reverse), dict(x=x, out=out), ("out",))
    dev = _same_place(x, out)
    if x.shape != out.shape or x.dtype != out.dtype or not (x.is_contiguous() and out.is_contiguous()):
        raise ValueError("cumsum: x and out must be contiguous with equal shape and dtype")
    if x.dim() == 0:
        raise ValueError("cumsum: a scalar has no axis")
    axis = axis % x.dim()
    dt = {torch.float16: HEXB_DT_F16, torch.float32: HEXB_DT_F32, torch.int32: HEXB_DT_I32}.get(x.dtype)
    if dt is None:
        raise TypeError(f"cumsum: unsupported dtype {x.dtype}")
    outer = math.prod(x.shape[:axis])
    inner = math.prod(x.shape[axis + 1:])
    with _guard(dev):
        check(lib.hexb_cumsum(dt, _ptr(x), _ptr(out), outer, x.shape[axis], inner, int(bool(reverse)), _stream(x)),
              "cumsum")


def rope(x, out, theta: float = 10000.0) -> None:
    """Interleaved-pair rotary embedding of a [B, L, H, D] tensor (reference: test_rope.py:98-190)."""
    lib = _lib.load()
    _same_place(x, out)
    if x.dim() != 4 or x.shape != out.shape or x.dtype != out.dtype:
        raise ValueError("rope: expected [B, L, H, D] tensors of equal shape and dtype")
    host, (xd,) = _on_device(x)
    od = torch.empty_like(xd) if host else out
    if xd.stride(3) != 1 or od.stride(3) != 1:
        raise ValueError("rope: innermost stride must be 1")
    B, L, H, D = x.shape
    xs = (C.c_int64 * 3)(xd.stride(0), xd.stride(1), xd.stride(2))
    os_ = (C.c_int64 * 3)(od.stride(0), od.stride(1), od.stride(2))
    with _guard(xd.device):
        check(lib.hexb_rope(_dt(x), _ptr(xd), _ptr(od), B, L, H, D, xs, os_, float(theta), _stream(xd)), "rope")
    if host:
        out.copy_(od)


class DecoderStack:
    """The decoder-only block stack on one GPU: holds the weight pointer tables and the workspace.

    weights: list (one dict per layer) with float16 CUDA tensors wqkv [d, 3d], wo [d, d],
    wgu [d, 2*d_ff], wd [d_ff, d], g1 [d], g2 [d].
    """

    def __init__(self, weights, n_heads: int, head_dim: int, d_ff: int, batch: int, seq: int,
                 rms_eps: float = 1e-6):
        self.lib = _lib.load()
        self.weights = weights
        d_model = n_heads * head_dim
        self.cfg = _lib.DecoderConfig(len(weights), d_model, n_heads, head_dim, d_ff, batch, seq, rms_eps)
        self.device = weights[0]["wqkv"].device if weights else torch.device("cuda")
        n = len(weights)
        self._tables = {}
        for name in ("wqkv", "wo", "wgu", "wd", "g1", "g2"):
            for w in weights:
                t = w[name]
                if t.dtype != torch.float16 or not t.is_contiguous() or t.device != self.device:
                    raise ValueError(f"decoder weight {name}: float16 contiguous CUDA tensor expected")
            self._tables[name] = (C.c_void_p * max(n, 1))(*[w[name].data_ptr() for w in weights])
        self.cweights = _lib.DecoderWeights(*[C.cast(self._tables[k], C.POINTER(C.c_void_p))
                                              for k in ("wqkv", "wo", "wgu", "wd", "g1", "g2")])
        self.ws_bytes = self.lib.hexb_decoder_workspace_bytes(C.byref(self.cfg))
        self.workspace = torch.empty(max(self.ws_bytes, 256), dtype=torch.uint8, device=self.device)

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> None:
        """x, out: float16 CUDA [batch*seq, d_model] (or [batch, seq, d_model]) contiguous."""
        if x.dtype != torch.float16 or out.dtype != torch.float16 or not (x.is_contiguous() and out.is_contiguous()):
            raise ValueError("decoder: float16 contiguous tensors expected")
        if x.numel() != self.cfg.batch * self.cfg.seq * self.cfg.d_model or out.numel() != x.numel():
            raise ValueError("decoder: x/out size does not match the configuration")
        with _guard(self.device):
            check(self.lib.hexb_decoder_forward_f16(C.byref(self.cfg), C.byref(self.cweights), _ptr(x), _ptr(out),
                                                    _ptr(self.workspace), self.ws_bytes, _stream(x)), "decoder_forward")
