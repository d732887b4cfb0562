"""Generates the golden fixtures in this directory from the reference's own Triton kernels.

Runs only where a checkout of the reference is present (its location: $HEXAGON_MLIR_REF).
The reference's test modules are imported unmodified with

  * TRITON_INTERPRET=1, so the @triton.jit kernels execute in Triton's NumPy interpreter on CPU,
  * a stub ``triton.backends.qcom_hexagon_backend.driver.HexagonDriver`` and a no-op
    ``triton.runtime.driver.set_active`` (the real ones need the Hexagon toolchain),
  * ``parameterize_func_name`` (a rename of the kernel per dtype) made the identity, because the
    interpreter finds the kernel by its source name,
  * ``torch.rand`` seeded and recorded, and ``torch.allclose`` / ``torch.testing.assert_close`` wrapped to capture the kernel's
    output and the torch reference the test compares it with.

Each fixture ``<case>.npz`` holds the recorded inputs (in0, in1, ...), ``output`` (what the
reference kernel produced) and ``expected`` (the torch value the reference test asserted against).
Usage: ``HEXAGON_MLIR_REF=<checkout of qualcomm/hexagon-mlir> python tests/golden/make_golden.py``.
"""
import importlib
import os
import sys
import types
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"
import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton  # noqa: E402

if not os.environ.get("HEXAGON_MLIR_REF"):
    raise SystemExit("set HEXAGON_MLIR_REF to a checkout of qualcomm/hexagon-mlir")
REF = Path(os.environ["HEXAGON_MLIR_REF"])
OUT = Path(__file__).resolve().parent


def _stub_backend():
    pkg = types.ModuleType("triton.backends.qcom_hexagon_backend")
    drv = types.ModuleType("triton.backends.qcom_hexagon_backend.driver")

    class HexagonDriver:  # the tests only construct it
        pass

    drv.HexagonDriver = HexagonDriver
    sys.modules[pkg.__name__] = pkg
    sys.modules[drv.__name__] = drv
    triton.runtime.driver.set_active = lambda *_a, **_k: None


class Recorder:
    """Records torch.rand results and the operands of torch.allclose while a reference test runs."""

    def __init__(self, seed):
        self.inputs, self.output, self.expected = [], None, None
        self.pairs = []  # every (output, expected) the test compared, in order
        self.seed = seed

    def __enter__(self):
        self._rand, self._allclose = torch.rand, torch.allclose
        self._randn, self._linspace = torch.randn, torch.linspace
        torch.manual_seed(self.seed)

        def recording(fn):
            def wrapped(*a, **k):
                t = fn(*a, **k)
                self.inputs.append(t.clone())
                return t
            return wrapped

        def allclose(a, b, *rest, **k):
            self.output, self.expected = a.clone(), torch.as_tensor(b).clone()
            self.pairs.append((self.output, self.expected))
            return self._allclose(a, b, *rest, **k)

        torch.rand, torch.randn, torch.linspace = recording(self._rand), recording(self._randn), recording(self._linspace)
        torch.allclose = allclose
        self._assert_close = torch.testing.assert_close

        def assert_close(a, b, *rest, **k):   # test_rope.py compares with torch.testing.assert_close
            self.output, self.expected = a.clone(), torch.as_tensor(b).clone()
            self.pairs.append((self.output, self.expected))
            return self._assert_close(a, b, *rest, **k)

        torch.testing.assert_close = assert_close
        return self

    def __exit__(self, *exc):
        torch.rand, torch.allclose = self._rand, self._allclose
        torch.randn, torch.linspace = self._randn, self._linspace
        torch.testing.assert_close = self._assert_close

    def save(self, name):
        arrays = {f"in{i}": t.numpy() for i, t in enumerate(self.inputs)}
        arrays["output"] = self.output.numpy()
        arrays["expected"] = self.expected.numpy()
        if len(self.pairs) > 1:
            for i, (o, e) in enumerate(self.pairs):
                arrays[f"output{i}"], arrays[f"expected{i}"] = o.numpy(), e.numpy()
        np.savez_compressed(OUT / f"{name}.npz", **arrays)
        err = float((self.output.float() - self.expected.float()).abs().max())
        print(f"{name}: {len(self.inputs)} inputs, output {tuple(self.output.shape)} {self.output.dtype}, "
              f"max |kernel - torch| = {err:.3e}")


def main():
    if not REF.exists():
        raise SystemExit(f"{REF} not found: fixtures can only be regenerated next to the reference checkout")
    _stub_backend()
    sys.path.insert(0, str(REF / "test"))
    # The interpreter re-parses the kernel source and looks the function up by its source name, so
    # the dtype suffix that parameterize_func_name appends to __name__ is left out here; the
    # suffix only renames the kernel.
    pkg = importlib.import_module("python")
    pkg.parameterize_func_name = lambda *_p: (lambda f: f)
    mod = lambda n: importlib.import_module(f"python.triton.{n}")

    sm = mod("test_softmax")
    for dt, tag in ((torch.float32, "f32"), (torch.float16, "f16")):
        with Recorder(11) as r:
            sm.test_softmax(dt)
        r.save(f"softmax_128x128_{tag}")

    osm = mod("test_online_softmax")
    with Recorder(12) as r:
        osm.test_online_softmax(4)
    r.save("online_softmax_128x128_f32")

    ln = mod("test_layer_norm")
    with Recorder(13) as r:
        ln.test_layer_norm(1024, 4, torch.float32)
    r.save("layer_norm_27x1024_f32")

    rn = mod("test_rms_norm")
    for dt, tag in ((torch.float32, "f32"), (torch.float16, "f16")):
        with Recorder(14) as r:
            rn.test_rms_norm(4, dt)
        r.save(f"rms_norm_{rn.NUM_ROWS}x{rn.NUM_COLS}_{tag}")

    mm = mod("test_matmul")
    with Recorder(15) as r:
        mm.test_matmul(256, 128, 64)
    r.save("matmul_256x128x64_f16")

    fa = mod("test_flash_attention")
    fa.N_CTX, fa.BLOCK_M = 256, 64  # module-level shape constants of the test; same kernel, smaller tensors
    fa.stride_0, fa.stride_1 = fa.H * 256 * fa.D_HEAD, 256 * fa.D_HEAD
    with Recorder(16) as r:
        fa.test_flash_attention()
    r.save("flash_attention_1x1x256x64_f32")

    si = mod("test_silu")
    for dt, tag in ((torch.float32, "f32"), (torch.float16, "f16")):
        with Recorder(17) as r:
            si.test_silu(16384, 4, dt, False, False)
        r.save(f"silu_16384_{tag}")

    ge = mod("test_gelu")
    for dt, tag in ((torch.float32, "f32"), (torch.float16, "f16")):
        with Recorder(18) as r:
            ge.test_gelu(16384, 4, dt, True)
        r.save(f"gelu_16384_{tag}")

    ro = mod("test_rope")
    for dt, tag in ((torch.float32, "f32"), (torch.float16, "f16")):
        with Recorder(19) as r:
            ro.test_rope(4, dt)
        r.save(f"rope_{ro.BATCH_SIZE}x{ro.SEQ_LEN}x{ro.N_HEADS}x{ro.N_FEATURES}_{tag}")

    su = mod("test_sum")
    with Recorder(20) as r:
        su.test_vec_add(16384, torch.float32)   # the sum test (its function is named test_vec_add)
    r.save("sum_16384_f32")

    va = mod("test_vec_add")
    va.BLOCK_SIZE = 4096                         # module-level size constant of the test; same kernel
    with Recorder(21) as r:
        va.test_vec_add()
    r.save("vec_add_f32")

    vd = mod("test_vec_div_2d")
    vd.N_ROWS, vd.N_COLUMNS = 8, 512             # module-level shape constants of the test; same kernel
    with Recorder(22) as r:
        vd.test_vec_div()
    r.save("vec_div_2d_f32")

    mo = mod("test_math_ops")
    with Recorder(23) as r:
        mo.test_math_ops()                       # two comparisons: cos, then sin
    r.save("math_ops_cos_sin_f32")
    # test_rsqrt.py calls libdevice.rsqrt, which Triton's interpreter cannot execute: no fixture;
    # the oracle for rsqrt is torch.rsqrt, the value that test asserts against.


if __name__ == "__main__":
    main()
