"""The reference launcher's on-disk formats and timing habit, for tooling that consumes them.

* raw tensor files: the generated wrapper dumps each output as
  ``[u32 dtype id][i64 rank][i64 shape[rank]][payload]`` (test/utils/dsp/include/tensor.h:236-260) and
  the Python side parses it back (qcom_hexagon_backend/backend/hexagon_executor.py:153-169); inputs
  (``<kernel>_t{i}.raw``) are the bare payload (tensor.h:218-234).  dtype ids: tensor.h:26-38.
* ``Test_Info{Name, Result, Perf, Units}`` blocks written to perf.txt
  (test/utils/dsp/include/test_report.h:43-66).
* ``benchmark_time_us``: the average of ``iterations`` back-to-back calls
  (test/utils/dsp/include/hexagon_benchmark.h:20-29) -- here timed with CUDA events on the stream.
"""
from __future__ import annotations

import struct

import numpy as np
import torch

# tensor.h:26-38
DTYPE_IDS = {torch.bool: 0, torch.float16: 1, torch.float32: 2, torch.float64: 3, torch.int8: 4, torch.int16: 5,
             torch.int32: 6, torch.int64: 7, torch.uint8: 8, torch.uint16: 9, torch.uint32: 10}
ID_DTYPES = {v: k for k, v in DTYPE_IDS.items()}


def _np_view(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.uint16, torch.uint32):
        return t.view(torch.int16 if t.dtype == torch.uint16 else torch.int32).numpy()
    return t.numpy()


def dump_tensor(path: str, t: torch.Tensor) -> None:
    """Writes ``t`` in the wrapper's output format (dtype id, rank, shape, payload)."""
    if t.dtype not in DTYPE_IDS:
        raise TypeError(f"dtype {t.dtype} has no id in the reference's tensor file format")
    with open(path, "wb") as f:
        f.write(struct.pack("I", DTYPE_IDS[t.dtype]))
        f.write(struct.pack("q", t.dim()))
        for s in t.shape:
            f.write(struct.pack("q", s))
        f.write(_np_view(t).tobytes())


def load_tensor(path: str) -> torch.Tensor:
    """Reads a file written by ``dump_tensor`` (or by the reference's wrapper)."""
    with open(path, "rb") as f:
        (dt_id,) = struct.unpack("I", f.read(4))
        (rank,) = struct.unpack("q", f.read(8))
        if dt_id not in ID_DTYPES or rank < 0 or rank > 64:
            raise ValueError(f"{path}: not a tensor file (dtype id {dt_id}, rank {rank})")
        shape = [struct.unpack("q", f.read(8))[0] for _ in range(rank)]
        data = f.read()
    dtype = ID_DTYPES[dt_id]
    n = int(np.prod(shape)) if shape else 1
    esz = torch.empty(0, dtype=dtype).element_size()
    if len(data) != n * esz:
        raise ValueError(f"{path}: payload is {len(data)} bytes, shape {shape} needs {n * esz}")
    if n == 0:
        return torch.empty(shape, dtype=dtype)
    return torch.frombuffer(bytearray(data), dtype=dtype).reshape(shape).clone()


def dump_input(path: str, t: torch.Tensor) -> None:
    """Writes the bare payload, the form of the launcher's ``<kernel>_t{i}.raw`` input files."""
    with open(path, "wb") as f:
        f.write(_np_view(t).tobytes())


def load_input(path: str, dtype: torch.dtype, shape) -> torch.Tensor:
    with open(path, "rb") as f:
        data = f.read()
    return torch.frombuffer(bytearray(data), dtype=dtype).reshape(tuple(shape)).clone()


class TestReport:
    """``Test_Info`` block of the reference's device tests (test_report.h:35-67)."""

    __test__ = False  # not a pytest class
    RESULTS = ("Pass", "Fail", "Unknown")

    def __init__(self, name: str, perf: float, units: str = "us", result: str = "Unknown"):
        if result not in self.RESULTS:
            raise ValueError(f"result must be one of {self.RESULTS}")
        self.name, self.perf, self.units, self.result = name, float(perf), units, result

    def text(self) -> str:
        return ("Test_Info: {\n" f"\tName:{self.name}\n" f"\tResult:{self.result}\n" f"\tPerf:{self.perf:f}\n"
                f"\tUnits:{self.units}\n" "}\n")

    def save(self, path: str) -> None:
        with open(path, "w") as f:
            f.write(self.text())

    @classmethod
    def parse(cls, text: str) -> "TestReport":
        fields = {}
        for line in text.splitlines():
            line = line.strip()
            if ":" in line and not line.startswith("Test_Info"):
                k, v = line.split(":", 1)
                fields[k] = v
        return cls(fields["Name"], float(fields["Perf"]), fields["Units"], fields["Result"])


def benchmark_time_us(iterations: int, op) -> float:
    """Average device time of ``iterations`` back-to-back calls of ``op`` on the current CUDA stream,
    in microseconds (the reference averages wall-clock microseconds on the DSP)."""
    if iterations < 1:
        raise ValueError("iterations must be >= 1")
    op()  # not timed: first-call set-up
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iterations):
        op()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iterations
