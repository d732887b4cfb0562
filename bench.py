#!/usr/bin/env python
"""Benchmark of the hexb200 hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of the hot path over one batch of seeded synthetic input.  The headline workload
is LayerNorm fp16 [16384 x 4096] (the benchmark's second configuration, the bandwidth-bound one the
HBM GB/s metric is quoted on); `--workload` selects softmax / gemm / attention / decoder (the benchmark's
other configurations) or gpt2 (the reference's two-layer GPT-2 test) instead.  Rank 0 prints ONE JSON
line.  The default run also measures the other configurations and lists them, compactly, under
"workloads" at the end of the line (device value, fraction of the measured peak, end-to-end value and,
at N = 1, the CPU baseline of each).

Timing: W untimed steps; the K steps are captured once into a CUDA graph; the timed region is R >= 9
back-to-back replays of it ("windows", each exactly K steps between two CUDA events on the launching
stream, R chosen so that the region lasts >= 50 ms), bracketed by a barrier and a synchronize on both
sides.  `ms_per_step` is the median window / K after taking, per window, the maximum over ranks.

With N > 1 (launched by torch.distributed.run, one rank per GPU over NCCL):
  * `value` is weak scaling: every rank runs the full-size configuration on its own GPU (independent
    rows / (batch, head) pairs / sequences, no data-path collective);
  * "strong" holds the partitioned form of each configuration: every rank takes its block of the
    configured tensor (hexb200.dist.partition), runs the kernels on it, the all-gather of the output
    blocks over NCCL is timed apart, and rank 0 compares sampled units of the gathered tensor with the
    CPU oracle (untimed).

`--impl reference` times the CPU implementation of the same path (the PyTorch CPU eager calls the
reference's tests compare against) on the host cores, on a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "HBM GB/s (softmax/LN) & TFLOP/s (GEMM/attn) vs roofline at 1/2/4/8 B200"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# ncu `dram__bytes_read.sum + dram__bytes_write.sum` per launch of the dominant kernel, copied from
# the committed summaries under profiles/ (bytes; output still dirty in L2 at kernel end is not in it).
# The timed run does not observe these: "traffic_source" in the JSON line says so.
NCU_TRAFFIC = {"layernorm": 212.33e6, "softmax": 33.98e6, "gemm": 87.44e6, "attention": 520.84e6, "decoder": None}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["_source"] = "measured"
        return p
    p = dict(FALLBACK_PEAKS)
    p["_source"] = "fallback"
    return p


# ---------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while a timed region runs."""

    NAMES = {0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
             0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
             0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def __init__(self, index: int):
        self.samples = []  # (t, sm_mhz, reasons_bitmask)
        self.max_mhz = None
        self._stop = threading.Event()
        self._thr = None
        self.ok = False
        try:
            import pynvml

            self.nv = pynvml
            pynvml.nvmlInit()
            # LOCAL_RANK indexes CUDA_VISIBLE_DEVICES; map through the UUID torch reports
            uuid = str(torch.cuda.get_device_properties(index).uuid)
            self.h = None
            for i in range(pynvml.nvmlDeviceGetCount()):
                h = pynvml.nvmlDeviceGetHandleByIndex(i)
                u = pynvml.nvmlDeviceGetUUID(h)
                u = u.decode() if isinstance(u, bytes) else u
                if uuid in u:
                    self.h = h
            if self.h is None:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                rs = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(
                    nv, "nvmlDeviceGetCurrentClocksEventReasons") else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((time.perf_counter(), mhz, rs))
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self.ok and self._thr is None:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()

    def stop(self):
        if self._thr:
            self._stop.set()
            self._thr.join()

    def summary(self, t0, t1):
        """Clock record of the samples taken between t0 and t1 (time.perf_counter values)."""
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0, "window": "none"}
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        window = "timed"
        if len(inside) < 3:
            inside, window = [s for s in self.samples if s[0] <= t1][-8:] or self.samples, "timed+before"
        mhz = sorted(s[1] for s in inside)
        bits = 0
        for s in inside:
            bits |= s[2]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz,
                "reasons": [n for b, n in self.NAMES.items() if bits & b], "samples": len(inside), "window": window}


# ---------------------------------------------------------------------------- workloads
class Workload:
    """One configuration: device buffers, a `step()` that launches the hot path, and its accounting.

    `shard=(world, rank)` builds the rank's block of the configuration (hexb200.dist.partition) instead
    of the whole: the partitioned multi-GPU form.  `host` always holds the whole seeded inputs.
    """

    name = ""
    unit = ""
    bound = ""
    dtype = ""
    launches_per_step = 1
    default_steps = 20
    strong_steps = 64

    def step(self, i: int):
        raise NotImplementedError

    def work_per_step(self) -> float:  # algorithmic bytes (hbm) or flops (tensor) of what this object runs
        raise NotImplementedError

    def local_output(self) -> torch.Tensor:  # the (shard's) output with the partition units along dimension 0
        raise NotImplementedError

    def host_inputs(self) -> dict:  # operand names of hexb200.dist.PARTITIONS[name] -> whole host tensors
        raise NotImplementedError


def _cut(name, inputs, shard):
    from hexb200 import dist

    if shard is None:
        return {k: dist.units_view(name, v) if k in dist.PARTITIONS[name][1] else v for k, v in inputs.items()}
    return dist.partition(name, inputs, shard[0], shard[1])


class LayerNormWL(Workload):
    name, unit, bound, dtype = "layernorm", "GB/s", "hbm", "f16"
    ROWS, COLS, SETS = 16384, 4096, 3
    default_steps, strong_steps = 20, 128

    def __init__(self, dev, shard=None):
        from hexb200 import ops, synth

        self.ops = ops
        x, w, b = synth.make_layer_norm_inputs(self.ROWS, self.COLS)
        self.host = (x, w, b)
        loc = _cut(self.name, self.host_inputs(), shard)
        self.rows = loc["x"].shape[0]
        self.w, self.b = w.to(dev), b.to(dev)
        sets = self.SETS if shard is None else max(self.SETS, 3 * shard[0])   # keep the footprint above L2
        self.x = [loc["x"].to(dev) for _ in range(sets)]
        self.y = [torch.empty_like(self.x[0]) for _ in range(sets)]
        self.mean = torch.empty(max(self.rows, 1), dtype=torch.float32, device=dev)
        self.rstd = torch.empty(max(self.rows, 1), dtype=torch.float32, device=dev)

    def host_inputs(self):
        return {"x": self.host[0], "weight": self.host[1], "bias": self.host[2]}

    def step(self, i):
        s = i % len(self.x)
        self.ops.layer_norm(self.x[s], self.y[s], self.w, self.b, self.mean[:self.rows], self.rstd[:self.rows], eps=1e-5)

    def work_per_step(self):
        return 2 * self.rows * self.COLS * 2 + 2 * self.COLS * 2  # x + y + gamma + beta

    def local_output(self):
        return self.y[0]

    def describe(self):
        return {"workload": "layer_norm fp16 [16384 x 4096], gamma/beta fp16, eps 1e-5, fp32 statistics, "
                            "mean/rstd fp32 written (configs[1])",
                "l2": "inputs larger than L2: 256 MiB touched per step, 3 rotating buffer sets"}


class SoftmaxWL(Workload):
    name, unit, bound, dtype = "softmax", "GB/s", "hbm", "f32"
    ROWS, COLS, SETS = 8192, 1024, 8
    default_steps, strong_steps = 200, 256

    def __init__(self, dev, shard=None):
        from hexb200 import ops, synth

        self.ops = ops
        x = synth.make_softmax_inputs(self.ROWS, self.COLS)
        self.host = (x,)
        loc = _cut(self.name, self.host_inputs(), shard)
        self.rows = loc["x"].shape[0]
        sets = self.SETS if shard is None else self.SETS * shard[0]
        self.x = [loc["x"].to(dev) for _ in range(sets)]
        self.y = [torch.empty_like(self.x[0]) for _ in range(sets)]

    def host_inputs(self):
        return {"x": self.host[0]}

    def step(self, i):
        s = i % len(self.x)
        self.ops.softmax(self.x[s], self.y[s])

    def work_per_step(self):
        return 2 * self.rows * self.COLS * 4

    def local_output(self):
        return self.y[0]

    def describe(self):
        return {"workload": "row softmax fp32 [8192 x 1024] (configs[0])",
                "l2": "8 rotating buffer sets (512 MiB footprint) so no step finds its rows in L2"}


class GemmWL(Workload):
    name, unit, bound, dtype = "gemm", "TFLOP/s", "tensor", "f16"
    M = N = K = 4096
    default_steps, strong_steps = 50, 64

    def __init__(self, dev, shard=None):
        from hexb200 import ops, synth

        self.ops = ops
        a, b = synth.make_matmul_inputs(self.M, self.N, self.K)
        self.host = (a, b)
        loc = _cut(self.name, self.host_inputs(), shard)
        self.m = loc["a"].shape[0]
        self.a, self.b = loc["a"].to(dev), b.to(dev)
        self.c = torch.empty(self.m, self.N, dtype=torch.float16, device=dev)

    def host_inputs(self):
        return {"a": self.host[0], "b": self.host[1]}

    def step(self, i):
        self.ops.matmul(self.a, self.b, self.c)

    def work_per_step(self):
        return 2.0 * self.m * self.N * self.K

    def local_output(self):
        return self.c

    def describe(self):
        if (GemmWL.M, GemmWL.N, GemmWL.K) != (4096, 4096, 4096):
            return {"workload": f"matmul fp16 {GemmWL.M} x {GemmWL.N} x {GemmWL.K} (--gemm-shape), fp32 accumulation, fp16 out",
                    "l2": "compute-bound; the same operands every step"}
        return {"workload": "matmul fp16 4096 x 4096 x 4096, fp32 accumulation, fp16 out (configs[2])",
                "l2": "compute-bound; operands (64 MiB) stay L2-resident between steps by design"}


class AttentionWL(Workload):
    name, unit, bound, dtype = "attention", "TFLOP/s", "tensor", "f16"
    Z, H, N, D = 4, 32, 4096, 128
    default_steps, strong_steps = 10, 16

    def __init__(self, dev, shard=None):
        from hexb200 import ops, synth

        self.ops = ops
        q, k, v = synth.make_attention_inputs(self.Z, self.H, self.N, self.D)
        self.host = (q, k, v)
        loc = _cut(self.name, self.host_inputs(), shard)      # [pairs, N, D] blocks
        self.pairs = loc["q"].shape[0]
        # a block of (batch, head) pairs is a [1, pairs, N, D] problem: pairs are independent
        self.q, self.k, self.v = (loc[n].to(dev).unsqueeze(0) for n in ("q", "k", "v"))
        self.o = torch.empty_like(self.q)

    def host_inputs(self):
        return {"q": self.host[0], "k": self.host[1], "v": self.host[2]}

    def step(self, i):
        self.ops.attention(self.q, self.k, self.v, self.o, causal=True)

    def work_per_step(self):
        return 4.0 * self.pairs * self.N * self.N * self.D / 2

    def local_output(self):
        return self.o[0]

    def describe(self):
        return {"workload": "causal flash attention fp16 [4, 32, 4096, 128] (configs[3])",
                "l2": "inputs larger than L2 (512 MiB of Q/K/V/O per step)"}


class DecoderWL(Workload):
    name, unit, bound, dtype = "decoder", "TFLOP/s", "tensor", "f16"
    L, DM, NH, FF, B, S = 4, 2048, 16, 8192, 8, 1024
    launches_per_step = 4 * 7
    default_steps, strong_steps = 5, 8

    def __init__(self, dev, shard=None):
        from hexb200 import ops, synth

        x, ws = synth.make_decoder_inputs(self.L, self.DM, self.NH, self.FF, self.B, self.S)
        self.host = (x, ws)
        loc = _cut(self.name, self.host_inputs(), shard)
        self.seqs = loc["x"].shape[0]
        self.wd = [{k: v.to(dev) for k, v in w.items()} for w in ws]
        self.stack = ops.DecoderStack(self.wd, self.NH, self.DM // self.NH, self.FF, max(self.seqs, 1), self.S, 1e-6)
        self.x = loc["x"].to(dev).contiguous()
        self.out = torch.empty_like(self.x)

    def host_inputs(self):
        return {"x": self.host[0], "weights": self.host[1]}

    def step(self, i):
        if self.seqs:
            self.stack.forward(self.x, self.out)

    def work_per_step(self):
        T = self.seqs * self.S
        lin = 2.0 * (3 * self.DM ** 2 + self.DM ** 2 + 3 * self.DM * self.FF) * T
        att = 4.0 * self.seqs * self.NH * self.S * self.S * (self.DM // self.NH) / 2
        return self.L * (lin + att)

    def local_output(self):
        return self.out

    def describe(self):
        return {"workload": "4-layer decoder fp16, d_model 2048, 16 x 128 heads, SwiGLU 8192, batch 8 x seq 1024 (configs[4])",
                "l2": "weights + activations (1.1 GiB) exceed L2"}


class GPT2WL(Workload):
    """GPT2LMHeadModel cut to two layers (the reference's largest test), random fp16 weights, batch 8 x 1024
    tokens, fp16 logits: embedding + 2 x 7 launches + final norm + tied LM head."""
    name, unit, bound, dtype = "gpt2", "TFLOP/s", "tensor", "f16"
    B, S = 8, 1024
    default_steps = 10

    def __init__(self, dev, shard=None):
        from hexb200 import gpt2

        self.cfg = gpt2.GPT2Config()
        self.runner = gpt2.GPT2Runner(self.cfg, gpt2.random_state_dict(self.cfg, seed=1006), device=dev)
        g = torch.Generator().manual_seed(1006)
        ids = torch.randint(0, self.cfg.vocab_size, (self.B, self.S), generator=g)
        self.host = (ids,)
        self.ids = ids.to(dev)
        self.launches_per_step = self.runner.launches()

    def step(self, i):
        self.runner.forward(self.ids, logits_dtype=torch.float16)

    def work_per_step(self):
        return self.runner.flops(self.B, self.S)

    def describe(self):
        return {"workload": "GPT-2 small geometry, 2 layers, fp16, batch 8 x seq 1024, logits [8192, 50257] fp16 "
                            "(the reference's torch-mlir GPT-2 test, random weights)",
                "l2": "wte (77 MB) + logits (823 MB) exceed L2"}


WORKLOADS = {"layernorm": LayerNormWL, "softmax": SoftmaxWL, "gemm": GemmWL, "attention": AttentionWL,
             "decoder": DecoderWL, "gpt2": GPT2WL}
PARTITIONED = ("softmax", "layernorm", "gemm", "attention", "decoder")


def config_of(name, world):
    """The `config` object of the JSON line: the same for both arms, so that they name one workload."""
    cfg = WORKLOADS[name].describe(None)
    cfg["parallelism"] = f"{world} x independent shard (one full-size workload per GPU), no data-path collective"
    return cfg


# ---------------------------------------------------------------------------- timing
class Comm:
    """The collective plumbing of the benchmark itself (barrier, max over ranks); a no-op at N = 1."""

    def __init__(self, dist, dev):
        self.dist, self.dev = dist, dev
        self.world = dist.get_world_size() if dist else 1
        self.rank = dist.get_rank() if dist else 0

    def barrier(self):
        if self.dist:
            self.dist.barrier()

    def max(self, values):
        if not self.dist:
            return list(values)
        t = torch.tensor(list(values), device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]


def time_steps(wl, steps, warmup, comm, use_graph=True, region_ms=50.0, min_windows=9, max_windows=48):
    """W untimed steps, then R windows of exactly K steps each between CUDA events on the launching
    stream (one replay of a CUDA graph of the K launches per window; K eager launches if capture is
    refused), back to back, with a barrier and a synchronize before the first and after the last.

    Returns (window_ms: per window, already the maximum over ranks; t0, t1: host clock around the
    region; mode)."""
    for i in range(warmup):
        wl.step(i)
    torch.cuda.synchronize()
    graph = None
    if use_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i in range(steps):
                    wl.step(warmup + i)
        except Exception:
            graph = None

    def one_window():
        if graph is not None:
            graph.replay()
        else:
            for i in range(steps):
                wl.step(warmup + i)

    one_window()  # untimed: uploads the graph
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    one_window()
    e1.record()
    torch.cuda.synchronize()
    est = comm.max([e0.elapsed_time(e1)])[0]
    windows = int(min(max_windows, max(min_windows, math.ceil(region_ms / max(est, 1e-3)))))
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(windows + 1)]
    comm.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ev[0].record()
    for r in range(windows):
        one_window()
        ev[r + 1].record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    comm.barrier()
    win = comm.max([ev[r].elapsed_time(ev[r + 1]) for r in range(windows)])
    return win, t0, t1, ("cuda_graph" if graph is not None else "eager")


def median(xs):
    s = sorted(xs)
    return s[len(s) // 2]


def roofline(wl, ms_per_step, peaks):
    work = wl.work_per_step()
    if wl.bound == "hbm":
        achieved = work / (ms_per_step * 1e-3) / 1e9
        peak = peaks["hbm_gbs"]
        unit = "GB/s"
    else:
        achieved = work / (ms_per_step * 1e-3) / 1e12
        peak = peaks["bf16_tflops"]   # the burst figure: these timed regions are short
        unit = "TFLOP/s"
    return {"bound": wl.bound, "achieved": round(achieved, 2), "peak": peak, "unit": unit,
            "frac": round(achieved / peak, 4), "traffic": NCU_TRAFFIC.get(wl.name),
            "traffic_source": "ncu capture summarised under profiles/ (not observed by this run)",
            "peak_source": peaks["_source"], "algorithmic_per_launch": work / wl.launches_per_step}


def measure(wl, steps, warmup, comm, sampler, peaks, eager=False):
    """Times one workload; returns the figures every JSON entry is built from."""
    win, t0, t1, mode = time_steps(wl, steps, warmup, comm, not eager)
    ms = median(win) / steps
    scale = 1e9 if wl.bound == "hbm" else 1e12
    return {"ms_per_step": ms, "ms_min": min(win) / steps, "ms_max": max(win) / steps, "windows": len(win),
            "value": comm.world * wl.work_per_step() / (ms * 1e-3) / scale, "mode": mode,
            "clocks": sampler.summary(t0, t1), "roofline": roofline(wl, ms, peaks),
            "region_s": t1 - t0}


def sustained(wl, comm, sampler, peaks, total_steps=120, k=5):
    """The decoder under the power cap: >= 100 back-to-back steps; the second half of the windows is
    what the part sustains, and it is compared with the sustained peak."""
    windows = max(2, total_steps // k)
    win, t0, t1, _ = time_steps(wl, k, 3, comm, True, region_ms=0.0, min_windows=windows, max_windows=windows)
    tail = win[len(win) // 2:]
    ms = sum(tail) / len(tail) / k
    tf = wl.work_per_step() / (ms * 1e-3) / 1e12
    clk = sampler.summary(t0 + (t1 - t0) / 2, t1)
    peak = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
    return {"steps": windows * k, "ms_per_step": round(ms, 4), "tflops": round(tf, 1), "peak_sustained": peak,
            "frac_sustained": round(tf / peak, 4), "sm_mhz": clk["sm_mhz"], "reasons": clk["reasons"],
            "ms_x_mhz": round(ms * clk["sm_mhz"], 1) if clk["sm_mhz"] else None}


# ---------------------------------------------------------------------------- CPU baseline (reference arm)
def cpu_reference_step(name):
    """Returns (fn, work, sample): one bounded sample of the workload on the host cores through the
    PyTorch CPU eager calls the reference's tests compare against (test_softmax.py:93,
    test_layer_norm.py:111-113, test_matmul.py:90, test_flash_attention.py:212)."""
    import torch.nn.functional as F
    from hexb200 import synth

    if name == "layernorm":
        rows = 16384  # the full workload: a smaller sample would sit in the CPU's caches
        x, w, b = synth.make_layer_norm_inputs(rows, 4096)
        return (lambda: F.layer_norm(x, (4096,), weight=w, bias=b, eps=1e-5), 2 * rows * 4096 * 2 + 4 * 4096,
                "full [16384 x 4096] fp16, F.layer_norm on CPU")
    if name == "softmax":
        x = synth.make_softmax_inputs(8192, 1024)
        return (lambda: F.softmax(x, dim=1), 2 * 8192 * 1024 * 4, "full [8192 x 1024] fp32, F.softmax on CPU")
    if name == "gemm":
        a, b = synth.make_matmul_inputs(1024, 4096, 4096)
        af, bf = a.float(), b.float()
        return (lambda: torch.matmul(af, bf), 2.0 * 1024 * 4096 * 4096,
                "1024 of 4096 rows of A, torch.matmul with fp32 compute from the fp16 inputs")
    if name == "attention":
        q, k, v = (t.float() for t in synth.make_attention_inputs(1, 4, 4096, 128))
        return (lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True), 4.0 * 4 * 4096 * 4096 * 128 / 2,
                "4 of 128 (batch, head) pairs, F.scaled_dot_product_attention(is_causal=True) fp32 on CPU")
    if name == "gpt2":
        from hexb200 import gpt2
        from oracle import oracle as O   # CPU leg: the fp32 restatement of the model
        cfg = gpt2.GPT2Config()
        sd = gpt2.random_state_dict(cfg, seed=1006)
        ids = torch.randint(0, cfg.vocab_size, (1, 256), generator=torch.Generator().manual_seed(1006))
        work = gpt2.GPT2Runner.flops_of(cfg, 1, 256)
        return (lambda: O.torch_gpt2(sd, cfg.n_layer, cfg.n_head, cfg.layer_norm_epsilon, ids), work,
                "1 sequence x 256 tokens, fp32 torch on the fp16-rounded weights")
    if name == "decoder":
        from oracle import oracle as O   # CPU leg: the block stack in plain PyTorch
        x, ws = synth.make_decoder_inputs(1, 2048, 16, 8192, 1, 1024)
        T = 1024
        work = 2.0 * (4 * 2048 ** 2 + 3 * 2048 * 8192) * T + 4.0 * 16 * 1024 * 1024 * 128 / 2
        return (lambda: O.torch_decoder(x, ws, 16, 128, 8192, 1, 1024, 1e-6, store_dtype=None), work,
                "1 of 4 layers on 1 of 8 sequences, plain PyTorch CPU fp32")
    raise KeyError(name)


def time_cpu(name, steps, warmup, limit_s=25.0):
    fn, work, sample = cpu_reference_step(name)
    torch.set_num_threads(os.cpu_count() or 1)
    for _ in range(max(1, warmup)):
        fn()
    ts = []
    t_all = time.perf_counter()
    for _ in range(max(1, steps)):
        t = time.perf_counter()
        fn()
        ts.append(time.perf_counter() - t)
        if time.perf_counter() - t_all > limit_s:
            break
    dt = sum(ts) / len(ts)
    return work / dt, dt, len(ts), sample


# ---------------------------------------------------------------------------- end to end (host buffers)
def e2e_call(wl):
    """Returns (call, h2d_bytes, d2h_bytes, api): one step through the reference-facing launcher with
    pinned HOST tensors -- every call copies the step's inputs to the device and its result back."""
    import hexb200
    from hexb200 import ops

    if wl.name == "layernorm":
        x, w, b = wl.host
        xp, wp, bp = x.pin_memory(), w.pin_memory(), b.pin_memory()
        y = torch.empty_like(x).pin_memory()
        mean = torch.empty(wl.ROWS, dtype=torch.float32).pin_memory()
        rstd = torch.empty(wl.ROWS, dtype=torch.float32).pin_memory()
        kern = hexb200.kernels.layer_norm_fwd_kernel
        call = lambda: kern[(4,)](xp, y, wp, bp, mean, rstd, EPSILON=1e-5, NUM_ROWS=wl.ROWS, NUM_COLS=wl.COLS,
                                  BLOCK_SIZE=4096, enableMultiThreading=True, enableVTCMTiling=True)
        return (call, x.numel() * 2 + 2 * wl.COLS * 2, x.numel() * 2 + 2 * wl.ROWS * 4,
                "hexb200.kernels.layer_norm_fwd_kernel[grid](host tensors) -> hexb_layer_norm_host")
    if wl.name == "softmax":
        (x,) = wl.host
        xp, y = x.pin_memory(), torch.empty_like(x).pin_memory()
        call = lambda: hexb200.kernels.softmax_kernel[(4,)](xp, y, NUM_ROWS=wl.ROWS, NUM_COLS=wl.COLS, BLOCK_SIZE=1024)
        return call, x.numel() * 4, x.numel() * 4, "kernels.softmax_kernel[grid](host tensors) -> hexb_softmax_host"
    if wl.name == "gemm":
        a, b = wl.host
        ap, bp, c = a.pin_memory(), b.pin_memory(), torch.empty(wl.M, wl.N, dtype=torch.float16).pin_memory()
        call = lambda: hexb200.kernels.matmul[(1,)](ap, bp, c, wl.M, wl.N, wl.K)
        return call, (a.numel() + b.numel()) * 2, c.numel() * 2, "kernels.matmul[grid](host tensors) -> hexb_matmul_f16_host"
    if wl.name == "attention":
        q, k, v = (t.pin_memory() for t in wl.host)
        o = torch.empty_like(q).pin_memory()
        call = lambda: ops.attention(q, k, v, o, causal=True)
        return call, 3 * q.numel() * 2, q.numel() * 2, "ops.attention(host tensors) -> hexb_attention_fwd_host"
    if wl.name == "gpt2":
        (ids,) = wl.host
        idp = ids.pin_memory()
        last = torch.empty(wl.B, wl.cfg.vocab_size, dtype=torch.float16).pin_memory()

        def call():  # prompt ids up, the last position's logits back (what the reference's top-5 check reads)
            wl.ids.copy_(idp, non_blocking=True)
            logits = wl.runner.forward(wl.ids, logits_dtype=torch.float16)
            last.copy_(logits[:, -1, :], non_blocking=True)
            torch.cuda.synchronize()

        return call, ids.numel() * 8, last.numel() * 2, "GPT2Runner.forward (ids up, last-position logits back)"
    x = wl.host[0]
    xp, outp = x.pin_memory(), torch.empty_like(x).pin_memory()

    def call():
        wl.x.copy_(xp, non_blocking=True)
        wl.stack.forward(wl.x, wl.out)
        outp.copy_(wl.out, non_blocking=True)
        torch.cuda.synchronize()

    return call, x.numel() * 2, x.numel() * 2, "DecoderStack.forward (activations up, result back)"


def e2e_measure(wl, steps, comm):
    """The same metric through the launcher with host buffers, on every rank at once; the time is the
    maximum over ranks and the value the aggregate over the job."""
    call, h2d, d2h, api = e2e_call(wl)
    call()
    call()
    n = max(3, min(steps, 20 if wl.bound == "hbm" else 5))
    comm.barrier()
    t = time.perf_counter()
    for _ in range(n):
        call()
    dt = (time.perf_counter() - t) / n
    dt = comm.max([dt])[0]
    scale = 1e9 if wl.bound == "hbm" else 1e12
    return {"value": round(comm.world * wl.work_per_step() / dt / scale, 3), "unit": wl.unit,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": round(dt * 1e3, 3), "steps": n,
            "ranks": comm.world, "api": api}


# ---------------------------------------------------------------------------- partitioned form (N > 1)
def oracle_units(name, host, units):
    """CPU values of the sampled units of the whole output (untimed check of the gathered tensor):
    the PyTorch CPU calls the reference's tests assert against, in fp32 from the stored inputs."""
    from oracle import oracle as O

    idx = torch.tensor(units, dtype=torch.long)
    if name == "softmax":
        return O.torch_softmax(host["x"][idx])
    if name == "layernorm":
        return O.torch_layer_norm(host["x"][idx], host["weight"], host["bias"], 1e-5)
    if name == "gemm":
        return O.torch_matmul(host["a"][idx], host["b"])
    if name == "attention":
        q, k, v = (host[n].reshape(-1, host[n].shape[2], host[n].shape[3])[idx].unsqueeze(0) for n in ("q", "k", "v"))
        return O.torch_attention(q, k, v, q.shape[-1] ** -0.5, causal=True)[0]
    if name == "decoder":
        x, ws = host["x"], host["weights"]
        dm, ff = ws[0]["wo"].shape[0], ws[0]["wd"].shape[0]
        return O.torch_decoder(x[idx].contiguous(), ws, dm // 128, 128, ff, len(units), x.shape[1], 1e-6)
    raise KeyError(name)


def strong_block(name, dev, comm, sampler, peaks, full_ms, eager=False):
    """One configuration cut across the ranks: kernel time of the blocks (max over ranks), the NCCL
    all-gather of the output blocks timed apart, and the gathered tensor checked against the oracle."""
    from hexb200 import dist as hd

    wl = WORKLOADS[name](dev, shard=(comm.world, comm.rank))
    m = measure(wl, wl.strong_steps, 3, comm, sampler, peaks, eager)
    y_local = wl.local_output()
    total = hd.units_of(name, wl.host_inputs())
    for _ in range(2):
        y = hd.all_gather_rows(y_local, total)
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
    comm.barrier()
    ev[0].record()
    for r in range(5):
        y = hd.all_gather_rows(y_local, total)
        ev[r + 1].record()
    torch.cuda.synchronize()
    gather_ms = median(comm.max([ev[r].elapsed_time(ev[r + 1]) for r in range(5)]))
    out_bytes = y.numel() * y.element_size()
    err = None
    if comm.rank == 0:
        units = hd.sample_units(total, comm.world, 1 if name == "decoder" else 2)
        if name == "decoder" and len(units) > 3:
            units = [units[0], units[len(units) // 2], units[-1]]
        got = y[torch.tensor(units, device=y.device)].float().cpu()
        ref = oracle_units(name, wl.host_inputs(), units).float()
        err = float((got - ref.reshape(got.shape)).abs().max() / ref.abs().max().clamp_min(1e-30))
    shard_ms = m["ms_per_step"]
    return {"speedup": round(full_ms / shard_ms, 2), "shard_ms": round(shard_ms, 5), "full_ms": round(full_ms, 5),
            "gather_ms": round(gather_ms, 4), "gather_GBps": round(out_bytes / (gather_ms * 1e-3) / 1e9, 1),
            "max_rel_err": None if err is None else float(f"{err:.3g}"), "steps": wl.strong_steps}


# ---------------------------------------------------------------------------- main
def main():
    # stdout must carry exactly one JSON line: keep a private handle to it and point fd 1 at stderr,
    # so that anything a library prints (NCCL's version banner, warnings) cannot land beside it.
    sys.stdout.flush()
    real_stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)

    def emit(obj):
        real_stdout.write(json.dumps(obj) + "\n")
        real_stdout.flush()

    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="layernorm", choices=sorted(WORKLOADS))
    ap.add_argument("--no-extras", action="store_true", help="skip the other workloads, the partitioned form and the CPU baselines")
    ap.add_argument("--eager", action="store_true", help="time K eager launches per window instead of a CUDA-graph replay of them")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end measurement (profiling runs)")
    ap.add_argument("--gemm-shape", default="", help="M,N,K for --workload gemm instead of 4096,4096,4096 (e.g. the decoder's "
                                                     "down projection 8192,2048,8192)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.gemm_shape:
        GemmWL.M, GemmWL.N, GemmWL.K = (int(v) for v in args.gemm_shape.split(","))

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    peaks = load_peaks()

    if args.impl == "reference":
        if rank != 0:
            return 0
        val, dt, n, sample = time_cpu(args.workload, args.steps, args.warmup)
        wl_cls = WORKLOADS[args.workload]
        scale = 1e9 if wl_cls.bound == "hbm" else 1e12
        cores = torch.get_num_threads()
        line = {"impl": "reference", "metric": METRIC, "value": round(val / scale, 4), "unit": wl_cls.unit,
                "n_gpus": args.gpus, "steps": n, "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3),
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl_cls.dtype,
                "data": "synthetic", "config": config_of(args.workload, max(world, args.gpus)),
                "cpu_baseline": {"value": round(val / scale, 4), "unit": wl_cls.unit, "cores": cores, "kind": "port",
                                 "sample": sample},
                "e2e": {"value": round(val / scale, 4), "unit": wl_cls.unit, "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0}}
        emit(line)
        return 0

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    import hexb200

    hexb200.load()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)
    comm = Comm(dist, dev)
    sampler = ClockSampler(local_rank)
    sampler.start()

    wl = WORKLOADS[args.workload](dev)
    m = measure(wl, args.steps, args.warmup, comm, sampler, peaks, args.eager)
    status = hexb200.device_status()
    e2e = None if args.no_e2e else e2e_measure(wl, args.steps, comm)
    full_ms = {args.workload: m["ms_per_step"]}
    launches = m["windows"] * args.steps * wl.launches_per_step

    line = {"metric": METRIC, "value": round(m["value"], 2), "unit": wl.unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(m["ms_per_step"], 5), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": config_of(args.workload, world), "roofline": m["roofline"], "clocks": m["clocks"],
            "gpu_launches": launches, "launch_mode": m["mode"], "device_status": status,
            "timing": {"windows": m["windows"], "steps_per_window": args.steps, "ms_per_step_min": round(m["ms_min"], 5),
                       "ms_per_step_max": round(m["ms_max"], 5), "timed_region_s": round(m["region_s"], 4),
                       "statistic": "median window / K, each window the max over ranks"},
            "e2e": e2e, "cpu_baseline": None}
    if wl.name == "decoder" and not args.no_extras:
        line["sustained"] = sustained(wl, comm, sampler, peaks)
    del wl
    torch.cuda.empty_cache()

    if not args.no_extras:
        # every other configuration, on every rank (max over ranks), compactly
        extras = {}
        for name in WORKLOADS:
            if name == args.workload:
                continue
            w2 = WORKLOADS[name](dev)
            m2 = measure(w2, w2.default_steps, 3, comm, sampler, peaks, args.eager)
            full_ms[name] = m2["ms_per_step"]
            ent = {"value": round(m2["value"], 1), "unit": w2.unit, "ms_per_step": round(m2["ms_per_step"], 5),
                   "frac": m2["roofline"]["frac"], "sm_mhz": m2["clocks"]["sm_mhz"]}
            if name == "decoder":
                s = sustained(w2, comm, sampler, peaks)
                ent["sustained"] = {k: s[k] for k in ("steps", "ms_per_step", "tflops", "frac_sustained", "sm_mhz", "ms_x_mhz")}
            if not args.no_e2e:
                ent["e2e"] = e2e_measure(w2, w2.default_steps, comm)["value"]
            st2 = hexb200.device_status()
            if st2:
                ent["device_status"] = st2
            extras[name] = ent
            del w2
            torch.cuda.empty_cache()
        strong = None
        if world > 1:
            strong = {}
            for name in PARTITIONED:
                strong[name] = strong_block(name, dev, comm, sampler, peaks, full_ms[name], args.eager)
                torch.cuda.empty_cache()
        if rank == 0 and world == 1:
            # CPU baselines: the headline's as the contract's object, the others inside their entries
            val, dt, n, sample = time_cpu(args.workload, 8, 2, limit_s=15.0)
            scale = 1e9 if WORKLOADS[args.workload].bound == "hbm" else 1e12
            line["cpu_baseline"] = {"value": round(val / scale, 4), "unit": WORKLOADS[args.workload].unit,
                                    "cores": torch.get_num_threads(), "kind": "port", "sample": sample,
                                    "ms_per_sample": round(dt * 1e3, 3)}
            for name, ent in extras.items():
                val, dt, n, sample = time_cpu(name, 4, 1, limit_s=8.0)
                sc = 1e9 if WORKLOADS[name].bound == "hbm" else 1e12
                ent["cpu_baseline"] = round(val / sc, 4)
            line["cpu_cores"] = torch.get_num_threads()
        # last in the line, so that the end of the output shows them whole
        if strong is not None:
            line["strong"] = strong
        line["workloads"] = extras

    sampler.stop()
    if rank == 0:
        emit(line)
    if dist:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
