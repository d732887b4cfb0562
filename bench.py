#!/usr/bin/env python
"""Benchmark of the hexb200 hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of the hot path over one batch of seeded synthetic input.  The headline workload
is LayerNorm fp16 [16384 x 4096] (the benchmark's second configuration, the bandwidth-bound one the
HBM GB/s metric is quoted on); `--workload` selects softmax / gemm / attention / decoder (the benchmark's
other configurations) or gpt2 (the reference's two-layer GPT-2 test) instead, and the default single-GPU
run also measures those five and lists them under "workloads".  Rank 0 prints
ONE JSON line.  With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank runs the
full-size workload on its own GPU (weak scaling: independent row blocks / (batch, head) pairs /
sequences, no data-path collective); the optional all-gather of output shards is timed apart.

`--impl reference` times the CPU implementation of the same path (the PyTorch CPU eager calls the
reference's tests compare against) on the host cores, on a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "HBM GB/s (softmax/LN) & TFLOP/s (GEMM/attn) vs roofline at 1/2/4/8 B200"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# ncu `dram__bytes_read.sum + dram__bytes_write.sum` per launch of the dominant kernel, filled in from
# the committed summaries under profiles/ (bytes; output still dirty in L2 at kernel end is not in it).
NCU_TRAFFIC = {"layernorm": 216.52e6, "softmax": 33.98e6, "gemm": 87.44e6, "attention": 519.9e6, "decoder": None}


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
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

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
        if self.ok:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()

    def stop(self):
        if self._thr:
            self._stop.set()
            self._thr.join()

    def summary(self, t0, t1):
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0, "window": "none"}
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        window = "timed"
        if len(inside) < 3:
            inside, window = self.samples, "warmup+timed"
        mhz = sorted(s[1] for s in inside)
        bits = 0
        for s in inside:
            bits |= s[2]
        names = {0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
                 0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
                 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz,
                "reasons": [n for b, n in names.items() if bits & b], "samples": len(inside), "window": window}


# ---------------------------------------------------------------------------- workloads
class Workload:
    """One configuration: device buffers, a `step()` that launches the hot path, and its accounting."""

    name = ""
    unit = ""
    bound = ""
    dtype = ""
    launches_per_step = 1

    def step(self, i: int):
        raise NotImplementedError

    def work_per_step(self) -> float:  # algorithmic bytes (hbm) or flops (tensor)
        raise NotImplementedError


class LayerNormWL(Workload):
    name, unit, bound, dtype = "layernorm", "GB/s", "hbm", "f16"
    ROWS, COLS, SETS = 16384, 4096, 3

    def __init__(self, dev):
        from hexb200 import ops
        from oracle import oracle as O  # input generator only (seeded synthetic data)

        self.ops = ops
        x, w, b = O.make_layer_norm_inputs(self.ROWS, self.COLS)
        self.host = (x, w, b)
        self.w, self.b = w.to(dev), b.to(dev)
        self.x = [x.to(dev) for _ in range(self.SETS)]
        self.y = [torch.empty_like(self.x[0]) for _ in range(self.SETS)]
        self.mean = torch.empty(self.ROWS, dtype=torch.float32, device=dev)
        self.rstd = torch.empty(self.ROWS, dtype=torch.float32, device=dev)

    def step(self, i):
        s = i % self.SETS
        self.ops.layer_norm(self.x[s], self.y[s], self.w, self.b, self.mean, self.rstd, eps=1e-5)

    def work_per_step(self):
        return 2 * self.ROWS * self.COLS * 2 + 2 * self.COLS * 2  # x + y + gamma + beta

    def describe(self):
        return {"workload": "layer_norm fp16 [16384 x 4096], gamma/beta fp16, eps 1e-5, fp32 statistics, "
                            "mean/rstd fp32 written (configs[1])",
                "l2": "inputs larger than L2: 256 MiB touched per step, 3 rotating buffer sets"}


class SoftmaxWL(Workload):
    name, unit, bound, dtype = "softmax", "GB/s", "hbm", "f32"
    ROWS, COLS, SETS = 8192, 1024, 8

    def __init__(self, dev):
        from hexb200 import ops
        from oracle import oracle as O

        self.ops = ops
        x = O.make_softmax_inputs(self.ROWS, self.COLS)
        self.host = (x,)
        self.x = [x.to(dev) for _ in range(self.SETS)]
        self.y = [torch.empty_like(self.x[0]) for _ in range(self.SETS)]

    def step(self, i):
        s = i % self.SETS
        self.ops.softmax(self.x[s], self.y[s])

    def work_per_step(self):
        return 2 * self.ROWS * self.COLS * 4

    def describe(self):
        return {"workload": "row softmax fp32 [8192 x 1024] (configs[0])",
                "l2": "8 rotating buffer sets (512 MiB footprint) so no step finds its rows in L2"}


class GemmWL(Workload):
    name, unit, bound, dtype = "gemm", "TFLOP/s", "tensor", "f16"
    M = N = K = 4096

    def __init__(self, dev):
        from hexb200 import ops
        from oracle import oracle as O

        self.ops = ops
        a, b = O.make_matmul_inputs(self.M, self.N, self.K)
        self.host = (a, b)
        self.a, self.b = a.to(dev), b.to(dev)
        self.c = torch.empty(self.M, self.N, dtype=torch.float16, device=dev)
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step(self, i):
        self.ops.matmul(self.a, self.b, self.c)

    def work_per_step(self):
        return 2.0 * self.M * self.N * self.K

    def describe(self):
        return {"workload": "matmul fp16 4096 x 4096 x 4096, fp32 accumulation, fp16 out (configs[2])",
                "l2": "compute-bound; operands (64 MiB) stay L2-resident between steps by design"}


class AttentionWL(Workload):
    name, unit, bound, dtype = "attention", "TFLOP/s", "tensor", "f16"
    Z, H, N, D = 4, 32, 4096, 128

    def __init__(self, dev):
        from hexb200 import ops
        from oracle import oracle as O

        self.ops = ops
        q, k, v = O.make_attention_inputs(self.Z, self.H, self.N, self.D)
        self.host = (q, k, v)
        self.q, self.k, self.v = q.to(dev), k.to(dev), v.to(dev)
        self.o = torch.empty_like(self.q)

    def step(self, i):
        self.ops.attention(self.q, self.k, self.v, self.o, causal=True)

    def work_per_step(self):
        return 4.0 * self.Z * self.H * self.N * self.N * self.D / 2

    def describe(self):
        return {"workload": "causal flash attention fp16 [4, 32, 4096, 128] (configs[3])",
                "l2": "inputs larger than L2 (512 MiB of Q/K/V/O per step)"}


class DecoderWL(Workload):
    name, unit, bound, dtype = "decoder", "TFLOP/s", "tensor", "f16"
    L, DM, NH, FF, B, S = 4, 2048, 16, 8192, 8, 1024
    launches_per_step = 4 * 7

    def __init__(self, dev):
        from hexb200 import ops
        from oracle import oracle as O

        x, ws = O.make_decoder_inputs(self.L, self.DM, self.NH, self.FF, self.B, self.S)
        self.host = (x,)
        self.wd = [{k: v.to(dev) for k, v in w.items()} for w in ws]
        self.stack = ops.DecoderStack(self.wd, self.NH, self.DM // self.NH, self.FF, self.B, self.S, 1e-6)
        self.x = x.to(dev)
        self.out = torch.empty_like(self.x)

    def step(self, i):
        self.stack.forward(self.x, self.out)

    def work_per_step(self):
        T = self.B * self.S
        lin = 2.0 * (3 * self.DM ** 2 + self.DM ** 2 + 3 * self.DM * self.FF) * T
        att = 4.0 * self.B * self.NH * self.S * self.S * (self.DM // self.NH) / 2
        return self.L * (lin + att)

    def describe(self):
        return {"workload": "4-layer decoder fp16, d_model 2048, 16 x 128 heads, SwiGLU 8192, batch 8 x seq 1024 (configs[4])",
                "l2": "weights + activations (1.1 GiB) exceed L2"}


class GPT2WL(Workload):
    """GPT2LMHeadModel cut to two layers (the reference's largest test), random fp16 weights, batch 8 x 1024
    tokens, fp16 logits: embedding + 2 x 7 launches + final norm + tied LM head."""
    name, unit, bound, dtype = "gpt2", "TFLOP/s", "tensor", "f16"
    B, S = 8, 1024

    def __init__(self, dev):
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


def time_steps(wl, steps, warmup, barrier, use_graph=True):
    """W untimed steps, then exactly K steps between two CUDA events on the launching stream.

    The K steps are captured once into a CUDA graph (the library's launches are plain stream
    launches, so they capture) and the timed region is one replay of it: the same K kernel
    launches, without the Python and driver launch gap between them.  Falls back to K eager calls
    if capture is refused.  Returns (ms for K steps, t0, t1, mode)."""
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
            graph.replay()  # untimed: uploads the graph
        except Exception:
            graph = None
    torch.cuda.synchronize()
    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    if graph is not None:
        graph.replay()
    else:
        for i in range(steps):
            wl.step(warmup + i)
    e1.record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    barrier()
    return e0.elapsed_time(e1), t0, t1, ("cuda_graph" if graph is not None else "eager")


def roofline(wl, ms_per_step, peaks):
    work = wl.work_per_step()
    if wl.bound == "hbm":
        achieved = work / (ms_per_step * 1e-3) / 1e9
        peak = peaks["hbm_gbs"]
        unit = "GB/s"
    else:
        achieved = work / (ms_per_step * 1e-3) / 1e12
        peak = peaks["bf16_tflops"] if wl.name != "decoder" else peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
        unit = "TFLOP/s"
    return {"bound": wl.bound, "achieved": round(achieved, 2), "peak": peak, "unit": unit,
            "frac": round(achieved / peak, 4), "traffic": NCU_TRAFFIC.get(wl.name),
            "peak_source": peaks["_source"], "algorithmic_per_launch": work / wl.launches_per_step}


# ---------------------------------------------------------------------------- CPU baseline (reference arm)
def cpu_reference_step(name):
    """Returns (fn, work, sample): one bounded sample of the workload on the host cores through the
    PyTorch CPU eager calls the reference's tests compare against."""
    import torch.nn.functional as F
    from oracle import oracle as O

    if name == "layernorm":
        rows = 16384  # the full workload: a smaller sample would sit in the CPU's caches
        x, w, b = O.make_layer_norm_inputs(rows, 4096)
        return (lambda: F.layer_norm(x, (4096,), weight=w, bias=b, eps=1e-5), 2 * rows * 4096 * 2 + 4 * 4096,
                "full [16384 x 4096] fp16, F.layer_norm on CPU")
    if name == "softmax":
        x = O.make_softmax_inputs(8192, 1024)
        return (lambda: F.softmax(x, dim=1), 2 * 8192 * 1024 * 4, "full [8192 x 1024] fp32, F.softmax on CPU")
    if name == "gemm":
        a, b = O.make_matmul_inputs(1024, 4096, 4096)
        af, bf = a.float(), b.float()
        return (lambda: torch.matmul(af, bf), 2.0 * 1024 * 4096 * 4096,
                "1024 of 4096 rows of A, torch.matmul with fp32 compute from the fp16 inputs")
    if name == "attention":
        q, k, v = (t.float() for t in O.make_attention_inputs(1, 4, 4096, 128))
        return (lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True), 4.0 * 4 * 4096 * 4096 * 128 / 2,
                "4 of 128 (batch, head) pairs, F.scaled_dot_product_attention(is_causal=True) fp32 on CPU")
    if name == "gpt2":
        from hexb200 import gpt2
        cfg = gpt2.GPT2Config()
        sd = gpt2.random_state_dict(cfg, seed=1006)
        ids = torch.randint(0, cfg.vocab_size, (1, 256), generator=torch.Generator().manual_seed(1006))
        work = gpt2.GPT2Runner.flops_of(cfg, 1, 256)
        return (lambda: O.torch_gpt2(sd, cfg.n_layer, cfg.n_head, cfg.layer_norm_epsilon, ids), work,
                "1 sequence x 256 tokens, fp32 torch on the fp16-rounded weights")
    if name == "decoder":
        x, ws = O.make_decoder_inputs(1, 2048, 16, 8192, 1, 1024)
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
def e2e_layernorm(wl, steps):
    """The same metric through the reference-signature launcher with HOST tensors: every step copies
    x, gamma, beta to the device and y, mean, rstd back (pinned host memory), inside the timed region."""
    import hexb200

    x, w, b = wl.host
    xp, wp, bp = x.pin_memory(), w.pin_memory(), b.pin_memory()
    y = torch.empty_like(x).pin_memory()
    mean = torch.empty(wl.ROWS, dtype=torch.float32).pin_memory()
    rstd = torch.empty(wl.ROWS, dtype=torch.float32).pin_memory()
    kern = hexb200.kernels.layer_norm_fwd_kernel

    def call():
        kern[(4,)](xp, y, wp, bp, mean, rstd, EPSILON=1e-5, NUM_ROWS=wl.ROWS, NUM_COLS=wl.COLS,
                   BLOCK_SIZE=4096, enableMultiThreading=True, enableVTCMTiling=True)

    call()
    call()
    n = max(3, min(steps, 20))
    t = time.perf_counter()
    for _ in range(n):
        call()
    dt = (time.perf_counter() - t) / n
    h2d = x.numel() * 2 + 2 * wl.COLS * 2
    d2h = x.numel() * 2 + 2 * wl.ROWS * 4
    return {"value": round(wl.work_per_step() / dt / 1e9, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h, "ms_per_step": round(dt * 1e3, 3), "steps": n,
            "api": "hexb200.kernels.layer_norm_fwd_kernel[grid](host tensors) -> hexb_layer_norm_host"}


def e2e_generic(wl, steps):
    import hexb200
    from hexb200 import ops

    n = max(2, min(steps, 5))
    if wl.name == "softmax":
        (x,) = wl.host
        xp, y = x.pin_memory(), torch.empty_like(x).pin_memory()
        call = lambda: hexb200.kernels.softmax_kernel[(4,)](xp, y, NUM_ROWS=wl.ROWS, NUM_COLS=wl.COLS, BLOCK_SIZE=1024)
        h2d = d2h = x.numel() * 4
    elif wl.name == "gemm":
        a, b = wl.host
        ap, bp, c = a.pin_memory(), b.pin_memory(), torch.empty(wl.M, wl.N, dtype=torch.float16).pin_memory()
        call = lambda: hexb200.kernels.matmul[(1,)](ap, bp, c, wl.M, wl.N, wl.K)
        h2d, d2h = (a.numel() + b.numel()) * 2, c.numel() * 2
    elif wl.name == "attention":
        q, k, v = (t.pin_memory() for t in wl.host)
        o = torch.empty_like(q).pin_memory()
        call = lambda: ops.attention(q, k, v, o, causal=True)
        h2d, d2h = 3 * q.numel() * 2, q.numel() * 2
    elif wl.name == "gpt2":
        (ids,) = wl.host
        idp = ids.pin_memory()
        last = torch.empty(wl.B, wl.cfg.vocab_size, dtype=torch.float16).pin_memory()

        def call():  # prompt ids up, the last position's logits back (what the reference's top-5 check reads)
            wl.ids.copy_(idp, non_blocking=True)
            logits = wl.runner.forward(wl.ids, logits_dtype=torch.float16)
            last.copy_(logits[:, -1, :], non_blocking=True)
            torch.cuda.synchronize()

        h2d, d2h = ids.numel() * 8, last.numel() * 2
    else:
        (x,) = wl.host
        xp, outp = x.pin_memory(), torch.empty_like(x).pin_memory()

        def call():
            wl.x.copy_(xp, non_blocking=True)
            wl.stack.forward(wl.x, wl.out)
            outp.copy_(wl.out, non_blocking=True)
            torch.cuda.synchronize()

        h2d = d2h = x.numel() * 2
    call()
    t = time.perf_counter()
    for _ in range(n):
        call()
    dt = (time.perf_counter() - t) / n
    scale = 1e9 if wl.bound == "hbm" else 1e12
    return {"value": round(wl.work_per_step() / dt / scale, 3), "unit": wl.unit, "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h, "ms_per_step": round(dt * 1e3, 3), "steps": n}


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
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="layernorm", choices=sorted(WORKLOADS))
    ap.add_argument("--no-extras", action="store_true", help="skip the other workloads and the CPU baseline")
    ap.add_argument("--eager", action="store_true", help="time K eager launches instead of one CUDA-graph replay of them")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end measurement (profiling runs)")
    ap.add_argument("--gather", action="store_true", help="also time the all-gather of output shards (N > 1)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

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
                "data": "synthetic", "config": {"workload": wl_cls.name + " (CPU, bounded sample: " + sample + ")"},
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
    barrier = (lambda: dist.barrier()) if dist else (lambda: None)

    wl = WORKLOADS[args.workload](dev)
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms_total, t0, t1, launch_mode = time_steps(wl, args.steps, args.warmup, barrier, not args.eager)
    sampler.stop()
    clocks = sampler.summary(t0, t1)
    if dist:
        t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_per_step = ms_total / args.steps
    scale = 1e9 if wl.bound == "hbm" else 1e12
    value = world * wl.work_per_step() / (ms_per_step * 1e-3) / scale
    status = hexb200.device_status()

    gather = None
    if dist and args.gather and hasattr(wl, "y"):
        from hexb200.dist import all_gather_rows

        y = wl.y[0]
        for _ in range(2):
            all_gather_rows(y, y.shape[0] * world)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        all_gather_rows(y, y.shape[0] * world)
        e1.record()
        torch.cuda.synchronize()
        gather = {"ms": round(e0.elapsed_time(e1), 4), "bytes_per_rank": y.numel() * y.element_size()}

    line = None
    if rank == 0:
        cfg = wl.describe()
        cfg["parallelism"] = f"{world} x independent shard (one full-size workload per GPU), no data-path collective"
        line = {"metric": METRIC, "value": round(value, 2), "unit": wl.unit, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": cfg,
                "roofline": roofline(wl, ms_per_step, peaks), "clocks": clocks,
                "gpu_launches": args.steps * wl.launches_per_step, "launch_mode": launch_mode,
                "device_status": status}
        if gather:
            line["gather"] = gather
        if args.no_e2e:
            line["e2e"] = None
        else:
            line["e2e"] = e2e_layernorm(wl, args.steps) if wl.name == "layernorm" else e2e_generic(wl, args.steps)

    if rank == 0 and world == 1 and not args.no_extras:
        del wl
        torch.cuda.empty_cache()
        extras = {}
        for name in WORKLOADS:
            if name == args.workload:
                continue
            w2 = WORKLOADS[name](dev)
            k2 = {"softmax": 200, "gemm": 50, "attention": 10, "decoder": 5, "gpt2": 10}.get(name, 20)
            ms2, _, _, _ = time_steps(w2, k2, 3, lambda: None, not args.eager)
            ms2 /= k2
            sc = 1e9 if w2.bound == "hbm" else 1e12
            extras[name] = {"value": round(w2.work_per_step() / (ms2 * 1e-3) / sc, 2), "unit": w2.unit,
                            "ms_per_step": round(ms2, 5), "steps": k2, "roofline": roofline(w2, ms2, peaks),
                            "config": w2.describe(), "device_status": hexb200.device_status(),
                            "e2e": None if args.no_e2e else (e2e_layernorm(w2, k2) if name == "layernorm"
                                                             else e2e_generic(w2, k2))}
            del w2
            torch.cuda.empty_cache()
        line["workloads"] = extras
        val, dt, n, sample = time_cpu(args.workload, 8, 2, limit_s=20.0)
        wl_cls = WORKLOADS[args.workload]
        line["cpu_baseline"] = {"value": round(val / scale, 4), "unit": wl_cls.unit, "cores": torch.get_num_threads(),
                                "kind": "port", "sample": sample, "ms_per_sample": round(dt * 1e3, 3)}
    elif rank == 0:
        line["cpu_baseline"] = None

    if rank == 0:
        emit(line)
    if dist:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
