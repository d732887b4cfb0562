"""CPU: the host-side mirror of the reference's launcher interface -- option filtering, argument
binding by the reference kernels' parameter names, name-based dispatch, the triton shim -- and the
multi-GPU partition/gather logic on two gloo ranks."""
import os
import socket
import sys
import warnings

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import hexb200
from hexb200 import kernels, options
from hexb200.dist import all_gather_rows, shard_range, shard_rows

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_split_options_accepts_every_reference_flag():
    kw = {"NUM_ROWS": 4, "enableVTCMTiling": False, "enableHexKL": True, "iterations": 1, "scratch": 0,
          "num_threads": 4, "hexKLMode": "macro"}
    args, opts = options.split_options(kw, ["x_ptr", "NUM_ROWS"])
    assert args == {"NUM_ROWS": 4}
    assert set(opts) == set(kw) - {"NUM_ROWS"}


def test_split_options_warns_on_option_like_typos_and_rejects_unknowns():
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        args, opts = options.split_options({"enableTurbo": True, "my_scratch": 1}, [])
        assert not args and not opts
        assert any("Unsupported runtime options ignored" in str(x.message) for x in w)
    with pytest.raises(TypeError):
        options.split_options({"bogus": 1}, [])
    with pytest.raises(ValueError):
        options.split_options({"target_artifact": "exe"}, [])


def test_option_field_list_matches_the_reference_dataclass():
    if not os.environ.get("HEXAGON_MLIR_REF"):
        pytest.skip("set HEXAGON_MLIR_REF to a checkout of the reference to run this check")
    ref = os.path.join(os.environ["HEXAGON_MLIR_REF"], "qcom_hexagon_backend/backend/hexagon_options.py")
    if not os.path.exists(ref):
        pytest.skip("reference checkout not present")
    import re

    fields = set(re.findall(r"^    (\w+): [\w\[\], \.]+ =", open(ref).read(), flags=re.M))
    assert fields == set(options.HEXAGON_OPTION_FIELDS)


def test_lookup_strips_the_dtype_suffix():
    assert kernels.lookup("softmax_kernel_float16").name == "softmax_kernel"
    assert kernels.lookup("layer_norm_fwd_kernel_float32").name == "layer_norm_fwd_kernel"
    assert kernels.lookup("matmul").name == "matmul"
    with pytest.raises(NotImplementedError):
        kernels.lookup("conv2d_kernel")


def test_launcher_binds_by_reference_parameter_names(monkeypatch):
    seen = {}
    monkeypatch.setattr(kernels.ops, "softmax", lambda x, out: seen.update(x=x, out=out))
    x, out = torch.zeros(4, 8), torch.zeros(4, 8)
    kernels.lookup("softmax_kernel_float32")[(4,)](x, out, NUM_ROWS=4, NUM_COLS=8, BLOCK_SIZE=8,
                                                   enableMultiThreading=False, enableHVXInlining=True)
    assert seen["x"] is x and seen["out"] is out
    with pytest.raises(TypeError):
        kernels.softmax_kernel[(1,)](x, out, NUM_ROWS=4)                     # NUM_COLS missing

    monkeypatch.setattr(kernels.ops, "layer_norm",
                        lambda x, y, w, b, mean, rstd, eps: seen.update(eps=eps, shape=tuple(x.shape)))
    flat = torch.zeros(27 * 16)
    kernels.layer_norm_fwd_kernel[(1,)](flat, flat.clone(), torch.zeros(16), torch.zeros(16), torch.zeros(27),
                                        torch.zeros(27), EPSILON=1e-5, NUM_ROWS=27, NUM_COLS=16, BLOCK_SIZE=16)
    assert seen["eps"] == 1e-5 and seen["shape"] == (27, 16)


def test_attention_launcher_selects_the_head_of_pid1(monkeypatch):
    calls = []

    def fake(q, k, v, o, sm_scale, causal):
        calls.append((q.clone(), causal))
        o.copy_(q)

    monkeypatch.setattr(kernels.ops, "attention", fake)
    Z, H, N, D = 2, 3, 8, 4
    q = torch.arange(Z * H * N * D, dtype=torch.float32).reshape(Z, H, N, D)
    out = torch.zeros_like(q)
    kernels.attention_fwd_kernel[(4,)](pid1=4, Q=q, K=q, V=q, sm_scale=0.5, Out=out, H=H, N_CTX=N, BLOCK_M=2,
                                       BLOCK_DMODEL=D, BLOCK_N=2, STAGE=1, stride_0=H * N * D, stride_1=N * D,
                                       stride_2=D, stride_3=1, enableHexKL=False)
    z, h = divmod(4, H)
    assert torch.equal(calls[0][0][0, 0], q[z, h]) and calls[0][1] is False
    assert torch.equal(out[z, h], q[z, h]) and out.sum() == q[z, h].sum()      # only that head was written


def test_triton_shim_routes_jit_kernels_by_name(monkeypatch):
    from hexb200 import triton_shim

    triton = triton_shim.install()
    from triton.backends.qcom_hexagon_backend.driver import HexagonDriver

    triton.runtime.driver.set_active(HexagonDriver())
    seen = {}
    monkeypatch.setattr(kernels.ops, "rms_norm", lambda x, y, w, eps: seen.update(eps=eps))

    @triton.jit
    def rms_norm_fwd_kernel(x_ptr, y_ptr, weights_ptr, BLOCK_SIZE, EPSILON, NUM_COLS, NUM_ROWS):
        raise AssertionError("the body of a jit function is never executed")

    rms_norm_fwd_kernel.__name__ = "rms_norm_fwd_kernel_float16"
    x = torch.zeros(3, 8)
    rms_norm_fwd_kernel[(4,)](x, x.clone(), torch.ones(8), EPSILON=1e-5, NUM_ROWS=3, NUM_COLS=8, BLOCK_SIZE=8,
                              enableHexagonmemCopyToDMA=True)
    assert seen["eps"] == 1e-5

    @triton.jit
    def _max(a, b):
        return a

    with pytest.raises(NotImplementedError):
        _max[(1,)](1, 2)


def test_host_tensors_reach_the_library_and_fail_loudly_without_a_gpu():
    if torch.cuda.is_available():
        pytest.skip("this check is for the GPU-less box")
    x = torch.rand(4, 8)
    with pytest.raises(hexb200.HexbError) as e:
        kernels.softmax_kernel[(1,)](x, torch.empty_like(x), NUM_ROWS=4, NUM_COLS=8, BLOCK_SIZE=8)
    assert e.value.status_name in ("HEXB_ERR_CUDA", "HEXB_ERR_NO_DEVICE")


def test_shard_range_covers_every_unit_once():
    for n in (0, 1, 7, 8, 128, 16384, 1001):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_range(n, world, r) for r in range(world)]
            assert sum(c for _, c in spans) == n
            pos = 0
            for s, c in spans:
                assert s == pos
                pos += c
            counts = [c for _, c in spans]
            assert max(counts) - min(counts) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _cpu_compute(name, O):
    """Stand-ins for the per-GPU kernels: the oracle's CPU calls on the rank's block."""
    if name == "softmax":
        return lambda x: O.torch_softmax(x)
    if name == "layernorm":
        return lambda x, weight, bias: O.torch_layer_norm(x, weight, bias, 1e-5)
    if name == "gemm":
        return lambda a, b: O.torch_matmul(a, b)
    if name == "attention":
        return lambda q, k, v: (O.torch_attention(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), q.shape[-1] ** -0.5, True)[0]
                                if q.shape[0] else q.clone())
    if name == "decoder":
        def run(x, weights):
            if x.shape[0] == 0:
                return x.clone()
            d, ff = weights[0]["wo"].shape[0], weights[0]["wd"].shape[0]
            return O.torch_decoder(x.contiguous(), weights, 2, d // 2, ff, x.shape[0], x.shape[1], 1e-6)
        return run
    raise KeyError(name)


def _small_inputs(name, units, O):
    """The five configurations at toy sizes with `units` partition units (same seeds on every rank)."""
    if name == "softmax":
        return {"x": O.make_softmax_inputs(units, 32, seed=77)}
    if name == "layernorm":
        x, w, b = O.make_layer_norm_inputs(units, 64, seed=78)
        return {"x": x, "weight": w, "bias": b}
    if name == "gemm":
        a, b = O.make_matmul_inputs(units, 24, 16, seed=79)
        return {"a": a, "b": b}
    if name == "attention":
        q, k, v = O.make_attention_inputs(1, units, 16, 8, seed=80)
        return {"q": q, "k": k, "v": v}
    x, ws = O.make_decoder_inputs(1, 16, 2, 32, units, 8, seed=81)
    return {"x": x, "weights": ws}


def _rank_main(rank, world, port, units, q):
    sys.path.insert(0, ROOT)
    from hexb200.dist import PARTITIONS, run_partitioned
    from oracle import oracle as O

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        res = {}
        for name in PARTITIONS:
            inputs = _small_inputs(name, units, O)                       # every rank draws the same tensors
            y = run_partitioned(name, inputs, _cpu_compute(name, O), world, rank)   # shard -> compute -> gather
            whole = run_partitioned(name, inputs, _cpu_compute(name, O), 1, 0, gather=False)
            if name == "attention":
                whole = whole.reshape(y.shape)
            res[name] = (bool(torch.allclose(y.float(), whole.float(), atol=1e-6)), tuple(y.shape))
        q.put((rank, res))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("units", [6, 5, 1])
def test_two_rank_shard_compute_gather_gloo(units):
    """The function the benchmark's multi-GPU leg uses (run_partitioned), on two CPU ranks over gloo,
    for all five configurations, with even, ragged and fewer-units-than-ranks partitions."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, units, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for _, per_name in res:
        for name, (ok, shape) in per_name.items():
            assert ok, name
            assert shape[0] == (1 if name == "attention" else units), (name, shape)


def test_partition_rejects_missing_operands_and_samples_every_rank():
    from hexb200.dist import partition, sample_units, units_of

    with pytest.raises(KeyError):
        partition("layernorm", {"x": torch.zeros(4, 4)}, 2, 0)
    q = torch.zeros(2, 3, 4, 8)
    assert units_of("attention", {"q": q}) == 6
    assert partition("attention", {"q": q, "k": q, "v": q}, 4, 3)["q"].shape == (1, 4, 8)
    for total, world in ((16384, 8), (128, 8), (8, 8), (3, 2), (1, 4)):
        picks = sample_units(total, world)
        owners = set()
        for u in picks:
            owners |= {r for r in range(world) if shard_range(total, world, r)[0] <= u < sum(shard_range(total, world, r))}
        assert owners == {r for r in range(world) if shard_range(total, world, r)[1] > 0}


def test_raw_tensor_file_round_trip(tmp_path):
    import struct

    from hexb200 import report

    for t in (torch.arange(24, dtype=torch.float32).reshape(2, 3, 4), torch.randn(5, 7).half(),
              torch.tensor(3.5), torch.arange(6, dtype=torch.int64), torch.empty(0, 4)):
        p = tmp_path / "t.raw"
        report.dump_tensor(str(p), t)
        back = report.load_tensor(str(p))
        assert back.dtype == t.dtype and back.shape == t.shape and torch.equal(back, t)
    # the header layout the reference's executor parses: u32 dtype id, i64 rank, i64 shape...
    report.dump_tensor(str(p), torch.zeros(2, 5, dtype=torch.float16))
    raw = p.read_bytes()
    assert struct.unpack("I", raw[:4])[0] == 1 and struct.unpack("q", raw[4:12])[0] == 2
    assert struct.unpack("qq", raw[12:28]) == (2, 5) and len(raw) == 28 + 20
    report.dump_input(str(p), torch.arange(8, dtype=torch.float32))
    assert torch.equal(report.load_input(str(p), torch.float32, (2, 4)), torch.arange(8.0).reshape(2, 4))
    p.write_bytes(b"\x63\x00\x00\x00" + b"\x00" * 8)
    with pytest.raises(ValueError):
        report.load_tensor(str(p))


def test_test_info_block():
    from hexb200 import report

    r = report.TestReport("softmax_kernel", 12.5, "us", "Pass")
    assert r.text() == "Test_Info: {\n\tName:softmax_kernel\n\tResult:Pass\n\tPerf:12.500000\n\tUnits:us\n}\n"
    back = report.TestReport.parse(r.text())
    assert (back.name, back.perf, back.units, back.result) == ("softmax_kernel", 12.5, "us", "Pass")
    with pytest.raises(ValueError):
        report.TestReport("x", 1.0, "us", "Maybe")


def test_gpt2_host_helpers():
    """The parts of the GPT-2 runner that need no GPU: weight naming, FLOP count, the acceptance rule."""
    import torch
    from hexb200 import gpt2

    cfg = gpt2.GPT2Config(n_layer=2, n_embd=64, n_head=4, n_positions=16, vocab_size=50)
    sd = gpt2.random_state_dict(cfg, seed=0)
    assert sd["transformer.h.1.attn.c_attn.weight"].shape == (64, 192)          # Conv1D: [in, out]
    assert sd["transformer.h.0.mlp.c_proj.weight"].shape == (256, 64)
    assert "lm_head.weight" not in sd                                            # tied to wte
    assert all(v.dtype == torch.float16 for v in sd.values())
    again = gpt2.random_state_dict(cfg, seed=0)
    assert all(torch.equal(sd[k], again[k]) for k in sd)                         # seeded
    # 2 layers x (qkv + proj + fc + proj2 + causal attention) + LM head, for 2 x 8 tokens
    T, d, V = 16, 64, 50
    per_layer = 2 * T * d * (3 * d + d + 4 * d + 4 * d) + 4 * 2 * 8 * 8 * d * 0.5
    assert gpt2.GPT2Runner.flops_of(cfg, 2, 8) == 2 * per_layer + 2 * T * d * V
    a = torch.zeros(1, 3, 50)
    a[0, -1, [7, 3, 9, 1, 4]] = torch.tensor([5.0, 4.0, 3.0, 2.0, 1.0])
    b = a.clone()
    assert gpt2.top5_match(a, b) == (True, True)
    b[0, -1, 7] = 5.1                                                            # within rtol 0.03
    assert gpt2.top5_match(a, b) == (True, True)
    b[0, -1, 3] = 6.0                                                            # order changes
    assert gpt2.top5_match(a, b)[0] is False
    with pytest.raises(KeyError):
        gpt2.GPT2Runner(cfg, {k: v for k, v in sd.items() if "ln_f" not in k}, device="cpu")
