"""GPU: the reference's own tests, restated.  Same launch syntax (`@triton.jit` kernel defined in the
test, `kernel[grid](...)` with HexagonDriver active and HexagonOptions flags as keywords), same
shapes, same CPU tensors, same tolerances as test/python/triton/test_{softmax,online_softmax,
layer_norm,rms_norm,matmul,flash_attention,silu}.py and docs/tutorials/triton/matmul_hexkl.md of
qualcomm/hexagon-mlir.  The kernel bodies are placeholders: with the shim installed the decorated
function is never compiled, its name selects the CUDA implementation."""
import pytest
import torch
import torch.nn.functional as F

from hexb200 import triton_shim

triton = triton_shim.install()
from triton.backends.qcom_hexagon_backend.driver import HexagonDriver  # noqa: E402

triton.runtime.driver.set_active(HexagonDriver())

pytestmark = pytest.mark.gpu


def parameterize_func_name(dtype):
    names = {torch.float16: "float16", torch.float32: "float32"}

    def deco(fn):
        fn.__name__ += "_" + names[dtype]
        return fn

    return deco


@pytest.fixture(autouse=True)
def _seed():
    assert torch.cuda.is_available()
    torch.manual_seed(0)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_softmax(dtype):
    NUM_THREADS, NUM_ROWS, NUM_COLS = 4, 128, 128

    @triton.jit
    @parameterize_func_name(dtype)
    def softmax_kernel(x_ptr, output_ptr, NUM_ROWS, NUM_COLS, BLOCK_SIZE):
        ...

    x = torch.rand(NUM_ROWS, NUM_COLS, dtype=dtype)
    output = torch.empty_like(x, dtype=dtype)
    softmax_kernel[(NUM_THREADS,)](
        x, output, NUM_ROWS=NUM_ROWS, NUM_COLS=NUM_COLS, BLOCK_SIZE=triton.next_power_of_2(NUM_COLS),
        enableMultiThreading=False, enableVTCMTiling=False, enableConvertToHexagonmem=False,
        enableHexagonmemCopyToDMA=False, enableHVXInlining=True, enableSCFLoopUnroll=True,
        enableSplitReduceGeneric=True)
    reference = F.softmax(x, dim=1, dtype=dtype)
    assert torch.allclose(output, reference, atol=1e-3 if dtype == torch.float16 else 1e-5)


@pytest.mark.parametrize("num_threads", [1, 4])
def test_online_softmax(num_threads):
    @triton.jit
    def online_softmax(x_ptr, output_ptr, NUM_ROWS, NUM_COLS, BLOCK_ROW_SIZE, BLOCK_COL_SIZE):
        ...

    x = torch.rand(128, 128)
    output = torch.empty_like(x)
    single = num_threads == 1
    online_softmax[(num_threads,)](
        x, output, NUM_ROWS=128, NUM_COLS=128, BLOCK_ROW_SIZE=128 // num_threads,
        BLOCK_COL_SIZE=128 // num_threads, enableMultiThreading=single, enableVTCMTiling=single,
        enableConvertToHexagonmem=single, enableHexagonmemCopyToDMA=single)
    assert torch.allclose(output, F.softmax(x, dim=1), atol=1e-5)


@pytest.mark.parametrize("num_cols", [8192])
@pytest.mark.parametrize("num_threads", [1, 4])
@pytest.mark.parametrize("dtype", [torch.float32])
def test_layer_norm(num_cols, num_threads, dtype):
    EPSILON, NUM_ROWS = 1e-5, 27

    @triton.jit
    @parameterize_func_name(dtype)
    def layer_norm_fwd_kernel(x_ptr, y_ptr, weights_ptr, biases_ptr, mean_ptr, rstd_ptr, BLOCK_SIZE, EPSILON,
                              NUM_COLS, NUM_ROWS):
        ...

    x = torch.rand(NUM_ROWS, num_cols, dtype=dtype)
    output = torch.empty_like(x, dtype=dtype)
    weights = torch.rand(num_cols, dtype=dtype)
    biases = torch.rand(num_cols, dtype=dtype)
    means = torch.empty(NUM_ROWS, dtype=dtype)
    rstds = torch.empty(NUM_ROWS, dtype=dtype)
    single = num_threads == 1
    layer_norm_fwd_kernel[(num_threads,)](
        x, output, weights, biases, means, rstds, EPSILON=EPSILON, NUM_ROWS=NUM_ROWS, NUM_COLS=num_cols,
        BLOCK_SIZE=triton.next_power_of_2(num_cols), enableMultiThreading=single, enableVTCMTiling=single,
        enableConvertToHexagonmem=single, enableHexagonmemCopyToDMA=single)
    reference = F.layer_norm(x, (num_cols,), weight=weights, bias=biases, eps=EPSILON)
    assert torch.allclose(output, reference, atol=1e-5)
    assert torch.allclose(means, x.mean(dim=1), atol=1e-5)             # the side outputs of the kernel
    assert torch.allclose(rstds, 1 / torch.sqrt(x.var(dim=1, unbiased=False) + EPSILON), rtol=1e-4)


@pytest.mark.parametrize("num_threads", [1, 4])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_rms_norm(num_threads, dtype):
    EPSILON, NUM_ROWS, NUM_COLS = 1e-5, 127, 513

    @triton.jit
    @parameterize_func_name(dtype)
    def rms_norm_fwd_kernel(x_ptr, y_ptr, weights_ptr, BLOCK_SIZE, EPSILON, NUM_COLS, NUM_ROWS):
        ...

    x = torch.rand(NUM_ROWS, NUM_COLS, dtype=dtype)
    output = torch.empty_like(x, dtype=dtype)
    weights = torch.rand(NUM_COLS, dtype=dtype)
    single = num_threads == 1
    rms_norm_fwd_kernel[(num_threads,)](
        x, output, weights, EPSILON=EPSILON, NUM_ROWS=NUM_ROWS, NUM_COLS=NUM_COLS,
        BLOCK_SIZE=triton.next_power_of_2(NUM_COLS), enableMultiThreading=single, enableVTCMTiling=single,
        enableConvertToHexagonmem=single, enableHexagonmemCopyToDMA=True)
    reference = F.rms_norm(x, (NUM_COLS,), weight=weights, eps=EPSILON)
    assert torch.allclose(output, reference, atol=1e-2)


@pytest.mark.parametrize("num_rows,num_cols,num_inner", [(1024, 512, 64)])
def test_matmul(num_rows, num_cols, num_inner):
    @triton.jit
    def matmul(A, B, C, N_ROWS, N_COLUMNS, N_INNER):
        ...

    mat_A = torch.rand((num_rows, num_inner), dtype=torch.float16)
    mat_B = torch.rand((num_inner, num_cols), dtype=torch.float16)
    mat_C = torch.zeros((num_rows, num_cols), dtype=torch.float16)
    matmul[(1,)](mat_A, mat_B, mat_C, num_rows, num_cols, num_inner, enableMultiThreading=True,
                 enableVTCMTiling=True, enableConvertToHexagonmem=True, enableHexagonmemCopyToDMA=True)
    assert torch.allclose(mat_C, torch.matmul(mat_A, mat_B), atol=2e-1)


def test_matmul_hexkl():
    N_ROWS, N_COLUMNS, N_INNER = 1024, 512, 64

    @triton.jit
    def matmul_hexkl(A, B, C, N_ROWS, N_COLUMNS, N_INNER):
        ...

    mat_A = torch.rand((N_ROWS, N_INNER), dtype=torch.float16)
    mat_B = torch.rand((N_INNER, N_COLUMNS), dtype=torch.float16)
    mat_C = torch.zeros((N_ROWS, N_COLUMNS), dtype=torch.float32)
    matmul_hexkl[(1,)](mat_A, mat_B, mat_C, N_ROWS, N_COLUMNS, N_INNER, enableHexKL=True, iterations=1)
    assert torch.allclose(mat_C, torch.matmul(mat_A, mat_B).to(torch.float32), rtol=1e-2)


def test_flash_attention():
    Z, H, N_CTX, D_HEAD = 1, 1, 1024, 64
    NUM_THREADS, BLOCK_N, SCALE = 4, 64, 0.5

    @triton.jit
    def attention_fwd_kernel(pid1, Q, K, V, sm_scale, Out, H, N_CTX, BLOCK_M, BLOCK_DMODEL, BLOCK_N, STAGE,
                             stride_0, stride_1, stride_2, stride_3):
        ...

    query = torch.rand(Z, H, N_CTX, D_HEAD)
    key = torch.rand(Z, H, N_CTX, D_HEAD)
    value = torch.rand(Z, H, N_CTX, D_HEAD)
    output = torch.zeros_like(query)
    attention_fwd_kernel[(NUM_THREADS,)](
        pid1=0, Q=query, K=key, V=value, sm_scale=SCALE, Out=output, H=H, N_CTX=N_CTX,
        BLOCK_M=N_CTX // NUM_THREADS, BLOCK_DMODEL=D_HEAD, BLOCK_N=BLOCK_N, STAGE=1,
        stride_0=H * N_CTX * D_HEAD, stride_1=N_CTX * D_HEAD, stride_2=D_HEAD, stride_3=1,
        enableVectorization=True, enableSplitReduceGeneric=True, enableHVXInlining=True,
        enableSCFLoopUnroll=True, enableMultiThreading=True, enableHexKL=False, enableVTCMTiling=False,
        enableConvertToHexagonmem=False, enableHexagonmemCopyToDMA=False)
    reference = F.scaled_dot_product_attention(query, key, value, scale=SCALE)
    # the reference asserts with allclose defaults; a different summation order of the same fp32
    # arithmetic needs the absolute floor lifted from 1e-8 to 1e-6
    assert torch.allclose(output, reference, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("num_elements,num_threads", [(16384, 1), (16384, 4)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_silu(num_elements, num_threads, dtype):
    @triton.jit
    @parameterize_func_name(dtype)
    def silu_kernel(x_ptr, output_ptr, BLOCK_SIZE):
        ...

    x = torch.rand(num_elements, dtype=dtype)
    output = torch.empty_like(x, dtype=dtype)
    silu_kernel[(num_threads,)](x, output, BLOCK_SIZE=triton.next_power_of_2(num_elements // num_threads),
                                enableMultiThreading=num_threads == 1)
    assert torch.allclose(output, F.silu(x), atol=1e-2)


# ------------------------------------------------------------------ the remaining Triton-test kernels
def test_gelu_block_ptr():
    """test_gelu_block_ptr.py: one program, block pointers over an [N, H, W, C] fp16 tensor."""
    N, H, W, C = 16, 16, 128, 2

    @triton.jit
    def gelu_bptr_kernel(x_ptr, output_ptr, N, H, W, C):
        ...

    x = torch.rand(N, H, W, C, dtype=torch.float16)
    output = torch.empty_like(x, dtype=torch.float16)
    gelu_bptr_kernel[(1,)](x, output, N, H, W, C)
    assert torch.allclose(output, F.gelu(x.float(), approximate="tanh").half(), atol=1e-2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_libd_gelu(dtype):
    """test_libd_gelu.py: the GELU formula with libdevice.tanh, 4 programs."""
    NUM_ELEMENTS, NUM_THREADS = 16384, 4

    @triton.jit
    @parameterize_func_name(dtype)
    def libd_gelu_kernel(x_ptr, output_ptr, BLOCK_SIZE):
        ...

    x = torch.rand(NUM_ELEMENTS, dtype=dtype)
    output = torch.empty_like(x, dtype=dtype)
    libd_gelu_kernel[(NUM_THREADS,)](x, output, BLOCK_SIZE=NUM_ELEMENTS // NUM_THREADS, enableVTCMTiling=False,
                                     enableConvertToHexagonmem=False)
    assert torch.allclose(output, F.gelu(x, approximate="tanh"), atol=1e-2 if dtype == torch.float16 else 1e-5)


def test_vec_add_multithread():
    NUM_ELEMENTS, NUM_THREADS = 16384, 4

    @triton.jit
    def add_kernel_mulithreaded(x_ptr, y_ptr, output_ptr, BLOCK_SIZE):
        ...

    x, y = torch.rand(NUM_ELEMENTS), torch.rand(NUM_ELEMENTS)
    output = torch.empty_like(x)
    add_kernel_mulithreaded[(NUM_THREADS,)](x, y, output, BLOCK_SIZE=NUM_ELEMENTS // NUM_THREADS,
                                            enableMultiThreading=False, enableVTCMTiling=False,
                                            enableConvertToHexagonmem=False, enableHexagonmemCopyToDMA=False)
    assert torch.allclose(output, x + y)


@pytest.mark.parametrize("use_scratch", [False, True], ids=["no-scratch", "vtcm-scratch"])
@pytest.mark.parametrize("grid", [(1,), (2,), (4,)], ids=["grid1", "grid2", "grid4"])
def test_static_allocator_vadd(grid, use_scratch):
    """test_static_allocator_vadd.py: add_kernel(x, y, out, n_elements, block_size=...) with a scratch option."""

    @triton.jit
    def add_kernel(x_ptr, y_ptr, output_ptr, n_elements, block_size):
        ...

    N = 131072
    x, y = torch.rand(N), torch.rand(N)
    output = torch.empty_like(x)
    alignment = 2048
    per_instance_vtcm = (1 * 1024 * 1024) & ~(alignment - 1)
    scratch = per_instance_vtcm if use_scratch else 0
    add_kernel[grid](x, y, output, N, block_size=N // grid[0], enableHexagonmemCopyToDMA=False, scratch=scratch)
    assert torch.allclose(output, x + y)


def test_multidim_grid():
    """test_multidim_grid.py: every program of a (10, 5, 2) grid stores its flattened id."""
    GRID = (10, 5, 2)

    @triton.jit
    def flatten_pid(ptr):
        ...

    num_elements = 100
    result = torch.zeros(num_elements)
    flatten_pid[GRID](result, enableVTCMTiling=True, enableConvertToHexagonmem=True, enableHexagonmemCopyToDMA=True)
    assert torch.allclose(result, torch.arange(num_elements, dtype=torch.float))


# ------------------------------------------------------------------ the single-operator torch-mlir tests
# test/python/torch-mlir/test_{gelu,softmax,layernorm}_torch.py compile a one-node torch module and compare
# with eager PyTorch on a 128 x 128 fp16 input; here the node is the library call, the comparison is theirs.
def test_gelu_torch_case():
    from hexb200 import ops
    inp = torch.rand(128, 128, dtype=torch.float16)
    out = torch.empty_like(inp)
    ops.unary("gelu_tanh", inp, out)
    assert torch.allclose(out, torch.nn.GELU(approximate="tanh")(inp), rtol=1e-4, atol=1e-3)


def test_softmax_torch_case():
    from hexb200 import ops
    inp = torch.rand(128, 128, dtype=torch.float16)
    out = torch.empty_like(inp)
    ops.softmax(inp, out)
    assert torch.allclose(out, torch.nn.Softmax(dim=1)(inp.float()).half(), rtol=1e-3, atol=1e-3)


def test_layernorm_torch_case():
    from hexb200 import ops
    model = torch.nn.LayerNorm(normalized_shape=128)
    inp = torch.rand(128, 128, dtype=torch.float16)
    out = torch.empty_like(inp)
    ops.layer_norm(inp, out, model.weight.detach().half(), model.bias.detach().half(), eps=model.eps)
    ref = model(inp.float()).half()
    assert torch.allclose(out, ref, rtol=5e-1, atol=1e-2)          # the reference's own (loose) bound
    assert torch.allclose(out, ref, rtol=1e-2, atol=2e-3)          # what this kernel actually holds
