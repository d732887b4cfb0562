/*
 * hexb.h -- C ABI of libhexb200: the hexagon-mlir kernel set (row softmax, LayerNorm, RMSNorm,
 * fp16 matmul, flash-attention forward, decoder block stack) as hand-written sm_100a CUDA kernels.
 *
 * Conventions (all entry points):
 *   - plain pointers and sizes, no C++ or torch types; every function returns an int status
 *     (HEXB_OK == 0, negative on error) and never aborts, traps or throws;
 *   - unless the name ends in `_host`, pointer arguments are DEVICE pointers on the current CUDA
 *     device; the call is asynchronous and ordered on `stream` (a cudaStream_t passed as void*,
 *     NULL = the legacy default stream);
 *   - strides are in ELEMENTS, with the meaning of the reference's memref strides
 *     (qcom_hexagon_backend: test/utils/dsp/include/common.h:15-27);
 *   - the caller owns every tensor; outputs are written in place, nothing is returned;
 *   - `_host` entry points take HOST pointers, stage the tensors through device memory that the
 *     library caches per device, and return after the result is back in host memory.
 *
 * Each declaration cites the reference interface it replaces (path inside qualcomm/hexagon-mlir).
 */
#ifndef HEXB_H_
#define HEXB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes.  Replaces: AEE_SUCCESS / AEE_ENOMEMORY / AEE_EFAILED returned by
 * hexkl_matmul_f16f16_f32 (qcom_hexagon_backend/bin/runtime/src/HexKLAPI.cpp:56-68) and the
 * abort-on-CHECK convention of the device runtime (bin/runtime/include/HexagonCommon.h:28-64). */
enum {
  HEXB_OK = 0,
  HEXB_ERR_BAD_ARG = -1,     /* null pointer, negative size, inconsistent strides            */
  HEXB_ERR_UNSUPPORTED = -2, /* shape or dtype outside what the kernels implement            */
  HEXB_ERR_MISALIGNED = -3,  /* pointer or stride not aligned as the entry point requires    */
  HEXB_ERR_CUDA = -4,        /* a CUDA runtime / driver call failed (see hexb_last_cuda_error) */
  HEXB_ERR_TIMEOUT = -5,     /* a device-side bounded wait gave up (see hexb_device_status)  */
  HEXB_ERR_WORKSPACE = -6,   /* workspace missing or too small                               */
  HEXB_ERR_NO_DEVICE = -7    /* no sm_100 device is current                                  */
};

/* dtype ids: the ids of the reference's raw tensor files (test/utils/dsp/include/tensor.h:26-38:
 * Float16 = 1, Float32 = 2, Int32 = 6; the other ids of that list name types no kernel here takes). */
enum { HEXB_DT_F16 = 1, HEXB_DT_F32 = 2, HEXB_DT_I32 = 6 /* hexb_cumsum only */ };

int hexb_version(void);
const char *hexb_status_string(int status);
/* Text of the last CUDA error seen by this thread inside the library ("" if none). */
const char *hexb_last_cuda_error(void);
/* Synchronises the current device, then reports and clears the sticky device-side status word
 * that bounded waits inside the tensor-core kernels set when they give up.  *out = HEXB_OK or
 * HEXB_ERR_TIMEOUT.  Replaces: DMAStatus out-param of the UserDMA runtime
 * (qcom_hexagon_backend/bin/runtime/include/RuntimeDMA.h:18). */
int hexb_device_status(int *out);
/* Self-test of that mechanism: launches one small CTA (producer / TMEM owner / consumer warps as in
 * the tensor-core kernels) whose only mbarrier is never arrived on.  The producer's wait runs out
 * after `limit_us` microseconds (1 .. 1 000 000), the other warps leave through the CTA's abort flag,
 * the common teardown releases the tensor memory, and the next hexb_device_status() reports
 * HEXB_ERR_TIMEOUT once.  The kernel returns by construction; nothing faults or traps.
 * Replaces: the 100 ms acquire timeout of the runtime's resource manager
 * (qcom_hexagon_backend/bin/runtime/src/HexagonAPI.cpp:57), the only bounded wait of the reference. */
int hexb_selftest_bounded_wait(int limit_us, void *stream);

/* ---- row softmax.  Replaces: softmax_kernel(x_ptr, output_ptr, NUM_ROWS, NUM_COLS, BLOCK_SIZE)
 * (test/python/triton/test_softmax.py:44-72) and online_softmax(...)
 * (test/python/triton/test_online_softmax.py:30-81).  y[r, :] = softmax(x[r, :]); fp32 math. */
int hexb_softmax_f32(const float *x, float *y, int64_t rows, int64_t cols, int64_t x_row_stride,
                     int64_t y_row_stride, void *stream);
int hexb_softmax_f16(const void *x, void *y, int64_t rows, int64_t cols, int64_t x_row_stride,
                     int64_t y_row_stride, void *stream);

/* ---- LayerNorm forward.  Replaces: layer_norm_fwd_kernel(x_ptr, y_ptr, weights_ptr, biases_ptr,
 * mean_ptr, rstd_ptr, BLOCK_SIZE, EPSILON, NUM_COLS, NUM_ROWS)
 * (test/python/triton/test_layer_norm.py:42-82).  Biased variance in the centred two-pass form,
 * fp32 statistics; mean/rstd (fp32, one per row) may be NULL. */
int hexb_layer_norm_f32(const float *x, float *y, const float *weight, const float *bias,
                        float *mean, float *rstd, int64_t rows, int64_t cols, int64_t x_row_stride,
                        int64_t y_row_stride, float eps, void *stream);
int hexb_layer_norm_f16(const void *x, void *y, const void *weight, const void *bias, float *mean,
                        float *rstd, int64_t rows, int64_t cols, int64_t x_row_stride,
                        int64_t y_row_stride, float eps, void *stream);

/* ---- RMSNorm forward.  Replaces: rms_norm_fwd_kernel(x_ptr, y_ptr, weights_ptr, BLOCK_SIZE,
 * EPSILON, NUM_COLS, NUM_ROWS) (test/python/triton/test_rms_norm.py:37-63). */
int hexb_rms_norm_f32(const float *x, float *y, const float *weight, int64_t rows, int64_t cols,
                      int64_t x_row_stride, int64_t y_row_stride, float eps, void *stream);
int hexb_rms_norm_f16(const void *x, void *y, const void *weight, int64_t rows, int64_t cols,
                      int64_t x_row_stride, int64_t y_row_stride, float eps, void *stream);

/* ---- fp16 matmul, fp32 accumulation.  C[M,N] = A[M,K] @ B[K,N] (+ residual), all row-major with
 * leading dimensions lda/ldb/ldc in elements.  out_dtype = HEXB_DT_F16 or HEXB_DT_F32.
 * `residual` (fp16, same shape and leading dimension as C when out is fp16) may be NULL.
 * Replaces: matmul(A, B, C, N_ROWS, N_COLUMNS, N_INNER) (test/python/triton/test_matmul.py:35-70)
 * and matmul_hexkl (docs/tutorials/triton/matmul_hexkl.md:61-97). */
int hexb_matmul_f16(const void *A, const void *B, void *C, const void *residual, int64_t M,
                    int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int out_dtype,
                    void *stream);

/* The same product with the weight given transposed: C[M,N] = A[M,K] @ Bt[N,K]^T (Bt row-major with
 * leading dimension ldbt).  Replaces: the `matmul(x, weight.T)` form of the HexKL macro test
 * (test/python/torch-mlir/test_hexkl_macro_matmul.py:24-28,51-69) and the transpose folding of
 * qcom_hexagon_backend/lib/Transforms/ScheduleMatmulForHVXPass.cpp. */
int hexb_matmul_f16_nt(const void *A, const void *Bt, void *C, const void *residual, int64_t M,
                       int64_t N, int64_t K, int64_t lda, int64_t ldbt, int64_t ldc, int out_dtype,
                       void *stream);

/* Linear layer in one launch: C = act(A @ W + bias) + residual.  W is [K, N] (ldw >= N), or [N, K]
 * (ldw >= K) when w_transposed != 0; bias is a [N] fp16 vector or NULL; residual as for
 * hexb_matmul_f16; act 0 = none, 1 = GELU in the tanh form of gelu_kernel
 * (test/python/triton/test_gelu.py:25-54).  Replaces: the addmm / gelu / add chains of the GPT-2 graph
 * the reference compiles through torch-mlir (test/python/torch-mlir/gpt2lmheadmodel.py:143-169) and
 * lowers op by op to linalg generics around hexkl matmuls.
 * C may be the residual buffer itself (x = x + A @ W + bias in place: every element is read by the warp
 * that later stores it); C must not overlap A, W or bias. */
int hexb_linear_f16(const void *A, const void *W, const void *bias, const void *residual, void *C,
                    int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldw, int64_t ldc,
                    int w_transposed, int act, int out_dtype, void *stream);

/* Gate/up projection with the SwiGLU gating fused into the epilogue:
 *   out[M, F] = silu(A @ B[:, 0:F]) * (A @ B[:, F:2F]),  B = [K, 2F] row-major (columns gate|up).
 * fp32 accumulation and gating, one rounding to fp16.  Composed from matmul
 * (test/python/triton/test_matmul.py:35-70) and silu_kernel (test/python/triton/test_silu.py:38-52);
 * the reference has no fused form.  Requires F, lda, ldb multiples of 8 and 16-byte aligned A, B. */
int hexb_matmul_swiglu_f16(const void *A, const void *B_gate_up, void *out, int64_t M, int64_t F,
                           int64_t K, int64_t lda, int64_t ldb, int64_t ldo, void *stream);

/* Symbol-level drop-in for the HexKL runtime call: same name, argument order (rows, cols, inner,
 * out first) and fp32 output; device pointers, legacy default stream.
 * Replaces: hexkl_matmul_f16f16_f32 (qcom_hexagon_backend/bin/runtime/include/HexKLAPI.h:16-21). */
int hexkl_matmul_f16f16_f32(int64_t n_row, int64_t n_col, int64_t n_inner, float *outM,
                            const void *inAct, const void *inW);

/* ---- flash-attention forward, fp16 in/out, fp32 online softmax in base 2.
 * Tensors are [Z, H, N_CTX, D] addressed as base + z*stride_z + h*stride_h + n*stride_n + d
 * (innermost stride 1), one stride triple per tensor: strides[0..2] = Q, [3..5] = K, [6..8] = V,
 * [9..11] = Out.  causal != 0 masks keys above the diagonal (the additive -inf mask of
 * tm_tensor.attention).  Replaces: attention_fwd_kernel(pid1, Q, K, V, sm_scale, Out, H, N_CTX,
 * BLOCK_M, BLOCK_DMODEL, BLOCK_N, STAGE, stride_0..3) with _attn_fwd_inner
 * (test/python/triton/test_flash_attention.py:37-168), the fp16 form
 * test/python/mlir/hexkl_attention/input.mlir:5-168, and tm_tensor.attention
 * (qcom_hexagon_backend/lib/Transforms/LowerTmTensor.cpp:70-235). */
int hexb_attention_fwd_f16(const void *Q, const void *K, const void *V, void *Out, int64_t Z,
                           int64_t H, int64_t N_CTX, int64_t D, const int64_t *strides,
                           float sm_scale, int causal, void *stream);
/* fp32 tensors (the dtype of the reference's own Triton test); same argument meaning. */
int hexb_attention_fwd_f32(const float *Q, const float *K, const float *V, float *Out, int64_t Z,
                           int64_t H, int64_t N_CTX, int64_t D, const int64_t *strides,
                           float sm_scale, int causal, void *stream);

/* ---- generalised forward: separate query and key lengths, fp16 or fp32 output from fp16 inputs, and an
 * optional additive mask: Out = softmax(Q.K^T * sm_scale + mask) . V, the mask added before the row
 * maximum exactly as the lowering of tm_tensor.attention does
 * (qcom_hexagon_backend/lib/Transforms/LowerTmTensor.cpp:126-160 scale, add mask, max, exp, sum, divide;
 * op definition include/hexagon/Dialect/TmTensor/IR/TmTensorOps.td:27-55: Q [batch, seq_q, d],
 * K/V [batch, seq_kv, d], mask [batch, seq_q, seq_kv], scale 1/sqrt(d)).  fp16 inputs with fp32 output
 * is the form of test/python/mlir/hexkl_attention/input.mlir:5 (memref<*xf16> x3, memref<*xf32>).
 * Tensors are [Z, H, N, D] as for hexb_attention_fwd_f16 (a rank-3 tm_tensor operand is H = 1);
 * the mask is [Z, H, N_Q, N_KV] addressed as mask + z*ms[0] + h*ms[1] + q*ms[2] + kv in elements of
 * mask_dtype (a stride of 0 broadcasts that dimension).  mask == NULL: no mask.  causal != 0
 * additionally drops keys kv > q.  A row whose keys are all masked to -inf yields NaN, as the
 * reference's exp(-inf - -inf) does.  in_dtype F32 requires out_dtype F32. */
typedef struct hexb_attention_desc {
  const void *Q, *K, *V;
  void *Out;
  const void *mask;
  int64_t Z, H, N_Q, N_KV, D;
  int64_t strides[12];       /* Q, K, V, Out: (z, h, n) each */
  int64_t mask_strides[3];   /* (z, h, q) */
  int in_dtype, out_dtype, mask_dtype;
  float sm_scale;
  int causal;
} hexb_attention_desc;
int hexb_attention_fwd_ex(const hexb_attention_desc *desc, void *stream);

/* ---- SiLU and SwiGLU gating.  Replaces: silu_kernel(x_ptr, output_ptr, BLOCK_SIZE)
 * (test/python/triton/test_silu.py:38-52).  hexb_swiglu_f16: out[r, c] = silu(gu[r, c]) *
 * gu[r, c + cols] for a [rows, 2*cols] gate|up matrix. */
int hexb_silu_f32(const float *x, float *y, int64_t n, void *stream);
int hexb_silu_f16(const void *x, void *y, int64_t n, void *stream);
int hexb_swiglu_f16(const void *gate_up, void *out, int64_t rows, int64_t cols, void *stream);

/* ---- elementwise operators of the remaining Triton tests (dtype = HEXB_DT_F16 / HEXB_DT_F32;
 * contiguous vectors of n elements; fp32 arithmetic, one rounding).
 * hexb_unary replaces: gelu_kernel (test/python/triton/test_gelu.py:25-54, tanh form),
 * cos_kernel / sin_kernel (test_math_ops.py:24-37), rsqrt_kernel (test_rsqrt.py:19-24).
 * hexb_binary replaces: add_kernel (test_vec_add.py:19-25), add_kernel_scalar
 * (test_vec_add_with_scalar.py:31-46), add_2d_kernel (test_vec_add_2d.py:21-56), div_kernel
 * (test_vec_div_2d.py:20-55).
 * hexb_sum replaces: sum_kernel (test_sum.py:31-36): out[0] = sum(x), fp32 accumulation.
 * hexb_rope replaces: rope_kernel (test_rope.py:98-190): interleaved-pair rotary embedding of a
 * [B, L, H, D] tensor (unit innermost stride; strides[0..2] = batch, position, head in elements),
 * angle = position * theta^(-(d - d%2)/D). */
enum { HEXB_OP_GELU_TANH = 1, HEXB_OP_COS = 2, HEXB_OP_SIN = 3, HEXB_OP_RSQRT = 4 };
enum { HEXB_OP_ADD = 1, HEXB_OP_SUB = 2, HEXB_OP_MUL = 3, HEXB_OP_DIV = 4 };
int hexb_unary(int op, int dtype, const void *x, void *y, int64_t n, void *stream);
int hexb_binary(int op, int dtype, const void *a, const void *b, void *y, int64_t n, void *stream);
int hexb_sum(int dtype, const void *x, void *out, int64_t n, void *stream);
/* out[i] = i for i < n.  Replaces: flatten_pid(ptr) launched on a 1-, 2- or 3-D grid, where every
 * program stores its flattened id at that index (test/python/triton/test_multidim_grid.py:21-37). */
int hexb_iota(int dtype, void *out, int64_t n, void *stream);
int hexb_rope(int dtype, const void *x, void *out, int64_t B, int64_t L, int64_t H, int64_t D,
              const int64_t *x_strides, const int64_t *out_strides, float theta, void *stream);

/* ---- token + position embedding: out[t, :] = wte[ids[t], :] + wpe[t % seq, :] for fp16 tables
 * wte [vocab, d_model], wpe [n_positions, d_model] and int64 ids [n_tokens] (n_tokens = batch * seq).
 * An id outside [0, vocab) writes a zero row and makes hexb_device_status report HEXB_ERR_BAD_ARG.
 * Replaces: the two embedding gathers and their sum at the top of the GPT-2 graph
 * (test/python/torch-mlir/gpt2lmheadmodel.py:143-169). */
int hexb_embedding_f16(const void *wte, const void *wpe, const int64_t *ids, void *out, int64_t n_tokens,
                       int64_t seq, int64_t d_model, int64_t vocab, int64_t n_positions, void *stream);

/* ---- cumulative sum along one axis.  The tensor is viewed as [outer, len, inner] (contiguous);
 * y[o, l, i] = x[o, 0, i] + ... + x[o, l, i], or from the far end when reverse != 0.
 * dtype = HEXB_DT_F32, HEXB_DT_F16 (fp32 accumulation, one rounding per output) or HEXB_DT_I32
 * (exact, wrapping).  Replaces: ttx.cumsum {axis}
 * (qcom_hexagon_backend/include/hexagon/Dialect/TTX/IR/TTXOps.td:61-75, lowering
 * lib/Transforms/LowerTTX.cpp:179-300) and ttx.scan {axis, reverse} with an addition body
 * (TTXOps.td:25-40, LowerTTX.cpp:75-176). */
int hexb_cumsum(int dtype, const void *x, void *y, int64_t outer, int64_t len, int64_t inner,
                int reverse, void *stream);

/* ---- decoder-only block stack, forward.  Pre-norm blocks:
 *   h = x + Wo . Attn(RMSNorm(x) . Wqkv);  x' = h + Wd . (SiLU(Wg . n) * (Wu . n)), n = RMSNorm(h)
 * causal attention, no bias, fp16 storage, fp32 accumulation and statistics.
 * Per layer l the weights are row-major fp16: wqkv[l] [d_model, 3*d_model] (columns q|k|v, head-major),
 * wo[l] [d_model, d_model], wgu[l] [d_model, 2*d_ff] (columns gate|up), wd[l] [d_ff, d_model],
 * g1[l], g2[l] [d_model] RMSNorm gains.  x and out are [batch*seq, d_model] fp16.
 * No single reference function: composed from rms_norm_fwd_kernel, matmul, attention_fwd_kernel and
 * silu_kernel above, the way test/python/torch-mlir/gpt2lmheadmodel.py:143-169 runs a whole model. */
typedef struct hexb_decoder_config {
  int32_t n_layers, d_model, n_heads, head_dim, d_ff, batch, seq;
  float rms_eps;
} hexb_decoder_config;

typedef struct hexb_decoder_weights { /* arrays of n_layers device pointers (host arrays) */
  const void *const *wqkv, *const *wo, *const *wgu, *const *wd, *const *g1, *const *g2;
} hexb_decoder_weights;

size_t hexb_decoder_workspace_bytes(const hexb_decoder_config *cfg);
int hexb_decoder_forward_f16(const hexb_decoder_config *cfg, const hexb_decoder_weights *w,
                             const void *x, void *out, void *workspace, size_t workspace_bytes,
                             void *stream);

/* ---- decoder forward for callers that must not allocate.  No counterpart in the reference.
 * Same computation and arguments as hexb_decoder_forward_f16, minus the workspace pair: the
 * intermediate activations live in a fixed HEXB_DECODER_STATIC_SCRATCH_BYTES array that is part of
 * the library image on every GPU that loads it (held until the process exits).  It is meant for
 * hosts that hand all device memory to their own pool at start-up, or that sit in a serving loop
 * where a cudaMalloc -- which may fail, fragment, or synchronise the device -- is not acceptable:
 * this call never calls cudaMalloc, cudaFree or any allocating library routine.
 *   - A configuration whose hexb_decoder_workspace_bytes() exceeds the array is refused with
 *     HEXB_ERR_WORKSPACE and nothing is launched (64 MiB: e.g. 862 tokens at d_model 2048 /
 *     d_ff 8192, or 10082 tokens at d_model 256 / d_ff 512).
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress,
 *     with that device current) and caches it; make that first call before starting any stream
 *     capture.  With the CUDA runtime's lazy module loading that first call is also the moment the
 *     driver instantiates the library's image on the device -- the array itself, the kernels' code
 *     and their function attributes -- so a host that hands the device's memory to its own pool must
 *     make one call (a tiny configuration will do) BEFORE it claims the rest of the memory;
 *     afterwards no call changes the amount of free device memory.
 *   - All calls on a device share the one array.  It keeps whatever the previous call left there;
 *     the block stack writes every intermediate before reading it, so nothing has to be cleared.
 *     Two calls that overlap on the GPU (different streams, or different host threads) race on
 *     the array: serialise them. */
#define HEXB_DECODER_STATIC_SCRATCH_BYTES (64u << 20)
int hexb_decoder_forward_f16_noalloc(const hexb_decoder_config *cfg, const hexb_decoder_weights *w,
                                     const void *x, void *out, void *stream);

/* ---- host-buffer entry points (the launcher path).  Replace the generated wrapper main() that
 * loads `<kernel>_t{i}.raw`, runs the kernel and dumps `<kernel>_o{i}.raw`
 * (qcom_hexagon_backend/backend/triton_hexagon_launcher.py:111-123,
 *  backend/hexagon_launcher_base.py:430-437): tensors cross the host/device boundary inside.
 * Tensors are contiguous and row-major.  Rows, 256-row blocks of A and (batch, head) pairs are cut into
 * pieces (option "host_chunks", default 8) whose upload, kernel and download overlap on three streams;
 * the overlap needs page-locked host memory (cudaHostAlloc / cudaHostRegister), pageable memory gives
 * the same result with the pieces one after the other.  One call at a time per process (a lock). */
int hexb_softmax_host(int dtype, const void *x, void *y, int64_t rows, int64_t cols);
int hexb_layer_norm_host(int dtype, const void *x, void *y, const void *weight, const void *bias,
                         float *mean, float *rstd, int64_t rows, int64_t cols, float eps);
int hexb_rms_norm_host(int dtype, const void *x, void *y, const void *weight, int64_t rows,
                       int64_t cols, float eps);
int hexb_matmul_f16_host(const void *A, const void *B, void *C, int64_t M, int64_t N, int64_t K,
                         int out_dtype);
int hexb_attention_fwd_host(int dtype, const void *Q, const void *K, const void *V, void *Out,
                            int64_t Z, int64_t H, int64_t N_CTX, int64_t D, float sm_scale,
                            int causal);
/* Releases the cached staging memory of the current device. */
int hexb_host_staging_release(void);

/* ---- variant switches: selects a kernel variant by name ("attn_kernel", "gemm_pair", "norm_ring",
 * "pdl", ...; the table is in INTEGRATION.md).  Every value of every key computes the same result by
 * another route.  Unknown keys return HEXB_ERR_BAD_ARG; hexb_get_option returns HEXB_ERR_BAD_ARG for a
 * key that was never set (the launchers then use their built-in defaults).  Replaces: the per-launch HexagonOptions overrides
 * (qcom_hexagon_backend/backend/hexagon_options.py:16-107). */
int hexb_set_option(const char *key, int value);
int hexb_get_option(const char *key, int *value);

#ifdef __cplusplus
}
#endif
#endif /* HEXB_H_ */
