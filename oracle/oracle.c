/*
 * oracle.c -- TEST INFRASTRUCTURE, not product code.
 *
 * A plain-C, CPU restatement of the algorithms of the hexagon-mlir kernel set, written from the
 * reference's operator definitions so that the CUDA kernels can be checked against them.  Only
 * tests, the smoke check and the CPU-baseline leg of the benchmark may call into this file; the
 * library never does.  Each function cites the reference source it follows (paths inside
 * qualcomm/hexagon-mlir).  Loops are written for clarity; `omp parallel for` on the outermost
 * independent loop only lets the baseline use the host's cores and does not change any result.
 *
 * Parity status: pinned against torch CPU eager (the comparator of the reference's own tests) and
 * against outputs of the reference's Triton kernels run in Triton's interpreter
 * (tests/golden/).  Parity with the Hexagon NPU's approximations (Quake rsqrt, qhmath, fp16 HMX
 * accumulation) is unpinned: no Hexagon toolchain, simulator or device output exists to pin it.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef _Float16 f16;

/* ------------------------------------------------------------------ softmax
 * softmax_kernel, test/python/triton/test_softmax.py:58-72:
 *   z = x - max(x); num = exp(z.to(f32)).to(x.dtype); denom = sum(num); y = num / denom. */
void oracle_softmax_f32(const float *x, float *y, int64_t rows, int64_t cols) {
#pragma omp parallel for
  for (int64_t r = 0; r < rows; ++r) {
    const float *xr = x + r * cols;
    float *yr = y + r * cols;
    float m = -INFINITY;
    for (int64_t c = 0; c < cols; ++c) m = fmaxf(m, xr[c]);
    double dsum = 0.0; /* the reduction order of tl.sum is unspecified: sum exactly, round once */
    for (int64_t c = 0; c < cols; ++c) {
      yr[c] = expf(xr[c] - m);
      dsum += yr[c];
    }
    const float denom = (float)dsum;
    for (int64_t c = 0; c < cols; ++c) yr[c] = yr[c] / denom;
  }
}

/* fp16 data: the subtraction happens in fp16, exp in fp32 and is cast back to fp16 before the sum
 * (test_softmax.py:67-69); the sum of fp16 values accumulates in fp32
 * (docs/tutorials/triton/softmax.md:196-204); the quotient is rounded to fp16. */
void oracle_softmax_f16(const f16 *x, f16 *y, int64_t rows, int64_t cols) {
#pragma omp parallel for
  for (int64_t r = 0; r < rows; ++r) {
    const f16 *xr = x + r * cols;
    f16 *yr = y + r * cols;
    f16 m = (f16)-INFINITY;
    for (int64_t c = 0; c < cols; ++c) m = xr[c] > m ? xr[c] : m;
    float denom = 0.f;
    for (int64_t c = 0; c < cols; ++c) {
      const f16 z = (f16)(xr[c] - m);
      yr[c] = (f16)expf((float)z);
      denom += (float)yr[c];
    }
    for (int64_t c = 0; c < cols; ++c) yr[c] = (f16)((float)yr[c] / denom);
  }
}

/* online_softmax, test/python/triton/test_online_softmax.py:53-80: running (m_i, l_i) over column
 * blocks of width block_cols, then y = exp(x - m_i) / l_i. */
void oracle_online_softmax_f32(const float *x, float *y, int64_t rows, int64_t cols, int64_t block_cols) {
  if (block_cols <= 0) block_cols = cols;
#pragma omp parallel for
  for (int64_t r = 0; r < rows; ++r) {
    const float *xr = x + r * cols;
    float *yr = y + r * cols;
    float m_i = -INFINITY, l_i = 0.f;
    for (int64_t c0 = 0; c0 < cols; c0 += block_cols) {
      const int64_t c1 = c0 + block_cols < cols ? c0 + block_cols : cols;
      float m_ij = m_i;
      for (int64_t c = c0; c < c1; ++c) m_ij = fmaxf(m_ij, xr[c]);
      float l_ij = 0.f;
      for (int64_t c = c0; c < c1; ++c) l_ij += expf(xr[c] - m_ij);
      const float alpha = expf(m_i - m_ij);
      l_i = l_i * alpha + l_ij;
      m_i = m_ij;
    }
    for (int64_t c = 0; c < cols; ++c) yr[c] = expf(xr[c] - m_i) / l_i;
  }
}

/* ------------------------------------------------------------------ LayerNorm
 * layer_norm_fwd_kernel, test/python/triton/test_layer_norm.py:58-82:
 *   mean = sum(x)/N; xc = x - mean; var = sum(xc*xc)/N; rstd = 1/sqrt(var+eps);
 *   y = xc*rstd*w + b; mean and rstd are stored per row. */
void oracle_layer_norm_f32(const float *x, float *y, const float *w, const float *b, float *mean,
                           float *rstd, int64_t rows, int64_t cols, float eps) {
#pragma omp parallel for
  for (int64_t r = 0; r < rows; ++r) {
    const float *xr = x + r * cols;
    float *yr = y + r * cols;
    double s = 0.0; /* the reduction order of tl.sum is unspecified: sum exactly, round once */
    for (int64_t c = 0; c < cols; ++c) s += xr[c];
    const float mu = (float)s / (float)cols;
    double q = 0.0;
    for (int64_t c = 0; c < cols; ++c) q += (double)((xr[c] - mu) * (xr[c] - mu));
    const float rs = 1.0f / sqrtf((float)q / (float)cols + eps);
    if (mean) mean[r] = mu;
    if (rstd) rstd[r] = rs;
    for (int64_t c = 0; c < cols; ++c) yr[c] = (xr[c] - mu) * rs * w[c] + b[c];
  }
}

/* fp16 storage, fp32 statistics and arithmetic, one rounding on the way out. */
void oracle_layer_norm_f16(const f16 *x, f16 *y, const f16 *w, const f16 *b, float *mean, float *rstd,
                           int64_t rows, int64_t cols, float eps) {
#pragma omp parallel for
  for (int64_t r = 0; r < rows; ++r) {
    const f16 *xr = x + r * cols;
    f16 *yr = y + r * cols;
    double s = 0.0;
    for (int64_t c = 0; c < cols; ++c) s += (double)xr[c];
    const float mu = (float)(s / (double)cols);
    double q = 0.0;
    for (int64_t c = 0; c < cols; ++c) q += ((double)xr[c] - mu) * ((double)xr[c] - mu);
    const float rs = 1.0f / sqrtf((float)(q / (double)cols) + eps);
    if (mean) mean[r] = mu;
    if (rstd) rstd[r] = rs;
    for (int64_t c = 0; c < cols; ++c) yr[c] = (f16)(((float)xr[c] - mu) * rs * (float)w[c] + (float)b[c]);
  }
}

/* ------------------------------------------------------------------ RMSNorm
 * rms_norm_fwd_kernel, test/python/triton/test_rms_norm.py:57-62:
 *   rms = sqrt(sum(x*x)/N + eps); y = (x / rms) * g. */
void oracle_rms_norm_f32(const float *x, float *y, const float *g, int64_t rows, int64_t cols, float eps) {
#pragma omp parallel for
  for (int64_t r = 0; r < rows; ++r) {
    const float *xr = x + r * cols;
    float *yr = y + r * cols;
    double s = 0.0;
    for (int64_t c = 0; c < cols; ++c) s += (double)(xr[c] * xr[c]);
    const float rms = sqrtf((float)s / (float)cols + eps);
    for (int64_t c = 0; c < cols; ++c) yr[c] = (xr[c] / rms) * g[c];
  }
}

void oracle_rms_norm_f16(const f16 *x, f16 *y, const f16 *g, int64_t rows, int64_t cols, float eps) {
#pragma omp parallel for
  for (int64_t r = 0; r < rows; ++r) {
    const f16 *xr = x + r * cols;
    f16 *yr = y + r * cols;
    double s = 0.0;
    for (int64_t c = 0; c < cols; ++c) s += (double)xr[c] * (double)xr[c];
    const float rms = sqrtf((float)(s / (double)cols) + eps);
    for (int64_t c = 0; c < cols; ++c) yr[c] = (f16)(((float)xr[c] / rms) * (float)g[c]);
  }
}

/* ------------------------------------------------------------------ matmul
 * The scalar check of the HexKL matmul test, test/python/mlir/hexkl_linalg_matmul/wrapper.cpp:47-67:
 *   acc (fp32) += (float)act[row*K + k] * w[k*N + col]. */
void oracle_matmul_f16_f32(const f16 *a, const f16 *b, float *c, int64_t M, int64_t N, int64_t K) {
#pragma omp parallel for
  for (int64_t i = 0; i < M; ++i) {
    float *ci = c + i * N;
    for (int64_t j = 0; j < N; ++j) ci[j] = 0.f;
    for (int64_t k = 0; k < K; ++k) {
      const float av = (float)a[i * K + k];
      const f16 *bk = b + k * N;
      for (int64_t j = 0; j < N; ++j) ci[j] += av * (float)bk[j];
    }
  }
}

/* fp16 output (matmul, test/python/triton/test_matmul.py:66-70: tl.dot(..., out_dtype=C dtype)),
 * with an optional fp16 residual added before the rounding (used by the decoder blocks). */
void oracle_matmul_f16_f16(const f16 *a, const f16 *b, f16 *c, const f16 *residual, int64_t M, int64_t N,
                           int64_t K) {
#pragma omp parallel for
  for (int64_t i = 0; i < M; ++i) {
    float *acc = (float *)calloc((size_t)N, sizeof(float));
    for (int64_t k = 0; k < K; ++k) {
      const float av = (float)a[i * K + k];
      const f16 *bk = b + k * N;
      for (int64_t j = 0; j < N; ++j) acc[j] += av * (float)bk[j];
    }
    for (int64_t j = 0; j < N; ++j)
      c[i * N + j] = (f16)(acc[j] + (residual ? (float)residual[i * N + j] : 0.f));
    free(acc);
  }
}

/* ------------------------------------------------------------------ flash attention
 * attention_fwd_kernel + _attn_fwd_inner, test/python/triton/test_flash_attention.py:37-168:
 *   m_i = -99999999999999, l_i = 1, acc = 0; qk_scale = sm_scale * 1.44269504;
 *   per key block: qk = q.k^T; m_ij = max(m_i, rowmax(qk)*qk_scale); p = exp2(qk*qk_scale - m_ij);
 *   alpha = exp2(m_i - m_ij); l_i = l_i*alpha + sum(p); acc = acc*alpha + p.v; m_i = m_ij;
 *   out = acc / l_i.
 * Tensors are contiguous [Z, H, N, D].  causal != 0 drops keys above the diagonal (the -inf
 * additive mask of tm_tensor.attention, lib/Transforms/LowerTmTensor.cpp:103-141).
 * p_half != 0 truncates p to fp16 before the second product, as the fp16 MLIR form does
 * (test/python/mlir/hexkl_attention/input.mlir:140-145). */
static void attention_rows(const float *q, const float *k, const float *v, float *o, int64_t N, int64_t D,
                           float sm_scale, int causal, int64_t block_n, int p_half, int64_t r0, int64_t r1) {
  const float qk_scale = sm_scale * 1.44269504f;
  float *acc = (float *)malloc((size_t)D * sizeof(float));
  float *p = (float *)malloc((size_t)block_n * sizeof(float));
  for (int64_t i = r0; i < r1; ++i) {
    float m_i = -99999999999999.0f, l_i = 1.0f;
    for (int64_t d = 0; d < D; ++d) acc[d] = 0.f;
    const int64_t kv_end = causal ? i + 1 : N;
    for (int64_t n0 = 0; n0 < kv_end; n0 += block_n) {
      const int64_t n1 = n0 + block_n < kv_end ? n0 + block_n : kv_end;
      float rowmax = -INFINITY;
      for (int64_t n = n0; n < n1; ++n) {
        float dot = 0.f;
        for (int64_t d = 0; d < D; ++d) dot += q[i * D + d] * k[n * D + d];
        p[n - n0] = dot;
        rowmax = fmaxf(rowmax, dot);
      }
      const float m_ij = fmaxf(m_i, rowmax * qk_scale);
      float l_ij = 0.f;
      for (int64_t n = n0; n < n1; ++n) {
        float pv = exp2f(p[n - n0] * qk_scale - m_ij);
        if (p_half) pv = (float)(f16)pv;
        p[n - n0] = pv;
        l_ij += pv;
      }
      const float alpha = exp2f(m_i - m_ij);
      l_i = l_i * alpha + l_ij;
      for (int64_t d = 0; d < D; ++d) acc[d] *= alpha;
      for (int64_t n = n0; n < n1; ++n)
        for (int64_t d = 0; d < D; ++d) acc[d] += p[n - n0] * v[n * D + d];
      m_i = m_ij;
    }
    for (int64_t d = 0; d < D; ++d) o[i * D + d] = acc[d] / l_i;
  }
  free(acc);
  free(p);
}

void oracle_attention_f32(const float *q, const float *k, const float *v, float *o, int64_t Z, int64_t H,
                          int64_t N, int64_t D, float sm_scale, int causal, int64_t block_n) {
  if (block_n <= 0) block_n = 64;
  const int64_t chunk = 16;
  const int64_t nchunks = (N + chunk - 1) / chunk;
#pragma omp parallel for collapse(2)
  for (int64_t zh = 0; zh < Z * H; ++zh)
    for (int64_t c = 0; c < nchunks; ++c) {
      const int64_t off = zh * N * D;
      const int64_t r1 = (c + 1) * chunk < N ? (c + 1) * chunk : N;
      attention_rows(q + off, k + off, v + off, o + off, N, D, sm_scale, causal, block_n, 0, c * chunk, r1);
    }
}

void oracle_attention_f16(const f16 *q, const f16 *k, const f16 *v, f16 *o, int64_t Z, int64_t H, int64_t N,
                          int64_t D, float sm_scale, int causal, int64_t block_n) {
  if (block_n <= 0) block_n = 64;
  const int64_t per = N * D;
#pragma omp parallel for
  for (int64_t zh = 0; zh < Z * H; ++zh) {
    float *buf = (float *)malloc((size_t)(4 * per) * sizeof(float));
    float *qf = buf, *kf = buf + per, *vf = buf + 2 * per, *of = buf + 3 * per;
    for (int64_t i = 0; i < per; ++i) {
      qf[i] = (float)q[zh * per + i];
      kf[i] = (float)k[zh * per + i];
      vf[i] = (float)v[zh * per + i];
    }
    attention_rows(qf, kf, vf, of, N, D, sm_scale, causal, block_n, 1, 0, N);
    for (int64_t i = 0; i < per; ++i) o[zh * per + i] = (f16)of[i];
    free(buf);
  }
}

/* The unfused check of the fp16 attention test, test/python/mlir/hexkl_attention/wrapper.cpp:55-188:
 * S = Q.K^T (fp32 accumulation of fp16 products), S *= scale, three-pass softmax, O = P.V with P
 * kept in fp32 (the intent of the check; its cast of the fp32 buffer to fp16 at :168 is not
 * followed), fp32 output.  The row maximum starts from the first element rather than from the
 * smallest positive float the check uses at :125. */
void oracle_attention_unfused_f16_f32(const f16 *q, const f16 *k, const f16 *v, float *o, int64_t Z, int64_t H,
                                      int64_t N, int64_t D, float scale, int causal) {
#pragma omp parallel for collapse(2)
  for (int64_t zh = 0; zh < Z * H; ++zh)
    for (int64_t i = 0; i < N; ++i) {
      const f16 *qb = q + zh * N * D, *kb = k + zh * N * D, *vb = v + zh * N * D;
      float *s = (float *)malloc((size_t)N * sizeof(float));
      const int64_t kv_end = causal ? i + 1 : N;
      float mx = -INFINITY;
      for (int64_t n = 0; n < kv_end; ++n) {
        float acc = 0.f;
        for (int64_t d = 0; d < D; ++d) acc += (float)qb[i * D + d] * (float)kb[n * D + d];
        s[n] = acc * scale;
        mx = fmaxf(mx, s[n]);
      }
      float sum = 0.f;
      for (int64_t n = 0; n < kv_end; ++n) sum += expf(s[n] - mx);
      for (int64_t n = 0; n < kv_end; ++n) s[n] = expf(s[n] - mx) / sum;
      for (int64_t d = 0; d < D; ++d) {
        float acc = 0.f;
        for (int64_t n = 0; n < kv_end; ++n) acc += s[n] * (float)vb[n * D + d];
        o[zh * N * D + i * D + d] = acc;
      }
      free(s);
    }
}

/* tm_tensor.attention as its lowering writes it, qcom_hexagon_backend/lib/Transforms/LowerTmTensor.cpp:70-235:
 * K^T (:126-130), QK^T by batch_matmul (:133-141), multiply by 1/sqrt(head_dim) (:144-156), add the mask
 * (:159-162), row maximum from -inf (:166-181), exp(x - max) (:184-200), row sum (:203-213), divide
 * (:216-230), batch_matmul with V accumulated onto the `outs` operand (:234-238).  Rank-3 operands:
 * q [batch, seq_q, d], k and v [batch, seq_kv, d], mask [batch, seq_q, seq_kv], out [batch, seq_q, d].
 * The arithmetic is fp32 here whatever the element type of the operands (the lowering computes in the
 * operands' own type); `out` must hold the initial value of the accumulator (zeros in the reference's
 * test, test/Conversion/TmTensorToLinalg/SDPA.mlir:5-13). */
void oracle_sdpa_masked_f32(const float *q, const float *k, const float *v, const float *mask, float *out,
                            int64_t batch, int64_t seq_q, int64_t seq_kv, int64_t d) {
  const float scale = (float)(1.0 / sqrt((double)d));
#pragma omp parallel for collapse(2)
  for (int64_t b = 0; b < batch; ++b)
    for (int64_t i = 0; i < seq_q; ++i) {
      float *s = (float *)malloc((size_t)seq_kv * sizeof(float));
      const float *qr = q + (b * seq_q + i) * d;
      float mx = -INFINITY;
      for (int64_t n = 0; n < seq_kv; ++n) {
        const float *kr = k + (b * seq_kv + n) * d;
        float acc = 0.f;
        for (int64_t c = 0; c < d; ++c) acc += qr[c] * kr[c];
        s[n] = acc * scale + mask[(b * seq_q + i) * seq_kv + n];
        mx = fmaxf(mx, s[n]);
      }
      float sum = 0.f;
      for (int64_t n = 0; n < seq_kv; ++n) {
        s[n] = expf(s[n] - mx);
        sum += s[n];
      }
      for (int64_t n = 0; n < seq_kv; ++n) s[n] = s[n] / sum;
      for (int64_t c = 0; c < d; ++c) {
        float acc = out[(b * seq_q + i) * d + c];
        for (int64_t n = 0; n < seq_kv; ++n) acc += s[n] * v[(b * seq_kv + n) * d + c];
        out[(b * seq_q + i) * d + c] = acc;
      }
      free(s);
    }
}

/* ------------------------------------------------------------------ SiLU
 * silu_kernel, test/python/triton/test_silu.py:48-51: x / (1 + exp((-x).to(f32)).to(x.dtype)). */
void oracle_silu_f32(const float *x, float *y, int64_t n) {
#pragma omp parallel for
  for (int64_t i = 0; i < n; ++i) y[i] = x[i] / (1.0f + expf(-x[i]));
}
void oracle_silu_f16(const f16 *x, f16 *y, int64_t n) {
#pragma omp parallel for
  for (int64_t i = 0; i < n; ++i) {
    const f16 e = (f16)expf(-(float)x[i]);
    y[i] = (f16)((float)x[i] / (1.0f + (float)e));
  }
}

/* ------------------------------------------------------------------ GELU (tanh form)
 * gelu_kernel + tanh, test/python/triton/test_gelu.py:25-54:
 *   tanh(u) = (1 - e) / (1 + e), e = exp((-2u).to(f32)).to(x.dtype);
 *   y = 0.5 * x * (1 + tanh(0.797885*x + 0.035677*x*x*x)); for fp16 data every step rounds to fp16. */
void oracle_gelu_f32(const float *x, float *y, int64_t n) {
#pragma omp parallel for
  for (int64_t i = 0; i < n; ++i) {
    const float u = 0.797885f * x[i] + 0.035677f * x[i] * x[i] * x[i];
    const float e = expf(-2.0f * u);
    y[i] = 0.5f * x[i] * (1.0f + (1.0f - e) / (1.0f + e));
  }
}
void oracle_gelu_f16(const f16 *x, f16 *y, int64_t n) {
#pragma omp parallel for
  for (int64_t i = 0; i < n; ++i) {
    const f16 xv = x[i];
    const f16 x3 = (f16)((f16)((f16)((f16)0.035677f * xv) * xv) * xv);
    const f16 u = (f16)((f16)((f16)0.797885f * xv) + x3);
    const f16 e = (f16)expf((float)(f16)((f16)-2.0f * u));
    const f16 th = (f16)((f16)((f16)1.0f - e) / (f16)((f16)1.0f + e));
    y[i] = (f16)((f16)((f16)0.5f * xv) * (f16)((f16)1.0f + th));
  }
}

/* ------------------------------------------------------------------ RoPE
 * rope_kernel + compute_thetas, test/python/triton/test_rope.py:40-190: steps = [0,0,2,2,...],
 * freq = 1 / theta^(steps/D), angle = position * freq; even d: x[d]*cos - x[d+1]*sin,
 * odd d: x[d-1]*sin + x[d]*cos.  Contiguous [B, L, H, D], fp32 arithmetic. */
void oracle_rope_f32(const float *x, float *y, int64_t B, int64_t L, int64_t H, int64_t D, float theta) {
#pragma omp parallel for collapse(2)
  for (int64_t b = 0; b < B; ++b)
    for (int64_t l = 0; l < L; ++l)
      for (int64_t h = 0; h < H; ++h) {
        const int64_t off = ((b * L + l) * H + h) * D;
        for (int64_t d = 0; d < D; ++d) {
          const float step = (float)(d - (d % 2));
          const float freq = 1.0f / expf(logf(theta) * (step / (float)D));
          const float cs = cosf((float)l * freq), sn = sinf((float)l * freq);
          y[off + d] = (d % 2 == 0) ? x[off + d] * cs - x[off + d + 1] * sn : x[off + d - 1] * sn + x[off + d] * cs;
        }
      }
}
void oracle_rope_f16(const f16 *x, f16 *y, int64_t B, int64_t L, int64_t H, int64_t D, float theta) {
  const int64_t n = B * L * H * D;
  float *xf = (float *)malloc((size_t)n * sizeof(float)), *yf = (float *)malloc((size_t)n * sizeof(float));
  for (int64_t i = 0; i < n; ++i) xf[i] = (float)x[i];
  oracle_rope_f32(xf, yf, B, L, H, D, theta);
  for (int64_t i = 0; i < n; ++i) y[i] = (f16)yf[i];
  free(xf);
  free(yf);
}

/* ------------------------------------------------------------------ whole-vector sum
 * sum_kernel, test/python/triton/test_sum.py:31-36: tl.sum over the block; the order of the
 * reduction is unspecified, so the oracle sums exactly (double) and rounds once. */
float oracle_sum_f32(const float *x, int64_t n) {
  double s = 0.0;
  for (int64_t i = 0; i < n; ++i) s += x[i];
  return (float)s;
}
float oracle_sum_f16(const f16 *x, int64_t n) {
  double s = 0.0;
  for (int64_t i = 0; i < n; ++i) s += (double)x[i];
  return (float)s;
}

/* out[r, c] = silu(gu[r, c]) * gu[r, cols + c], fp32 arithmetic, one rounding. */
void oracle_swiglu_f16(const f16 *gu, f16 *out, int64_t rows, int64_t cols) {
#pragma omp parallel for
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < cols; ++c) {
      const float g = (float)gu[r * 2 * cols + c], u = (float)gu[r * 2 * cols + cols + c];
      out[r * cols + c] = (f16)((g / (1.0f + expf(-g))) * u);
    }
}

/* ------------------------------------------------------------------ decoder block stack
 * Pre-norm blocks composed from the operators above (no single reference function; the reference
 * runs whole models through its graph flow, test/python/torch-mlir/gpt2lmheadmodel.py:143-169):
 *   h = x + Attn(RMSNorm(x, g1).Wqkv).Wo;  x' = h + (SiLU(n.Wg) * (n.Wu)).Wd, n = RMSNorm(h, g2).
 * Activations are stored in fp16 between operators, like the CUDA pipeline stores them.
 * Weights per layer, row-major: wqkv [d, 3d] (q|k|v, head-major), wo [d, d], wgu [d, 2f], wd [f, d]. */
void oracle_decoder_f16(const f16 *x, f16 *out, const f16 *const *wqkv, const f16 *const *wo,
                        const f16 *const *wgu, const f16 *const *wd, const f16 *const *g1,
                        const f16 *const *g2, int n_layers, int d, int n_heads, int head_dim, int f,
                        int batch, int seq, float eps) {
  const int64_t T = (int64_t)batch * seq;
  f16 *cur = (f16 *)malloc((size_t)(T * d) * sizeof(f16));
  f16 *n = (f16 *)malloc((size_t)(T * d) * sizeof(f16));
  f16 *qkv = (f16 *)malloc((size_t)(T * 3 * d) * sizeof(f16));
  f16 *hq = (f16 *)malloc((size_t)(T * d) * sizeof(f16));
  f16 *hk = (f16 *)malloc((size_t)(T * d) * sizeof(f16));
  f16 *hv = (f16 *)malloc((size_t)(T * d) * sizeof(f16));
  f16 *ho = (f16 *)malloc((size_t)(T * d) * sizeof(f16));
  f16 *attn = (f16 *)malloc((size_t)(T * d) * sizeof(f16));
  f16 *h = (f16 *)malloc((size_t)(T * d) * sizeof(f16));
  f16 *gu = (f16 *)malloc((size_t)(T * 2 * f) * sizeof(f16));
  f16 *act = (f16 *)malloc((size_t)(T * f) * sizeof(f16));
  memcpy(cur, x, (size_t)(T * d) * sizeof(f16));
  const float scale = 1.0f / sqrtf((float)head_dim);
  for (int l = 0; l < n_layers; ++l) {
    oracle_rms_norm_f16(cur, n, g1[l], T, d, eps);
    oracle_matmul_f16_f16(n, wqkv[l], qkv, NULL, T, 3 * d, d);
    /* split heads: [b, s, {q,k,v}, head, hd] -> [b, head, s, hd] */
    for (int64_t b = 0; b < batch; ++b)
      for (int64_t s = 0; s < seq; ++s)
        for (int64_t hh = 0; hh < n_heads; ++hh)
          for (int64_t e = 0; e < head_dim; ++e) {
            const int64_t src = (b * seq + s) * 3 * d + hh * head_dim + e;
            const int64_t dst = ((b * n_heads + hh) * seq + s) * head_dim + e;
            hq[dst] = qkv[src];
            hk[dst] = qkv[src + d];
            hv[dst] = qkv[src + 2 * d];
          }
    oracle_attention_f16(hq, hk, hv, ho, batch, n_heads, seq, head_dim, scale, 1, 64);
    for (int64_t b = 0; b < batch; ++b)
      for (int64_t s = 0; s < seq; ++s)
        for (int64_t hh = 0; hh < n_heads; ++hh)
          for (int64_t e = 0; e < head_dim; ++e)
            attn[(b * seq + s) * d + hh * head_dim + e] = ho[((b * n_heads + hh) * seq + s) * head_dim + e];
    oracle_matmul_f16_f16(attn, wo[l], h, cur, T, d, d);
    oracle_rms_norm_f16(h, n, g2[l], T, d, eps);
    oracle_matmul_f16_f16(n, wgu[l], gu, NULL, T, 2 * f, d);
    oracle_swiglu_f16(gu, act, T, f);
    oracle_matmul_f16_f16(act, wd[l], cur, h, T, d, f);
  }
  memcpy(out, cur, (size_t)(T * d) * sizeof(f16));
  free(cur); free(n); free(qkv); free(hq); free(hk); free(hv); free(ho); free(attn); free(h); free(gu); free(act);
}

/* ------------------------------------------------------------------ cumulative sum
 * ttx.cumsum {axis} as lowered by qcom_hexagon_backend/lib/Transforms/LowerTTX.cpp:179-300: the first
 * slice along the axis is the initial partial sum, then for i = 1 .. len-1: p = p + x[.., i, ..];
 * y[.., i, ..] = p (FileCheck'd in test/Conversion/TtxToLinalg/cumsum_2D.mlir:20-33).  ttx.scan
 * {reverse = true} with an addition body walks from index len-1 down (LowerTTX.cpp:75-176,
 * reverse_associative_scan_1D.mlir:26-40).  Tensor viewed as [outer, len, inner].  The float version
 * keeps the partial sum in fp32; int32 wraps. */
void oracle_cumsum_f32(const float *x, float *y, int64_t outer, int64_t len, int64_t inner, int reverse) {
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t i = 0; i < inner; ++i) {
      float p = 0.f;
      for (int64_t s = 0; s < len; ++s) {
        const int64_t l = reverse ? len - 1 - s : s;
        const int64_t idx = (o * len + l) * inner + i;
        p = s == 0 ? x[idx] : p + x[idx];
        y[idx] = p;
      }
    }
}

void oracle_cumsum_i32(const int32_t *x, int32_t *y, int64_t outer, int64_t len, int64_t inner, int reverse) {
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t i = 0; i < inner; ++i) {
      uint32_t p = 0;
      for (int64_t s = 0; s < len; ++s) {
        const int64_t l = reverse ? len - 1 - s : s;
        const int64_t idx = (o * len + l) * inner + i;
        p += (uint32_t)x[idx];
        y[idx] = (int32_t)p;
      }
    }
}
