// Elementwise operators, RoPE and the full-vector sum of the reference's remaining Triton tests.
//
// Reference semantics (qualcomm/hexagon-mlir, test/python/triton/):
//   gelu_kernel        test_gelu.py:25-54      0.5*x*(1 + tanh(0.797885*x + 0.035677*x^3)),
//                                              tanh(u) = (1 - e^{-2u}) / (1 + e^{-2u}), exp in fp32
//   cos_kernel / sin_kernel  test_math_ops.py:24-37;   rsqrt_kernel  test_rsqrt.py:19-24
//   add_kernel (test_vec_add.py:19-25), add_kernel_scalar (test_vec_add_with_scalar.py:31-46),
//   add_2d_kernel (test_vec_add_2d.py:21-56), div_kernel (test_vec_div_2d.py:20-55)
//   sum_kernel         test_sum.py:31-36       one program reduces the whole vector
//   rope_kernel        test_rope.py:98-190     interleaved-pair rotation, freq = theta^(-steps/D),
//                                              steps = [0,0,2,2,...], angle = position * freq
// All are one read and one write per element (two reads for the binary ones) with 16-byte
// accesses; arithmetic in fp32, one rounding on the way out.
#include "common.cuh"

namespace hexb {

struct GeluTanh {
  static __device__ __forceinline__ float apply(float x) {
    const float u = 0.797885f * x + 0.035677f * x * x * x;
    // tanh(u) = (1 - e^{-2u}) / (1 + e^{-2u}) = 1 - 2 / (1 + e^{2u}); the second form has no inf/inf
    // for u << 0 (the reference's form gives NaN below x ~ -10.3; its test only feeds [0, 1))
    const float t = 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * u));  // fast division: 2 ulp, no slow path at overflow
    return 0.5f * x * (1.0f + t);
  }
  // fp16 data: the result is rounded to 11 bits, so tanh.approx (2^-11) is enough and halves the
  // special-function work, which bounds this kernel for fp16 (two values per 4 bytes moved)
  static __device__ __forceinline__ float apply_h(float x) {
    const float u = x * fmaf(0.035677f * x, x, 0.797885f);
    const float hx = 0.5f * x;
    return fmaf(hx, tanh_approx(u), hx);
  }
};
struct Cos { static __device__ __forceinline__ float apply(float x) { return cosf(x); } static __device__ __forceinline__ float apply_h(float x) { return cosf(x); } };
struct Sin { static __device__ __forceinline__ float apply(float x) { return sinf(x); } static __device__ __forceinline__ float apply_h(float x) { return sinf(x); } };
struct Rsqrt { static __device__ __forceinline__ float apply(float x) { return rsqrtf(x); } static __device__ __forceinline__ float apply_h(float x) { return rsqrtf(x); } };  // 2 ulp
struct Add { static __device__ __forceinline__ float apply(float a, float b) { return a + b; } };
struct Sub { static __device__ __forceinline__ float apply(float a, float b) { return a - b; } };
struct Mul { static __device__ __forceinline__ float apply(float a, float b) { return a * b; } };
struct Div { static __device__ __forceinline__ float apply(float a, float b) { return a / b; } };

// Elementwise skeleton: every thread keeps U independent 16-byte loads per operand in flight (issued
// before any arithmetic: the software form of the reference's double-buffered elementwise loops,
// qcom_hexagon_backend/lib/Transforms/DoubleBufferGenericS1.cpp), CTA-interleaved so that each load
// instruction of a warp covers 512 contiguous bytes.
constexpr int EW_U = 4;

template <typename T, typename Op>
__global__ void __launch_bounds__(256) unary_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t n, int vec_ok) {
  constexpr int E = Vec16<T>::N;
  using Raw = decltype(Vec16<T>::raw);
  const int64_t tid = (int64_t)blockIdx.x * 256 + threadIdx.x, nth = (int64_t)gridDim.x * 256;
  const int64_t nvec = vec_ok ? n / E : 0;
  for (int64_t v0 = tid; v0 < nvec; v0 += nth * EW_U) {
    Vec16<T> a[EW_U];
#pragma unroll
    for (int u = 0; u < EW_U; ++u)
      if (v0 + u * nth < nvec) a[u].raw = ld_stream_as<Raw>(x + (v0 + u * nth) * E);
#pragma unroll
    for (int u = 0; u < EW_U; ++u) {
      if (v0 + u * nth < nvec) {
        float f[E];
        a[u].unpack(f);
#pragma unroll
        for (int e = 0; e < E; ++e) f[e] = sizeof(T) == 2 ? Op::apply_h(f[e]) : Op::apply(f[e]);
        a[u].pack(f);
        st_stream_as<Raw>(y + (v0 + u * nth) * E, a[u].raw);
      }
    }
  }
  for (int64_t i = nvec * E + tid; i < n; i += nth)
    y[i] = from_f32<T>(sizeof(T) == 2 ? Op::apply_h(to_f32<T>(x[i])) : Op::apply(to_f32<T>(x[i])));
}

template <typename T, typename Op>
__global__ void __launch_bounds__(256) binary_kernel(const T *__restrict__ a, const T *__restrict__ b,
                                                     T *__restrict__ y, int64_t n, int vec_ok) {
  constexpr int E = Vec16<T>::N;
  using Raw = decltype(Vec16<T>::raw);
  const int64_t tid = (int64_t)blockIdx.x * 256 + threadIdx.x, nth = (int64_t)gridDim.x * 256;
  const int64_t nvec = vec_ok ? n / E : 0;
  for (int64_t v0 = tid; v0 < nvec; v0 += nth * EW_U) {
    Vec16<T> va[EW_U], vb[EW_U];
#pragma unroll
    for (int u = 0; u < EW_U; ++u)
      if (v0 + u * nth < nvec) {
        va[u].raw = ld_stream_as<Raw>(a + (v0 + u * nth) * E);
        vb[u].raw = ld_stream_as<Raw>(b + (v0 + u * nth) * E);
      }
#pragma unroll
    for (int u = 0; u < EW_U; ++u) {
      if (v0 + u * nth < nvec) {
        float fa[E], fb[E];
        va[u].unpack(fa);
        vb[u].unpack(fb);
#pragma unroll
        for (int e = 0; e < E; ++e) fa[e] = Op::apply(fa[e], fb[e]);
        va[u].pack(fa);
        st_stream_as<Raw>(y + (v0 + u * nth) * E, va[u].raw);
      }
    }
  }
  for (int64_t i = nvec * E + tid; i < n; i += nth)
    y[i] = from_f32<T>(Op::apply(to_f32<T>(a[i]), to_f32<T>(b[i])));
}

// Whole-vector sum.  The reference reduces the whole vector in one program (sum_kernel, test_sum.py:31-36);
// here every CTA sums a CTA-interleaved share with 16-byte loads into fp32 partials, and a second launch
// adds the partials in index order: the grid is a function of n and the SM count only, so the order of
// additions -- and the result -- is the same on every call.
template <typename T>
__global__ void __launch_bounds__(256) sum_partial_kernel(const T *__restrict__ x, float *__restrict__ partial, int64_t n,
                                                          int vec_ok) {
  constexpr int E = Vec16<T>::N;
  using Raw = decltype(Vec16<T>::raw);
  __shared__ float part[8];
  const int64_t tid = (int64_t)blockIdx.x * 256 + threadIdx.x, nth = (int64_t)gridDim.x * 256;
  const int64_t nvec = vec_ok ? n / E : 0;
  float acc[EW_U] = {};
  for (int64_t v0 = tid; v0 < nvec; v0 += nth * EW_U) {
    Vec16<T> a[EW_U];
#pragma unroll
    for (int u = 0; u < EW_U; ++u)
      if (v0 + u * nth < nvec) a[u].raw = ld_stream_as<Raw>(x + (v0 + u * nth) * E);
#pragma unroll
    for (int u = 0; u < EW_U; ++u)
      if (v0 + u * nth < nvec) {
        float f[E];
        a[u].unpack(f);
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) s += f[e];
        acc[u] += s;
      }
  }
  for (int64_t i = nvec * E + tid; i < n; i += nth) acc[0] += to_f32<T>(x[i]);
  float s = warp_sum((acc[0] + acc[1]) + (acc[2] + acc[3]));
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = warp_sum(threadIdx.x < 8 ? part[threadIdx.x] : 0.f);
    if (threadIdx.x == 0) partial[blockIdx.x] = s;
  }
}

template <typename T>
__global__ void __launch_bounds__(1024) sum_final_kernel(const float *__restrict__ partial, T *__restrict__ out, int count) {
  __shared__ float part[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < count; i += 1024) s += partial[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = warp_sum(part[threadIdx.x]);
    if (threadIdx.x == 0) out[0] = from_f32<T>(s);
  }
}

template <typename T>
static int launch_sum(const T *x, T *out, int64_t n, int sm, cudaStream_t st) {
  int64_t ctas = (n / Vec16<T>::N + 256 * EW_U - 1) / (256 * EW_U);
  if (ctas < 1) ctas = 1;
  const int64_t cap = (int64_t)sm * 8;
  const int grid = (int)(ctas < cap ? ctas : cap);
  float *partial = nullptr;
  if (int e = scratch_alloc(reinterpret_cast<void **>(&partial), (size_t)grid * sizeof(float), st)) return e;
  sum_partial_kernel<T><<<grid, 256, 0, st>>>(x, partial, n, aligned16(x) ? 1 : 0);
  sum_final_kernel<T><<<1, 1024, 0, st>>>(partial, out, grid);
  const int rc = check_launch("sum");
  if (int e = scratch_free(partial, st)) return e;
  return rc;
}

// out[b,l,h,d] = d even: x[d]*cos - x[d+1]*sin;  d odd: x[d-1]*sin + x[d]*cos, angle = l * theta^(-(d - d%2)/D).
template <typename T>
__global__ void __launch_bounds__(256) rope_kernel(const T *__restrict__ x, T *__restrict__ out, int64_t B, int64_t L,
                                                   int64_t H, int64_t D, int64_t sb, int64_t sl, int64_t sh,
                                                   int64_t ob, int64_t ol, int64_t oh, float neg_log2_theta_over_d) {
  const int64_t pairs = D / 2;
  const int64_t total = B * L * H * pairs;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
    const int64_t pr = i % pairs;
    int64_t t = i / pairs;
    const int64_t h = t % H; t /= H;
    const int64_t l = t % L;
    const int64_t b = t / L;
    const float freq = exp2f((float)(2 * pr) * neg_log2_theta_over_d);
    float sn, cs;
    sincosf((float)l * freq, &sn, &cs);
    const T *xp = x + b * sb + l * sl + h * sh + 2 * pr;
    T *op = out + b * ob + l * ol + h * oh + 2 * pr;
    const float x0 = to_f32<T>(xp[0]), x1 = to_f32<T>(xp[1]);
    op[0] = from_f32<T>(x0 * cs - x1 * sn);
    op[1] = from_f32<T>(x0 * sn + x1 * cs);
  }
}

// Vector form: one CTA per position l.  A thread owns one 16-byte column group of a row and computes
// the sines and cosines of its pairs once -- the angle depends on (l, pair) only -- then walks all
// (batch, head) rows of that position, so the trigonometry is amortised over B * H rows.
template <typename T>
__global__ void __launch_bounds__(256) rope_rows_kernel(const T *__restrict__ x, T *__restrict__ out, int64_t B, int64_t L,
                                                        int64_t H, int64_t D, int64_t sb, int64_t sl, int64_t sh,
                                                        int64_t ob, int64_t ol, int64_t oh, float neg_log2_theta_over_d) {
  constexpr int E = Vec16<T>::N;
  using Raw = decltype(Vec16<T>::raw);
  const int cgs = (int)(D / E);             // column groups per row (<= 256)
  const int rows_par = 256 / cgs;           // rows the CTA handles at a time
  const int cg = threadIdx.x % cgs, rlane = threadIdx.x / cgs;
  if (rlane >= rows_par) return;
  const int64_t l = blockIdx.x;
  float sn[E / 2], cs[E / 2];
#pragma unroll
  for (int i = 0; i < E / 2; ++i) {
    const float freq = exp2f((float)(cg * E + 2 * i) * neg_log2_theta_over_d);
    sincosf((float)l * freq, &sn[i], &cs[i]);
  }
  const int64_t R = B * H;
  for (int64_t r = rlane; r < R; r += rows_par) {
    const int64_t b = r / H, h = r - b * H;
    Vec16<T> v;
    v.raw = ld_stream_as<Raw>(x + b * sb + l * sl + h * sh + cg * E);
    float f[E];
    v.unpack(f);
#pragma unroll
    for (int i = 0; i < E / 2; ++i) {
      const float x0 = f[2 * i], x1 = f[2 * i + 1];
      f[2 * i] = x0 * cs[i] - x1 * sn[i];
      f[2 * i + 1] = x0 * sn[i] + x1 * cs[i];
    }
    v.pack(f);
    st_stream_as<Raw>(out + b * ob + l * ol + h * oh + cg * E, v.raw);
  }
}

// out[i] = i: what the reference's grid test computes when every program of a grid stores its
// flattened id (test/python/triton/test_multidim_grid.py:21-37).
template <typename T>
__global__ void __launch_bounds__(256) iota_kernel(T *__restrict__ out, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256)
    out[i] = from_f32<T>((float)i);
}

template <typename T, typename Op>
static int launch_unary(const T *x, T *y, int64_t n, int sm, cudaStream_t st) {
  const int vec_ok = aligned16(x) && aligned16(y);
  int64_t ctas = (n / Vec16<T>::N + 256 * EW_U - 1) / (256 * EW_U) + 1;
  const int64_t cap = (int64_t)sm * 16;
  unary_kernel<T, Op><<<(unsigned)(ctas < cap ? ctas : cap), 256, 0, st>>>(x, y, n, vec_ok);
  return check_launch("unary");
}
template <typename T, typename Op>
static int launch_binary(const T *a, const T *b, T *y, int64_t n, int sm, cudaStream_t st) {
  const int vec_ok = aligned16(a) && aligned16(b) && aligned16(y);
  int64_t ctas = (n / Vec16<T>::N + 256 * EW_U - 1) / (256 * EW_U) + 1;
  const int64_t cap = (int64_t)sm * 16;
  binary_kernel<T, Op><<<(unsigned)(ctas < cap ? ctas : cap), 256, 0, st>>>(a, b, y, n, vec_ok);
  return check_launch("binary");
}

template <typename T>
static int unary_dispatch(int op, const void *x, void *y, int64_t n, int sm, cudaStream_t st) {
  const T *xi = (const T *)x;
  T *yo = (T *)y;
  switch (op) {
    case HEXB_OP_GELU_TANH: return launch_unary<T, GeluTanh>(xi, yo, n, sm, st);
    case HEXB_OP_COS: return launch_unary<T, Cos>(xi, yo, n, sm, st);
    case HEXB_OP_SIN: return launch_unary<T, Sin>(xi, yo, n, sm, st);
    case HEXB_OP_RSQRT: return launch_unary<T, Rsqrt>(xi, yo, n, sm, st);
    default: return HEXB_ERR_UNSUPPORTED;
  }
}
template <typename T>
static int binary_dispatch(int op, const void *a, const void *b, void *y, int64_t n, int sm, cudaStream_t st) {
  const T *ai = (const T *)a, *bi = (const T *)b;
  T *yo = (T *)y;
  switch (op) {
    case HEXB_OP_ADD: return launch_binary<T, Add>(ai, bi, yo, n, sm, st);
    case HEXB_OP_SUB: return launch_binary<T, Sub>(ai, bi, yo, n, sm, st);
    case HEXB_OP_MUL: return launch_binary<T, Mul>(ai, bi, yo, n, sm, st);
    case HEXB_OP_DIV: return launch_binary<T, Div>(ai, bi, yo, n, sm, st);
    default: return HEXB_ERR_UNSUPPORTED;
  }
}

}  // namespace hexb

using namespace hexb;

extern "C" int hexb_unary(int op, int dtype, const void *x, void *y, int64_t n, void *stream) {
  if (n < 0) return HEXB_ERR_BAD_ARG;
  if (dtype != HEXB_DT_F16 && dtype != HEXB_DT_F32) return HEXB_ERR_UNSUPPORTED;
  if (op < HEXB_OP_GELU_TANH || op > HEXB_OP_RSQRT) return HEXB_ERR_UNSUPPORTED;
  if (n == 0) return HEXB_OK;
  if (!x || !y) return HEXB_ERR_BAD_ARG;
  DeviceInfo di;
  if (int s = current_device(&di)) return s;
  return dtype == HEXB_DT_F16 ? unary_dispatch<__half>(op, x, y, n, di.sm_count, (cudaStream_t)stream)
                              : unary_dispatch<float>(op, x, y, n, di.sm_count, (cudaStream_t)stream);
}

extern "C" int hexb_binary(int op, int dtype, const void *a, const void *b, void *y, int64_t n, void *stream) {
  if (n < 0) return HEXB_ERR_BAD_ARG;
  if (dtype != HEXB_DT_F16 && dtype != HEXB_DT_F32) return HEXB_ERR_UNSUPPORTED;
  if (op < HEXB_OP_ADD || op > HEXB_OP_DIV) return HEXB_ERR_UNSUPPORTED;
  if (n == 0) return HEXB_OK;
  if (!a || !b || !y) return HEXB_ERR_BAD_ARG;
  DeviceInfo di;
  if (int s = current_device(&di)) return s;
  return dtype == HEXB_DT_F16 ? binary_dispatch<__half>(op, a, b, y, n, di.sm_count, (cudaStream_t)stream)
                              : binary_dispatch<float>(op, a, b, y, n, di.sm_count, (cudaStream_t)stream);
}

extern "C" int hexb_sum(int dtype, const void *x, void *out, int64_t n, void *stream) {
  if (n < 0) return HEXB_ERR_BAD_ARG;
  if (dtype != HEXB_DT_F16 && dtype != HEXB_DT_F32) return HEXB_ERR_UNSUPPORTED;
  if (!out || (n > 0 && !x)) return HEXB_ERR_BAD_ARG;
  DeviceInfo di;
  if (int s = current_device(&di)) return s;
  if (dtype == HEXB_DT_F16) return launch_sum<__half>((const __half *)x, (__half *)out, n, di.sm_count, (cudaStream_t)stream);
  return launch_sum<float>((const float *)x, (float *)out, n, di.sm_count, (cudaStream_t)stream);
}

extern "C" int hexb_rope(int dtype, const void *x, void *out, int64_t B, int64_t L, int64_t H, int64_t D,
                         const int64_t *x_strides, const int64_t *out_strides, float theta, void *stream) {
  if (B < 0 || L < 0 || H < 0 || D < 0) return HEXB_ERR_BAD_ARG;
  if (dtype != HEXB_DT_F16 && dtype != HEXB_DT_F32) return HEXB_ERR_UNSUPPORTED;
  if (B == 0 || L == 0 || H == 0 || D == 0) return HEXB_OK;
  if (!x || !out || !x_strides || !out_strides || !(theta > 0.f)) return HEXB_ERR_BAD_ARG;
  if (D % 2) return HEXB_ERR_UNSUPPORTED;
  DeviceInfo di;
  if (int s = current_device(&di)) return s;
  const float k = -log2f(theta) / (float)D;
  const int E = dtype == HEXB_DT_F16 ? 8 : 4;
  bool vec = aligned16(x) && aligned16(out) && D % E == 0 && D / E <= 256 && L <= 0x7fffffffll;
  for (int i = 0; i < 3 && vec; ++i) vec = x_strides[i] % E == 0 && out_strides[i] % E == 0;
  if (vec) {
    if (dtype == HEXB_DT_F16)
      rope_rows_kernel<__half><<<(unsigned)L, 256, 0, (cudaStream_t)stream>>>((const __half *)x, (__half *)out, B, L, H, D,
          x_strides[0], x_strides[1], x_strides[2], out_strides[0], out_strides[1], out_strides[2], k);
    else
      rope_rows_kernel<float><<<(unsigned)L, 256, 0, (cudaStream_t)stream>>>((const float *)x, (float *)out, B, L, H, D,
          x_strides[0], x_strides[1], x_strides[2], out_strides[0], out_strides[1], out_strides[2], k);
    return check_launch("rope_rows");
  }
  const int64_t total = B * L * H * (D / 2);
  int64_t ctas = (total + 255) / 256;
  const int64_t cap = (int64_t)di.sm_count * 16;
  const unsigned grid = (unsigned)(ctas < cap ? ctas : cap);
  if (dtype == HEXB_DT_F16)
    rope_kernel<__half><<<grid, 256, 0, (cudaStream_t)stream>>>((const __half *)x, (__half *)out, B, L, H, D, x_strides[0],
        x_strides[1], x_strides[2], out_strides[0], out_strides[1], out_strides[2], k);
  else
    rope_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>((const float *)x, (float *)out, B, L, H, D, x_strides[0],
        x_strides[1], x_strides[2], out_strides[0], out_strides[1], out_strides[2], k);
  return check_launch("rope");
}

extern "C" int hexb_iota(int dtype, void *out, int64_t n, void *stream) {
  if (n < 0) return HEXB_ERR_BAD_ARG;
  if (dtype != HEXB_DT_F16 && dtype != HEXB_DT_F32) return HEXB_ERR_UNSUPPORTED;
  if (n == 0) return HEXB_OK;
  if (!out) return HEXB_ERR_BAD_ARG;
  DeviceInfo di;
  if (int s = current_device(&di)) return s;
  int64_t ctas = (n + 255) / 256;
  const int64_t cap = (int64_t)di.sm_count * 16;
  const unsigned grid = (unsigned)(ctas < cap ? ctas : cap);
  if (dtype == HEXB_DT_F16) iota_kernel<__half><<<grid, 256, 0, (cudaStream_t)stream>>>((__half *)out, n);
  else iota_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>((float *)out, n);
  return check_launch("iota");
}
