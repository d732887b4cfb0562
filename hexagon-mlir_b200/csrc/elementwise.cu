// SiLU and SwiGLU gating for sm_100a.
//
// Reference semantics: silu_kernel, test/python/triton/test_silu.py:38-52 of qualcomm/hexagon-mlir:
// y = x / (1 + exp(-x)) with exp evaluated in fp32.  hexb_swiglu_f16 applies it to the gate half of
// a [rows, 2*cols] gate|up matrix and multiplies by the up half (the SwiGLU MLP of the decoder
// block stack).  Both are one read and one write per element with 16-byte accesses.
#include "common.cuh"

namespace hexb {

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

template <typename T>
__global__ void __launch_bounds__(256) silu_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t n,
                                                   int vec_ok) {
  constexpr int E = Vec16<T>::N;
  using Raw = decltype(Vec16<T>::raw);
  const int64_t tid = (int64_t)blockIdx.x * 256 + threadIdx.x;
  const int64_t nth = (int64_t)gridDim.x * 256;
  const int64_t nvec = vec_ok ? n / E : 0;
  for (int64_t v = tid; v < nvec; v += nth) {
    Vec16<T> a;
    a.raw = ld_stream_as<Raw>(x + v * E);
    float f[E];
    a.unpack(f);
#pragma unroll
    for (int e = 0; e < E; ++e) f[e] = silu_f(f[e]);
    a.pack(f);
    st_stream_as<Raw>(y + v * E, a.raw);
  }
  for (int64_t i = nvec * E + tid; i < n; i += nth) y[i] = from_f32<T>(silu_f(to_f32<T>(x[i])));
}

// out[r, c] = silu(gu[r, c]) * gu[r, cols + c]; cols % 8 == 0.
__global__ void __launch_bounds__(256) swiglu_kernel(const __half *__restrict__ gu, __half *__restrict__ out,
                                                     int64_t rows, int cols_vec) {
  const int64_t total = rows * cols_vec;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
    const int64_t r = i / cols_vec;
    const int c = (int)(i - r * cols_vec);
    const uint4 *row = reinterpret_cast<const uint4 *>(gu) + r * 2 * cols_vec;
    Vec16<__half> g, u;
    g.raw = ld_stream_as<uint4>(row + c);
    u.raw = ld_stream_as<uint4>(row + cols_vec + c);
    float gf[8], uf[8];
    g.unpack(gf);
    u.unpack(uf);
#pragma unroll
    for (int e = 0; e < 8; ++e) gf[e] = silu_f(gf[e]) * uf[e];
    g.pack(gf);
    st_stream_as<uint4>(reinterpret_cast<uint4 *>(out) + i, g.raw);
  }
}

template <typename T>
static int silu_launch(const T *x, T *y, int64_t n, cudaStream_t st) {
  if (n < 0) return HEXB_ERR_BAD_ARG;
  if (n == 0) return HEXB_OK;
  if (!x || !y) return HEXB_ERR_BAD_ARG;
  DeviceInfo di;
  if (int s = current_device(&di)) return s;
  const int vec_ok = aligned16(x) && aligned16(y);
  int64_t ctas = (n / Vec16<T>::N + 255) / 256 + 1;
  const int64_t cap = (int64_t)di.sm_count * 16;
  silu_kernel<T><<<(unsigned)(ctas < cap ? ctas : cap), 256, 0, st>>>(x, y, n, vec_ok);
  return check_launch("silu");
}

}  // namespace hexb

extern "C" int hexb_silu_f32(const float *x, float *y, int64_t n, void *stream) {
  return hexb::silu_launch<float>(x, y, n, (cudaStream_t)stream);
}
extern "C" int hexb_silu_f16(const void *x, void *y, int64_t n, void *stream) {
  return hexb::silu_launch<__half>((const __half *)x, (__half *)y, n, (cudaStream_t)stream);
}
extern "C" int hexb_swiglu_f16(const void *gu, void *out, int64_t rows, int64_t cols, void *stream) {
  using namespace hexb;
  if (rows < 0 || cols < 0) return HEXB_ERR_BAD_ARG;
  if (rows == 0 || cols == 0) return HEXB_OK;
  if (!gu || !out) return HEXB_ERR_BAD_ARG;
  if (cols % 8) return HEXB_ERR_UNSUPPORTED;
  if (!aligned16(gu) || !aligned16(out)) return HEXB_ERR_MISALIGNED;
  DeviceInfo di;
  if (int s = current_device(&di)) return s;
  const int64_t total = rows * (cols / 8);
  int64_t ctas = (total + 255) / 256;
  const int64_t cap = (int64_t)di.sm_count * 16;
  swiglu_kernel<<<(unsigned)(ctas < cap ? ctas : cap), 256, 0, (cudaStream_t)stream>>>(
      (const __half *)gu, (__half *)out, rows, (int)(cols / 8));
  return check_launch("swiglu");
}
