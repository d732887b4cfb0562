// Row softmax for sm_100a.
//
// Reference semantics: softmax_kernel (test/python/triton/test_softmax.py:44-72) and the two-phase
// online_softmax (test/python/triton/test_online_softmax.py:30-81) of qualcomm/hexagon-mlir:
// y = exp(x - rowmax) / sum(exp(x - rowmax)), exp evaluated in fp32 for fp16 data as well.
// The Hexagon lowering walks each row four times through memory
// (docs/tutorials/triton/softmax.md:160-229); here a row is read once, kept in registers and
// written once, so the kernel moves the algorithmic 2 * rows * cols * sizeof(T) bytes.
#include "rowwise.cuh"

namespace hexb {

constexpr float kLog2e = 1.4426950408889634f;

// Register-resident path: cols is a multiple of the 16-byte vector, pointers/strides 16-byte aligned.
template <typename T, int VPT, int TPR, int THREADS>
__global__ void __launch_bounds__(THREADS)
softmax_rows_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t rows, int nvec,
                    int64_t xs, int64_t ys) {
  constexpr int E = Vec16<T>::N;
  constexpr int RPC = THREADS / TPR;
  __shared__ float red[3 * (THREADS / 32)];
  const int tr = threadIdx.x % TPR;
  const int rl = threadIdx.x / TPR;

  for (int64_t row0 = (int64_t)blockIdx.x * RPC; row0 < rows; row0 += (int64_t)gridDim.x * RPC) {
    const int64_t row = row0 + rl;
    const bool rv = row < rows;
    float f[VPT][E];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tr + i * TPR;
      if (rv && vi < nvec) {
        Vec16<T> v;
        v.raw = __ldg(reinterpret_cast<const decltype(v.raw) *>(x + row * xs + (int64_t)vi * E));
        v.unpack(f[i]);
      } else {
#pragma unroll
        for (int e = 0; e < E; ++e) f[i][e] = -INFINITY;
      }
#pragma unroll
      for (int e = 0; e < E; ++e) m = fmaxf(m, f[i][e]);
    }
    m = group_allreduce<MaxOp, TPR, THREADS>(m, red, 0);
    if (m == -INFINITY) m = 0.f;  // fully masked (out-of-range) row: keep the arithmetic finite
    const float mb = m * kLog2e;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int e = 0; e < E; ++e) {
        f[i][e] = exp2f(fmaf(f[i][e], kLog2e, -mb));
        s += f[i][e];
      }
    s = group_allreduce<SumOp, TPR, THREADS>(s, red, 1);
    const float inv = 1.0f / s;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tr + i * TPR;
      if (rv && vi < nvec) {
#pragma unroll
        for (int e = 0; e < E; ++e) f[i][e] *= inv;
        Vec16<T> v;
        v.pack(f[i]);
        *reinterpret_cast<decltype(v.raw) *>(y + row * ys + (int64_t)vi * E) = v.raw;
      }
    }
    if constexpr (TPR > 32) __syncthreads();  // `red` slots are reused by the next row
  }
}

// Streaming path for any width / alignment: one CTA per row, online (max, sum) over the row, then
// a second sweep that normalises (the row is re-read; at these sizes it comes from L2).
template <typename T>
__global__ void __launch_bounds__(256)
softmax_stream_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t rows, int64_t cols,
                      int64_t xs, int64_t ys) {
  __shared__ float sm[8], sl[8];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T *xr = x + row * xs;
    T *yr = y + row * ys;
    float m = -INFINITY, l = 0.f;
    for (int64_t c = threadIdx.x; c < cols; c += 256) {
      const float v = to_f32<T>(xr[c]);
      const float mn = fmaxf(m, v);
      if (mn != -INFINITY) l = l * exp2f((m - mn) * kLog2e) + exp2f((v - mn) * kLog2e);
      m = mn;
    }
    // merge (m, l) pairs: warp, then CTA
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float mo = __shfl_xor_sync(0xffffffffu, m, o);
      const float lo = __shfl_xor_sync(0xffffffffu, l, o);
      const float mn = fmaxf(m, mo);
      const float a = (m == -INFINITY) ? 0.f : exp2f((m - mn) * kLog2e);
      const float b = (mo == -INFINITY) ? 0.f : exp2f((mo - mn) * kLog2e);
      l = l * a + lo * b;
      m = mn;
    }
    const int warp = threadIdx.x >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) { sm[warp] = m; sl[warp] = l; }
    __syncthreads();
    float M = sm[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) M = fmaxf(M, sm[i]);
    float L = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) L += (sm[i] == -INFINITY) ? 0.f : sl[i] * exp2f((sm[i] - M) * kLog2e);
    const float inv = 1.0f / L;
    for (int64_t c = threadIdx.x; c < cols; c += 256)
      yr[c] = from_f32<T>(exp2f((to_f32<T>(xr[c]) - M) * kLog2e) * inv);
  }
}

template <typename T>
static int softmax_launch(const T *x, T *y, int64_t rows, int64_t cols, int64_t xs, int64_t ys,
                          cudaStream_t st) {
  if (rows < 0 || cols < 0) return HEXB_ERR_BAD_ARG;
  if (rows == 0 || cols == 0) return HEXB_OK;
  if (!x || !y) return HEXB_ERR_BAD_ARG;
  if (xs < cols || ys < cols) return HEXB_ERR_BAD_ARG;
  DeviceInfo di;
  if (int s = current_device(&di)) return s;
  constexpr int E = Vec16<T>::N;
  const bool vec_ok = (cols % E == 0) && (xs % E == 0) && (ys % E == 0) && aligned16(x) && aligned16(y);
  int tpr = 0, vpt = 0;
  if (vec_ok && !option("softmax_force_stream", 0) &&
      choose_row_shape(cols / E, option("softmax_vpt_max", 8), &tpr, &vpt)) {
    const int nvec = (int)(cols / E);
#define LAUNCH(TPR, VPT)                                                                       \
  {                                                                                            \
    constexpr int TH = CtaThreads<TPR>::value;                                                 \
    const int64_t ctas = (rows + TH / TPR - 1) / (TH / TPR);                                   \
    const int64_t cap = (int64_t)di.sm_count * 16;                                             \
    softmax_rows_kernel<T, VPT, TPR, TH><<<(unsigned)(ctas < cap ? ctas : cap), TH, 0, st>>>(  \
        x, y, rows, nvec, xs, ys);                                                             \
  }
    HEXB_ROW_SHAPE_SWITCH(tpr, vpt, LAUNCH)
#undef LAUNCH
  } else {
    const int64_t cap = (int64_t)di.sm_count * 8;
    softmax_stream_kernel<T><<<(unsigned)(rows < cap ? rows : cap), 256, 0, st>>>(x, y, rows, cols, xs, ys);
  }
  return check_launch("softmax");
}

}  // namespace hexb

extern "C" int hexb_softmax_f32(const float *x, float *y, int64_t rows, int64_t cols,
                                int64_t xs, int64_t ys, void *stream) {
  return hexb::softmax_launch<float>(x, y, rows, cols, xs, ys, (cudaStream_t)stream);
}
extern "C" int hexb_softmax_f16(const void *x, void *y, int64_t rows, int64_t cols, int64_t xs,
                                int64_t ys, void *stream) {
  return hexb::softmax_launch<__half>((const __half *)x, (__half *)y, rows, cols, xs, ys,
                                      (cudaStream_t)stream);
}
