// LayerNorm / RMSNorm forward for sm_100a.
//
// Reference semantics (qualcomm/hexagon-mlir):
//   layer_norm_fwd_kernel, test/python/triton/test_layer_norm.py:42-82:
//     mean = sum(x)/N; var = sum((x-mean)^2)/N (biased, centred two-pass form);
//     rstd = 1/sqrt(var+eps); y = (x-mean)*rstd*w + b; mean[row], rstd[row] are stored too.
//   rms_norm_fwd_kernel, test/python/triton/test_rms_norm.py:37-63:
//     y = (x / sqrt(sum(x^2)/N + eps)) * g.
// The row lives in registers between the statistics and the normalisation, so HBM is touched once
// each way; the two reduction passes of the reference run over registers, not memory.  Gains and
// biases are loaded once per thread and reused for every row the thread's CTA walks.
#include "rowwise.cuh"

namespace hexb {

template <typename T, int VPT, int TPR, int THREADS, bool RMS>
__global__ void __launch_bounds__(THREADS)
norm_rows_kernel(const T *__restrict__ x, T *__restrict__ y, const T *__restrict__ w,
                 const T *__restrict__ b, float *__restrict__ mean_out,
                 float *__restrict__ rstd_out, int64_t rows, int nvec, int64_t xs, int64_t ys,
                 float inv_n, float eps) {
  constexpr int E = Vec16<T>::N;
  constexpr int RPC = THREADS / TPR;
  using Raw = decltype(Vec16<T>::raw);
  __shared__ float red[3 * (THREADS / 32)];
  const int tr = threadIdx.x % TPR;
  const int rl = threadIdx.x / TPR;

  Vec16<T> wv[VPT], bv[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = tr + i * TPR;
    if (vi < nvec) {
      wv[i].raw = __ldg(reinterpret_cast<const Raw *>(w) + vi);
      if constexpr (!RMS) bv[i].raw = __ldg(reinterpret_cast<const Raw *>(b) + vi);
    } else {
      wv[i].raw = Raw{};
      if constexpr (!RMS) bv[i].raw = Raw{};
    }
  }

  for (int64_t row0 = (int64_t)blockIdx.x * RPC; row0 < rows; row0 += (int64_t)gridDim.x * RPC) {
    const int64_t row = row0 + rl;
    const bool rv = row < rows;
    float f[VPT][E];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tr + i * TPR;
      if (rv && vi < nvec) {
        Vec16<T> v;
        v.raw = ld_stream_as<Raw>(x + row * xs + (int64_t)vi * E);
        v.unpack(f[i]);
      } else {
#pragma unroll
        for (int e = 0; e < E; ++e) f[i][e] = 0.f;
      }
#pragma unroll
      for (int e = 0; e < E; ++e) s += RMS ? f[i][e] * f[i][e] : f[i][e];
    }
    s = group_allreduce<SumOp, TPR, THREADS>(s, red, 0);
    float mean = 0.f, rstd;
    if constexpr (RMS) {
      rstd = 1.0f / sqrtf(s * inv_n + eps);
    } else {
      mean = s * inv_n;
      float q = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const bool vv = tr + i * TPR < nvec;
#pragma unroll
        for (int e = 0; e < E; ++e) {
          f[i][e] = vv ? f[i][e] - mean : 0.f;
          q += f[i][e] * f[i][e];
        }
      }
      q = group_allreduce<SumOp, TPR, THREADS>(q, red, 1);
      rstd = 1.0f / sqrtf(q * inv_n + eps);
      if (rv && tr == 0) {
        if (mean_out) mean_out[row] = mean;
        if (rstd_out) rstd_out[row] = rstd;
      }
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tr + i * TPR;
      if (rv && vi < nvec) {
        float wf[E], bf[E];
        wv[i].unpack(wf);
        if constexpr (!RMS) bv[i].unpack(bf);
#pragma unroll
        for (int e = 0; e < E; ++e)
          f[i][e] = RMS ? (f[i][e] * rstd) * wf[e] : fmaf(f[i][e] * rstd, wf[e], bf[e]);
        Vec16<T> v;
        v.pack(f[i]);
        st_stream_as<Raw>(y + row * ys + (int64_t)vi * E, v.raw);
      }
    }
    if constexpr (TPR > 32) __syncthreads();
  }
}

// Any width / alignment: one CTA per row, the reference's pass structure over global memory
// (sum; centred squares; normalise).  Rows this path sees are short or odd-sized, so the re-reads
// are served by L1/L2.
template <typename T, bool RMS>
__global__ void __launch_bounds__(256)
norm_stream_kernel(const T *__restrict__ x, T *__restrict__ y, const T *__restrict__ w,
                   const T *__restrict__ b, float *__restrict__ mean_out,
                   float *__restrict__ rstd_out, int64_t rows, int64_t cols, int64_t xs, int64_t ys,
                   float inv_n, float eps) {
  __shared__ float red[3 * 8];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T *xr = x + row * xs;
    T *yr = y + row * ys;
    float s = 0.f;
    for (int64_t c = threadIdx.x; c < cols; c += 256) {
      const float v = to_f32<T>(xr[c]);
      s += RMS ? v * v : v;
    }
    s = group_allreduce<SumOp, 256, 256>(s, red, 0);
    float mean = 0.f, rstd;
    if constexpr (RMS) {
      rstd = 1.0f / sqrtf(s * inv_n + eps);
    } else {
      mean = s * inv_n;
      float q = 0.f;
      for (int64_t c = threadIdx.x; c < cols; c += 256) {
        const float d = to_f32<T>(xr[c]) - mean;
        q += d * d;
      }
      q = group_allreduce<SumOp, 256, 256>(q, red, 1);
      rstd = 1.0f / sqrtf(q * inv_n + eps);
      if (threadIdx.x == 0) {
        if (mean_out) mean_out[row] = mean;
        if (rstd_out) rstd_out[row] = rstd;
      }
    }
    for (int64_t c = threadIdx.x; c < cols; c += 256) {
      const float v = to_f32<T>(xr[c]);
      const float o = RMS ? (v * rstd) * to_f32<T>(w[c])
                          : fmaf((v - mean) * rstd, to_f32<T>(w[c]), to_f32<T>(b[c]));
      yr[c] = from_f32<T>(o);
    }
    __syncthreads();
  }
}

template <typename T, bool RMS>
static int norm_launch(const T *x, T *y, const T *w, const T *b, float *mean, float *rstd,
                       int64_t rows, int64_t cols, int64_t xs, int64_t ys, float eps,
                       cudaStream_t st) {
  if (rows < 0 || cols < 0) return HEXB_ERR_BAD_ARG;
  if (rows == 0 || cols == 0) return HEXB_OK;
  if (!x || !y || !w || (!RMS && !b)) return HEXB_ERR_BAD_ARG;
  if (xs < cols || ys < cols) return HEXB_ERR_BAD_ARG;
  DeviceInfo di;
  if (int s = current_device(&di)) return s;
  constexpr int E = Vec16<T>::N;
  const float inv_n = 1.0f / (float)cols;
  const bool vec_ok = (cols % E == 0) && (xs % E == 0) && (ys % E == 0) && aligned16(x) &&
                      aligned16(y) && aligned16(w) && (RMS || aligned16(b));
  int tpr = 0, vpt = 0;
  const int vpt_max = option("norm_vpt_max", sizeof(T) == 2 ? 4 : 8);
  if (vec_ok && !option("norm_force_stream", 0) && choose_row_shape(cols / E, vpt_max, &tpr, &vpt)) {
    const int nvec = (int)(cols / E);
    const int waves = option("norm_ctas_per_sm", 8);
#define LAUNCH(TPR, VPT)                                                                          \
  {                                                                                               \
    constexpr int TH = CtaThreads<TPR>::value;                                                    \
    const int64_t ctas = (rows + TH / TPR - 1) / (TH / TPR);                                      \
    const int64_t cap = (int64_t)di.sm_count * waves;                                             \
    norm_rows_kernel<T, VPT, TPR, TH, RMS><<<(unsigned)(ctas < cap ? ctas : cap), TH, 0, st>>>(   \
        x, y, w, b, mean, rstd, rows, nvec, xs, ys, inv_n, eps);                                  \
  }
    HEXB_ROW_SHAPE_SWITCH(tpr, vpt, LAUNCH)
#undef LAUNCH
  } else {
    const int64_t cap = (int64_t)di.sm_count * 8;
    norm_stream_kernel<T, RMS><<<(unsigned)(rows < cap ? rows : cap), 256, 0, st>>>(
        x, y, w, b, mean, rstd, rows, cols, xs, ys, inv_n, eps);
  }
  return check_launch(RMS ? "rms_norm" : "layer_norm");
}

}  // namespace hexb

using hexb::norm_launch;

extern "C" int hexb_layer_norm_f32(const float *x, float *y, const float *w, const float *b,
                                   float *mean, float *rstd, int64_t rows, int64_t cols, int64_t xs,
                                   int64_t ys, float eps, void *stream) {
  return norm_launch<float, false>(x, y, w, b, mean, rstd, rows, cols, xs, ys, eps, (cudaStream_t)stream);
}
extern "C" int hexb_layer_norm_f16(const void *x, void *y, const void *w, const void *b, float *mean,
                                   float *rstd, int64_t rows, int64_t cols, int64_t xs, int64_t ys,
                                   float eps, void *stream) {
  return norm_launch<__half, false>((const __half *)x, (__half *)y, (const __half *)w,
                                    (const __half *)b, mean, rstd, rows, cols, xs, ys, eps,
                                    (cudaStream_t)stream);
}
extern "C" int hexb_rms_norm_f32(const float *x, float *y, const float *w, int64_t rows,
                                 int64_t cols, int64_t xs, int64_t ys, float eps, void *stream) {
  return norm_launch<float, true>(x, y, w, nullptr, nullptr, nullptr, rows, cols, xs, ys, eps,
                                  (cudaStream_t)stream);
}
extern "C" int hexb_rms_norm_f16(const void *x, void *y, const void *w, int64_t rows, int64_t cols,
                                 int64_t xs, int64_t ys, float eps, void *stream) {
  return norm_launch<__half, true>((const __half *)x, (__half *)y, (const __half *)w, nullptr,
                                   nullptr, nullptr, rows, cols, xs, ys, eps, (cudaStream_t)stream);
}
