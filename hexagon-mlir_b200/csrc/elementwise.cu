// SiLU and SwiGLU gating for sm_100a.
//
// Reference semantics: silu_kernel, test/python/triton/test_silu.py:38-52 of qualcomm/hexagon-mlir:
// y = x / (1 + exp(-x)) with exp evaluated in fp32.  hexb_swiglu_f16 applies it to the gate half of
// a [rows, 2*cols] gate|up matrix and multiplies by the up half (the SwiGLU MLP of the decoder
// block stack).  Both are one read and one write per element with 16-byte accesses.
#include "common.cuh"

namespace hexb {

__device__ __forceinline__ float silu_f(float x) { return __fdividef(x, 1.0f + __expf(-x)); }  // 2 ulp
// fp16 data: x * sigmoid(x) = x/2 * (1 + tanh(x/2)) with the one-instruction tanh (2^-11), see tanh_approx
__device__ __forceinline__ float silu_h(float x) {
  const float hx = 0.5f * x;
  return fmaf(hx, tanh_approx(hx), hx);
}

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
    for (int e = 0; e < E; ++e) f[e] = sizeof(T) == 2 ? silu_h(f[e]) : silu_f(f[e]);
    a.pack(f);
    st_stream_as<Raw>(y + v * E, a.raw);
  }
  for (int64_t i = nvec * E + tid; i < n; i += nth)
    y[i] = from_f32<T>(sizeof(T) == 2 ? silu_h(to_f32<T>(x[i])) : silu_f(to_f32<T>(x[i])));
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

// ------------------------------------------------------------------ token + position embedding
// out[t, :] = wte[ids[t], :] + wpe[t % seq, :]: the first op of the GPT-2 graph the reference compiles
// through torch-mlir (test/python/torch-mlir/gpt2lmheadmodel.py:143-169).  One warp per token row,
// 16-byte accesses.  An id outside [0, vocab) writes a zero row and raises the device status word.
namespace hexb {

static __device__ int g_embed_status = 0;

__global__ void __launch_bounds__(256)
embedding_kernel(const __half *__restrict__ wte, const __half *__restrict__ wpe, const int64_t *__restrict__ ids,
                 __half *__restrict__ out, int64_t n_tokens, int64_t seq, int d_model, int64_t vocab, int vec_ok) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= n_tokens) return;
  const int64_t id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  if (!ok && lane == 0) atomicExch(&g_embed_status, (int)HEXB_ERR_BAD_ARG);
  const __half *te = wte + (ok ? id : 0) * d_model;
  const __half *pe = wpe + (t % seq) * d_model;
  __half *o = out + t * d_model;
  const int nvec = vec_ok ? d_model / 8 : 0;
  for (int v = lane; v < nvec; v += 32) {
    Vec16<__half> a, b;
    a.raw = __ldg(reinterpret_cast<const uint4 *>(te + v * 8));
    b.raw = __ldg(reinterpret_cast<const uint4 *>(pe + v * 8));
    float fa[8], fb[8];
    a.unpack(fa);
    b.unpack(fb);
#pragma unroll
    for (int e = 0; e < 8; ++e) fa[e] = ok ? fa[e] + fb[e] : 0.f;
    a.pack(fa);
    *reinterpret_cast<uint4 *>(o + v * 8) = a.raw;
  }
  for (int c = nvec * 8 + lane; c < d_model; c += 32)
    o[c] = ok ? __float2half_rn(__half2float(te[c]) + __half2float(pe[c])) : __float2half_rn(0.f);
}

int embed_device_status_fetch_and_clear(int *out) {
  int v = 0, zero = 0;
  HEXB_CUDA_OK(cudaMemcpyFromSymbol(&v, g_embed_status, sizeof(int)));
  if (v) HEXB_CUDA_OK(cudaMemcpyToSymbol(g_embed_status, &zero, sizeof(int)));
  *out = v;
  return HEXB_OK;
}

}  // namespace hexb

extern "C" int hexb_embedding_f16(const void *wte, const void *wpe, const int64_t *ids, void *out, int64_t n_tokens,
                                  int64_t seq, int64_t d_model, int64_t vocab, int64_t n_positions, void *stream) {
  using namespace hexb;
  if (n_tokens < 0 || seq <= 0 || d_model < 0 || vocab <= 0 || n_positions < seq) return HEXB_ERR_BAD_ARG;
  if (n_tokens == 0 || d_model == 0) return HEXB_OK;
  if (!wte || !wpe || !ids || !out) return HEXB_ERR_BAD_ARG;
  if (d_model >= (1ll << 31)) return HEXB_ERR_UNSUPPORTED;
  const int64_t ctas = (n_tokens + 7) / 8;
  if (ctas > 0x7fffffffll) return HEXB_ERR_UNSUPPORTED;
  const int vec_ok = d_model % 8 == 0 && aligned16(wte) && aligned16(wpe) && aligned16(out);
  embedding_kernel<<<(unsigned)ctas, 256, 0, (cudaStream_t)stream>>>((const __half *)wte, (const __half *)wpe, ids,
                                                                    (__half *)out, n_tokens, seq, (int)d_model, vocab,
                                                                    vec_ok);
  return check_launch("embedding");
}
