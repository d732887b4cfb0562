// Row softmax for sm_100a.
//
// Reference semantics: softmax_kernel (test/python/triton/test_softmax.py:44-72) and the two-phase
// online_softmax (test/python/triton/test_online_softmax.py:30-81) of qualcomm/hexagon-mlir:
// y = exp(x - rowmax) / sum(exp(x - rowmax)), exp evaluated in fp32 for fp16 data as well.
// The Hexagon lowering walks each row four times through memory
// (docs/tutorials/triton/softmax.md:160-229); here a row is read once, kept in registers and
// written once, so the kernel moves the algorithmic 2 * rows * cols * sizeof(T) bytes.
#include "rowring.cuh"
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
  pdl_launch_dependents();
  pdl_wait();

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


static __device__ int g_softmax_status = 0;

// Persistent ring kernel (rowring.cuh): one warp per row, rows up to 8 KiB.
template <typename T, int VPL>
__global__ void __launch_bounds__(ring::THREADS, 1)
softmax_ring_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t rows, int nvec, int64_t xs,
                    int64_t ys, int slots, int slot_bytes, int map, int out_slots) {
  constexpr int E = Vec16<T>::N;
  using Raw = decltype(Vec16<T>::raw);
  extern __shared__ uint8_t smem_raw[];
  // out_slots > 0: a finished row is written to a shared-memory slot and leaves as one bulk store
  ring::WarpRing rg = ring::setup(smem_raw, slots, slot_bytes, 0, out_slots);
  int n_out = 0;
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t row_bytes = (uint32_t)nvec * 16u;
  const ring::RowWalk walk = ring::row_walk(rows, map);
  const int64_t stride_rows = walk.step, first = walk.first, row_end = walk.end;
  (void)warp;
  if (lane == 0) {
    for (int s = 0; s < slots; ++s) {
      const int64_t r = first + (int64_t)s * stride_rows;
      if (r < row_end) rg.arm(s, x + r * xs, row_bytes);
    }
  }
  int s = 0;
  uint32_t phase = 0;
  for (int64_t r = first; r < row_end; r += stride_rows) {
    if (!tc::mbar_wait(rg.bar(s), phase, rg.abort_flag)) break;
    float f[VPL][E];
    float m = -INFINITY;
    const uint32_t slot = rg.slot_addr(s);
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int vi = lane + 32 * j;
      if (vi < nvec) {
        uint4 raw = ring::lds128(slot + (uint32_t)vi * 16u);
        Vec16<T> v;
        v.raw = *reinterpret_cast<Raw *>(&raw);
        v.unpack(f[j]);
      } else {
#pragma unroll
        for (int e = 0; e < E; ++e) f[j][e] = -INFINITY;
      }
#pragma unroll
      for (int e = 0; e < E; ++e) m = fmaxf(m, f[j][e]);
    }
    m = warp_max(m);  // every lane's shared loads have completed once this returns
    if (lane == 0) {
      const int64_t rn = r + (int64_t)slots * stride_rows;
      if (rn < row_end) {
        tc::fence_proxy_async_smem();
        rg.arm(s, x + rn * xs, row_bytes);
      }
    }
    const float mb = m * kLog2e;
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j)
#pragma unroll
      for (int e = 0; e < E; ++e) {
        f[j][e] = exp2f(fmaf(f[j][e], kLog2e, -mb));
        sum += f[j][e];
      }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    T *yr = y + r * ys;
    uint32_t oslot = 0;
    if (out_slots) {
      if (lane == 0) {  // the bulk store that last used this output slot has finished reading it
        if (out_slots >= 2) tc::bulk_wait_group_read<1>();
        else tc::bulk_wait_group_read<0>();
      }
      __syncwarp();
      oslot = rg.out0 + (uint32_t)((n_out % out_slots) * slot_bytes);
    }
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int vi = lane + 32 * j;
      if (vi < nvec) {
#pragma unroll
        for (int e = 0; e < E; ++e) f[j][e] *= inv;
        Vec16<T> o;
        o.pack(f[j]);
        if (out_slots) ring::sts128(oslot + (uint32_t)vi * 16u, *reinterpret_cast<uint4 *>(&o.raw));
        else st_stream_as<Raw>(yr + (int64_t)vi * E, o.raw);
      }
    }
    if (out_slots) {
      tc::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        ring::bulk_store(yr, oslot, row_bytes);
        tc::bulk_commit_group();
      }
      ++n_out;
    }
    if (++s == slots) { s = 0; phase ^= 1u; }
  }
  if (out_slots && lane == 0) tc::bulk_wait_group_read<0>();
  if (*rg.abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    if (threadIdx.x == 0) atomicExch(&g_softmax_status, (int)HEXB_ERR_TIMEOUT);
  }
}

template <typename T, int VPL>
static int launch_softmax_ring(const T *x, T *y, int64_t rows, int nvec, int64_t xs, int64_t ys,
                               int sm_count, cudaStream_t st) {
  const int out_slots = (int)option(OPT_softmax_bulk_store, 0);  // measured slower here ([8192 x 1024] fp32: 12.6 vs 12.4 us)
  const ring::Layout lay = ring::make_layout(nvec * 16, 0, out_slots);
  auto kern = softmax_ring_kernel<T, VPL>;
  static PerDeviceOnce attr_done;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done.is_done(dev)) {
    HEXB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_done.mark(dev);
  }
  const int64_t groups = (rows + ring::WARPS - 1) / ring::WARPS;
  const int grid = (int)(groups < sm_count ? groups : sm_count);
  launch_pdl(kern, dim3(grid), dim3(ring::THREADS), (size_t)lay.smem_bytes, st, x, y, rows, nvec, xs, ys, lay.slots,
             lay.slot_bytes, (int)option(OPT_ring_map, 0), out_slots);
  return check_launch("softmax_ring");
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
  const int64_t row_bytes = cols * (int64_t)sizeof(T);
  // The ring form is kept selectable; for the row sizes measured (4 KiB rows) the register kernel
  // below is faster (11.8 vs 12.6 us on [8192 x 1024] fp32), so it is off by default.
  if (vec_ok && option(OPT_softmax_ring, 0) && row_bytes >= 512 && row_bytes <= ring::MAX_ROW_BYTES &&
      rows * row_bytes >= (4ll << 20)) {
    const int nvec = (int)(cols / E);
    const int need = (nvec + 31) / 32;
#define RING(VPL) return launch_softmax_ring<T, VPL>(x, y, rows, nvec, xs, ys, di.sm_count, st)
    if (need <= 1) RING(1);
    if (need <= 2) RING(2);
    if (need <= 4) RING(4);
    if (need <= 8) RING(8);
    RING(16);
#undef RING
  }
  // Vectors per thread: at most 8 for fp32, 4 for fp16.  A 16-byte vector of fp16 unpacks to eight fp32
  // registers, so 8 of them leave two CTAs per SM and too few loads in flight: [16384 x 4096] fp16 ran at
  // 3910 GB/s with 8 and 5895 with 4, [4096 x 8192] 3601 -> 5780; fp32 is level or better with 8.
  int tpr = 0, vpt = 0;
  if (vec_ok && !option(OPT_softmax_force_stream, 0) &&
      choose_row_shape(cols / E, option(OPT_softmax_vpt_max, sizeof(T) == 2 ? 4 : 8), &tpr, &vpt)) {
    const int nvec = (int)(cols / E);
#define LAUNCH(TPR, VPT)                                                                       \
  {                                                                                            \
    constexpr int TH = CtaThreads<TPR>::value;                                                 \
    const int64_t ctas = (rows + TH / TPR - 1) / (TH / TPR);                                   \
    const int64_t cap = (int64_t)di.sm_count * 16;                                             \
    launch_pdl(softmax_rows_kernel<T, VPT, TPR, TH>, dim3((unsigned)(ctas < cap ? ctas : cap)), dim3(TH), 0, st, \
               x, y, rows, nvec, xs, ys);                                                      \
  }
    HEXB_ROW_SHAPE_SWITCH(tpr, vpt, LAUNCH)
#undef LAUNCH
  } else {
    const int64_t cap = (int64_t)di.sm_count * 8;
    softmax_stream_kernel<T><<<(unsigned)(rows < cap ? rows : cap), 256, 0, st>>>(x, y, rows, cols, xs, ys);
  }
  return check_launch("softmax");
}

int softmax_device_status_fetch_and_clear(int *out) {
  int v = 0, zero = 0;
  HEXB_CUDA_OK(cudaMemcpyFromSymbol(&v, g_softmax_status, sizeof(int)));
  if (v) HEXB_CUDA_OK(cudaMemcpyToSymbol(g_softmax_status, &zero, sizeof(int)));
  *out = v;
  return HEXB_OK;
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
