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
#include "rowring.cuh"
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


// ---- fp16 fast path of the ring kernel: the row, gains and biases stay packed (two fp16 per
// register).  Statistics accumulate in fp32 straight from the fp16 operands with the sm_100
// mixed-precision add / sub / fma (no separate conversion); the normalised value
// (x - mean) * rstd is formed in fp32, rounded to fp16 and the affine step runs as one packed
// fp16 fma per pair.
__device__ __forceinline__ void h2_sum(uint32_t w, float &s) {
  asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\t"
      "add.rn.f32.f16 %0, lo, %0;\n\tadd.rn.f32.f16 %0, hi, %0;\n\t}"
      : "+f"(s) : "r"(w));
}
__device__ __forceinline__ void h2_sumsq(uint32_t w, float &q) {
  asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\t"
      "fma.rn.f32.f16 %0, lo, lo, %0;\n\tfma.rn.f32.f16 %0, hi, hi, %0;\n\t}"
      : "+f"(q) : "r"(w));
}
__device__ __forceinline__ void h2_centred_sumsq(uint32_t w, float mean, float &q) {
  asm("{\n\t.reg .b16 lo, hi;\n\t.reg .f32 d0, d1;\n\tmov.b32 {lo, hi}, %1;\n\t"
      "sub.rn.f32.f16 d0, lo, %2;\n\tsub.rn.f32.f16 d1, hi, %2;\n\t"
      "fma.rn.f32 %0, d0, d0, %0;\n\tfma.rn.f32 %0, d1, d1, %0;\n\t}"
      : "+f"(q) : "r"(w), "f"(mean));
}
// ((x - mean) * rstd) -> fp16 pair, then * g + b in packed fp16.
__device__ __forceinline__ uint32_t h2_norm_affine(uint32_t w, float mean, float rstd, uint32_t g, uint32_t b) {
  uint32_t out;
  asm("{\n\t.reg .b16 lo, hi;\n\t.reg .f32 d0, d1;\n\t.reg .b32 t;\n\tmov.b32 {lo, hi}, %1;\n\t"
      "sub.rn.f32.f16 d0, lo, %2;\n\tsub.rn.f32.f16 d1, hi, %2;\n\t"
      "mul.rn.f32 d0, d0, %3;\n\tmul.rn.f32 d1, d1, %3;\n\t"
      "cvt.rn.f16x2.f32 t, d1, d0;\n\tfma.rn.f16x2 %0, t, %4, %5;\n\t}"
      : "=r"(out) : "r"(w), "f"(mean), "f"(rstd), "r"(g), "r"(b));
  return out;
}
// (x * rstd) -> fp16 pair, then * g in packed fp16.
__device__ __forceinline__ uint32_t h2_norm_scale(uint32_t w, float rstd, uint32_t g) {
  uint32_t out;
  asm("{\n\t.reg .b16 lo, hi;\n\t.reg .f32 d0, d1;\n\t.reg .b32 t;\n\tmov.b32 {lo, hi}, %1;\n\t"
      "sub.rn.f32.f16 d0, lo, 0f00000000;\n\tsub.rn.f32.f16 d1, hi, 0f00000000;\n\t"
      "mul.rn.f32 d0, d0, %2;\n\tmul.rn.f32 d1, d1, %2;\n\t"
      "cvt.rn.f16x2.f32 t, d1, d0;\n\tmul.rn.f16x2 %0, t, %3;\n\t}"
      : "=r"(out) : "r"(w), "f"(rstd), "r"(g));
  return out;
}
// The same two steps with the affine part in fp32 and ONE rounding at the end, as the reference's
// fp32 expression (x - mean) * rstd * w + b rounds (test/python/triton/test_layer_norm.py:78-81).  The
// gains and biases are widened by a mixed-precision subtract of +0 (exact, FMA pipe) rather than by
// cvt.f32.f16, which runs on the special-function unit at 16 per clock and SM (two per element kept that
// unit 81 % busy in the [16384 x 4096] launch); RMSNorm forms x * g exactly with the mixed-precision
// multiply-add (the product of two fp16 values fits fp32) and applies rstd to that.
__device__ __forceinline__ uint32_t h2_norm_affine_f32(uint32_t w, float mean, float rstd, uint32_t g, uint32_t b) {
  uint32_t out;
  asm("{\n\t.reg .b16 lo, hi, glo, ghi, blo, bhi;\n\t.reg .f32 d0, d1, g0, g1, b0, b1;\n\t"
      "mov.b32 {lo, hi}, %1;\n\tmov.b32 {glo, ghi}, %4;\n\tmov.b32 {blo, bhi}, %5;\n\t"
      "sub.rn.f32.f16 d0, lo, %2;\n\tsub.rn.f32.f16 d1, hi, %2;\n\t"
      "mul.rn.f32 d0, d0, %3;\n\tmul.rn.f32 d1, d1, %3;\n\t"
      "sub.rn.f32.f16 g0, glo, 0f00000000;\n\tsub.rn.f32.f16 g1, ghi, 0f00000000;\n\t"
      "sub.rn.f32.f16 b0, blo, 0f00000000;\n\tsub.rn.f32.f16 b1, bhi, 0f00000000;\n\t"
      "fma.rn.f32 d0, d0, g0, b0;\n\tfma.rn.f32 d1, d1, g1, b1;\n\t"
      "cvt.rn.f16x2.f32 %0, d1, d0;\n\t}"
      : "=r"(out) : "r"(w), "f"(mean), "f"(rstd), "r"(g), "r"(b));
  return out;
}
__device__ __forceinline__ uint32_t h2_norm_scale_f32(uint32_t w, float rstd, uint32_t g) {
  uint32_t out;
  asm("{\n\t.reg .b16 lo, hi, glo, ghi;\n\t.reg .f32 d0, d1;\n\t"
      "mov.b32 {lo, hi}, %1;\n\tmov.b32 {glo, ghi}, %3;\n\t"
      "fma.rn.f32.f16 d0, lo, glo, 0f00000000;\n\tfma.rn.f32.f16 d1, hi, ghi, 0f00000000;\n\t"
      "mul.rn.f32 d0, d0, %2;\n\tmul.rn.f32 d1, d1, %2;\n\t"
      "cvt.rn.f16x2.f32 %0, d1, d0;\n\t}"
      : "=r"(out) : "r"(w), "f"(rstd), "r"(g));
  return out;
}
__device__ __forceinline__ uint32_t &word(uint4 &v, int c) { return c == 0 ? v.x : c == 1 ? v.y : c == 2 ? v.z : v.w; }

static __device__ int g_norm_status = 0;

// Persistent ring kernel (rowring.cuh): one warp per row, the row pulled from the warp's
// shared-memory ring into registers (packed, VPL 16-byte vectors per lane), gains and biases held in
// registers for the whole launch.  Rows up to 8 KiB.
template <typename T, int VPL, bool RMS>
__global__ void __launch_bounds__(ring::THREADS, 1)
norm_ring_kernel(const T *__restrict__ x, T *__restrict__ y, const T *__restrict__ w,
                 const T *__restrict__ b, float *__restrict__ mean_out, float *__restrict__ rstd_out,
                 int64_t rows, int nvec, int64_t xs, int64_t ys, float inv_n, float eps, int slots,
                 int slot_bytes, int map, int out_slots, int affine_f32) {
  constexpr int E = Vec16<T>::N;
  using Raw = decltype(Vec16<T>::raw);
  extern __shared__ uint8_t smem_raw[];
  // out_slots > 0: a finished row is written to a shared-memory slot and leaves as one bulk store
  ring::WarpRing rg = ring::setup(smem_raw, slots, slot_bytes, 0, out_slots);
  int n_out = 0;
  pdl_launch_dependents();
  pdl_wait();  // the ring is set up; from here on global memory is touched
  constexpr int store_mode = 0;  // streaming stores (default-policy, .cs and evict-first hints measured within noise)
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
  // Widest rows: x (64 registers) and the gains (64) stay in registers, the biases live in shared
  // memory (one 16-byte load per vector and row) so that nothing spills.
  constexpr bool B_SMEM = false;  // set to (!RMS && VPL == 16) to park the biases in shared memory
  constexpr int BREG = (RMS || B_SMEM) ? 1 : VPL;
  Vec16<T> wv[VPL], bv[BREG];
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int vi = lane + 32 * j;
    wv[j].raw = vi < nvec ? __ldg(reinterpret_cast<const Raw *>(w) + vi) : Raw{};
    if constexpr (!RMS && !B_SMEM) bv[j].raw = vi < nvec ? __ldg(reinterpret_cast<const Raw *>(b) + vi) : Raw{};
  }
  if constexpr (B_SMEM) {
    for (int vi = threadIdx.x; vi < nvec; vi += ring::THREADS)
      ring::sts128(rg.extra + (uint32_t)vi * 16u, __ldg(reinterpret_cast<const uint4 *>(b) + vi));
    __syncthreads();
  }

  int s = 0;
  uint32_t phase = 0;
  for (int64_t r = first; r < row_end; r += stride_rows) {
    if (!tc::mbar_wait(rg.bar(s), phase, rg.abort_flag)) break;
    Vec16<T> xv[VPL];
    float sum = 0.f;
    const uint32_t slot = rg.slot_addr(s);
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int vi = lane + 32 * j;
      uint4 raw = make_uint4(0u, 0u, 0u, 0u);
      if (vi < nvec) raw = ring::lds128(slot + (uint32_t)vi * 16u);
      xv[j].raw = *reinterpret_cast<Raw *>(&raw);
    }
    if constexpr (sizeof(T) == 2) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < VPL; ++j) {
        uint4 &raw = *reinterpret_cast<uint4 *>(&xv[j].raw);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          if constexpr (RMS) h2_sumsq(word(raw, c), acc[c]);
          else h2_sum(word(raw, c), acc[c]);
        }
      }
      sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    } else {
#pragma unroll
      for (int j = 0; j < VPL; ++j) {
        float f[E];
        xv[j].unpack(f);
#pragma unroll
        for (int e = 0; e < E; ++e) sum += RMS ? f[e] * f[e] : f[e];
      }
    }
    sum = warp_sum(sum);  // every lane's shared loads have completed once this returns
    if (lane == 0) {
      const int64_t rn = r + (int64_t)slots * stride_rows;
      if (rn < row_end) {
        tc::fence_proxy_async_smem();
        rg.arm(s, x + rn * xs, row_bytes);
      }
    }
    float mean = 0.f, rstd;
    if constexpr (RMS) {
      rstd = 1.0f / sqrtf(sum * inv_n + eps);
    } else {
      mean = sum * inv_n;
      float q = 0.f;
      if constexpr (sizeof(T) == 2) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
          if (lane + 32 * j < nvec) {
            uint4 &raw = *reinterpret_cast<uint4 *>(&xv[j].raw);
#pragma unroll
            for (int c = 0; c < 4; ++c) h2_centred_sumsq(word(raw, c), mean, acc[c]);
          }
        }
        q = (acc[0] + acc[1]) + (acc[2] + acc[3]);
      } else {
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
          if (lane + 32 * j < nvec) {
            float f[E];
            xv[j].unpack(f);
#pragma unroll
            for (int e = 0; e < E; ++e) {
              const float d = f[e] - mean;
              q = fmaf(d, d, q);
            }
          }
        }
      }
      q = warp_sum(q);
      rstd = 1.0f / sqrtf(q * inv_n + eps);
      if (lane == 0) {
        if (mean_out) mean_out[r] = mean;
        if (rstd_out) rstd_out[r] = rstd;
      }
    }
    T *yr = y + r * ys;
    uint32_t oslot = 0;
    if (out_slots) {
      // the bulk store that last used this output slot has finished reading it
      if (lane == 0) {
        if (out_slots >= 2) tc::bulk_wait_group_read<1>();
        else tc::bulk_wait_group_read<0>();
      }
      __syncwarp();
      oslot = rg.out0 + (uint32_t)((n_out % out_slots) * slot_bytes);
    }
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int vi = lane + 32 * j;
      if constexpr (sizeof(T) == 2) {
        if (vi < nvec) {
          uint4 &xr = *reinterpret_cast<uint4 *>(&xv[j].raw);
          uint4 &gr = *reinterpret_cast<uint4 *>(&wv[j].raw);
          uint4 o;
          if constexpr (RMS) {
#pragma unroll
            for (int c = 0; c < 4; ++c)
              word(o, c) = affine_f32 ? h2_norm_scale_f32(word(xr, c), rstd, word(gr, c))
                                      : h2_norm_scale(word(xr, c), rstd, word(gr, c));
          } else {
            uint4 br;
            if constexpr (B_SMEM) br = ring::lds128(rg.extra + (uint32_t)vi * 16u);
            else br = *reinterpret_cast<uint4 *>(&bv[j].raw);
#pragma unroll
            for (int c = 0; c < 4; ++c)
              word(o, c) = affine_f32 ? h2_norm_affine_f32(word(xr, c), mean, rstd, word(gr, c), word(br, c))
                                      : h2_norm_affine(word(xr, c), mean, rstd, word(gr, c), word(br, c));
          }
          if (out_slots) ring::sts128(oslot + (uint32_t)vi * 16u, o);
          else ring::store_out16(yr + (int64_t)vi * E, o, store_mode, rg.policy);
        }
      } else if (vi < nvec) {
        float f[E], wf[E], bf[E];
        xv[j].unpack(f);
        wv[j].unpack(wf);
        if constexpr (B_SMEM) {
          uint4 raw = ring::lds128(rg.extra + (uint32_t)vi * 16u);
          Vec16<T> bt;
          bt.raw = *reinterpret_cast<Raw *>(&raw);
          bt.unpack(bf);
        } else if constexpr (!RMS) {
          bv[j].unpack(bf);
        }
#pragma unroll
        for (int e = 0; e < E; ++e)
          f[e] = RMS ? (f[e] * rstd) * wf[e] : fmaf((f[e] - mean) * rstd, wf[e], bf[e]);
        Vec16<T> o;
        o.pack(f);
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
  if (out_slots && lane == 0) tc::bulk_wait_group_read<0>();  // shared memory outlives the last store's read
  if (*rg.abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);  // let copies in flight land before the CTA retires
    if (threadIdx.x == 0) atomicExch(&g_norm_status, (int)HEXB_ERR_TIMEOUT);
  }
}

template <typename T, int VPL, bool RMS>
static int launch_norm_ring(const T *x, T *y, const T *w, const T *b, float *mean, float *rstd,
                            int64_t rows, int nvec, int64_t xs, int64_t ys, float inv_n, float eps,
                            int sm_count, cudaStream_t st) {
  // norm_bulk_store = 1: rows leave as one bulk store each from a per-warp output slot in shared memory.  A single
  // short burst measured that slightly faster (44.3 -> 43.7 us on [16384 x 4096] fp16); under back-to-back replays
  // (>= 50 ms) the lanes' own streaming stores win clearly (50.4 -> 44.2 us, RMSNorm [8192 x 2048] 14.3 -> 12.9 us),
  // so they are the default.
  const int out_slots = option(OPT_norm_bulk_store, 0) ? 1 : 0;
  const ring::Layout lay = ring::make_layout(nvec * 16, 0, out_slots);
  auto kern = norm_ring_kernel<T, VPL, RMS>;
  static PerDeviceOnce attr_done;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done.is_done(dev)) {
    HEXB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 212 * 1024));
    attr_done.mark(dev);
  }
  const int64_t groups = (rows + ring::WARPS - 1) / ring::WARPS;
  const int grid = (int)(groups < sm_count ? groups : sm_count);
  launch_pdl(kern, dim3(grid), dim3(ring::THREADS), (size_t)lay.smem_bytes, st, x, y, w, b, mean, rstd, rows, nvec, xs, ys,
             inv_n, eps, lay.slots, lay.slot_bytes, (int)option(OPT_ring_map, 0), out_slots,
             (int)option(OPT_norm_affine_f32, 1));
  return check_launch(RMS ? "rms_norm_ring" : "layer_norm_ring");
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
  const int64_t row_bytes = cols * (int64_t)sizeof(T);
  if (vec_ok && option(OPT_norm_ring, 1) && row_bytes >= 512 && row_bytes <= ring::MAX_ROW_BYTES &&
      rows * row_bytes >= (4ll << 20)) {
    const int nvec = (int)(cols / E);
    const int need = (nvec + 31) / 32;
#define RING(VPL)                                                                                  \
  return launch_norm_ring<T, VPL, RMS>(x, y, w, b, mean, rstd, rows, nvec, xs, ys, inv_n, eps,      \
                                       di.sm_count, st)
    if (need <= 1) RING(1);
    if (need <= 2) RING(2);
    if (need <= 4) RING(4);
    if (need <= 8) RING(8);
    RING(16);
#undef RING
  }
  int tpr = 0, vpt = 0;
  const int vpt_max = option(OPT_norm_vpt_max, sizeof(T) == 2 ? 4 : 8);
  if (vec_ok && !option(OPT_norm_force_stream, 0) && choose_row_shape(cols / E, vpt_max, &tpr, &vpt)) {
    const int nvec = (int)(cols / E);
    const int waves = option(OPT_norm_ctas_per_sm, 8);
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

int norm_device_status_fetch_and_clear(int *out) {
  int v = 0, zero = 0;
  HEXB_CUDA_OK(cudaMemcpyFromSymbol(&v, g_norm_status, sizeof(int)));
  if (v) HEXB_CUDA_OK(cudaMemcpyToSymbol(g_norm_status, &zero, sizeof(int)));
  *out = v;
  return HEXB_OK;
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
