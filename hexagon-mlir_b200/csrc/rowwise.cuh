// Row-group machinery shared by the softmax / LayerNorm / RMSNorm kernels.
//
// A row is owned by TPR threads (a power of two, 32..1024); each thread keeps VPT 16-byte vectors
// of the row in registers, so the row is read from HBM once and written once.  Thread t of the
// group owns vectors t, t+TPR, t+2*TPR, ... so that every warp-wide access is one contiguous
// 512-byte segment.  A CTA of THREADS threads holds THREADS/TPR rows and walks the matrix with a
// grid stride.
#pragma once
#include "common.cuh"

namespace hexb {

struct SumOp {
  static __device__ __forceinline__ float apply(float a, float b) { return a + b; }
};
struct MaxOp {
  static __device__ __forceinline__ float apply(float a, float b) { return fmaxf(a, b); }
};

// All-reduce of `v` over the TPR threads that own one row.  `red` is a shared array of
// (THREADS/32) floats per slot; the caller rotates `slot` (0..2) between consecutive reductions
// so that a fast warp never overwrites a value a slow warp still has to read.
template <typename Op, int TPR, int THREADS>
__device__ __forceinline__ float group_allreduce(float v, float *red, int slot) {
  constexpr int W = TPR < 32 ? TPR : 32;
#pragma unroll
  for (int o = W / 2; o > 0; o >>= 1) v = Op::apply(v, __shfl_xor_sync(0xffffffffu, v, o));
  if constexpr (TPR > 32) {
    constexpr int WPR = TPR / 32;          // warps per row
    constexpr int NW = THREADS / 32;       // warps per CTA
    const int warp = threadIdx.x >> 5;
    float *s = red + slot * NW;
    if ((threadIdx.x & 31) == 0) s[warp] = v;
    __syncthreads();
    const int first = (warp / WPR) * WPR;
    float r = s[first];
#pragma unroll
    for (int i = 1; i < WPR; ++i) r = Op::apply(r, s[first + i]);
    v = r;
  }
  return v;
}

// Picks (TPR, VPT) for a row of `nvec` 16-byte vectors: the smallest group whose per-thread
// vector count (rounded up to a power of two) does not exceed vpt_max.  Returns false if the row
// does not fit 1024 threads x vpt_max vectors.
inline bool choose_row_shape(int64_t nvec, int vpt_max, int *tpr, int *vpt) {
  for (int t = 32; t <= 1024; t <<= 1) {
    int64_t need = (nvec + t - 1) / t;
    int v = 1;
    while (v < need) v <<= 1;
    if (v <= vpt_max) {
      *tpr = t;
      *vpt = v;
      return true;
    }
  }
  return false;
}

// Expands to a switch over the (TPR, VPT) pairs the library instantiates.
#define HEXB_ROW_SHAPE_SWITCH(TPR_, VPT_, LAUNCH)                         \
  switch ((TPR_) * 16 + (VPT_)) {                                         \
    case 32 * 16 + 1:   { LAUNCH(32, 1); break; }                         \
    case 32 * 16 + 2:   { LAUNCH(32, 2); break; }                         \
    case 32 * 16 + 4:   { LAUNCH(32, 4); break; }                         \
    case 32 * 16 + 8:   { LAUNCH(32, 8); break; }                         \
    case 64 * 16 + 1:   { LAUNCH(64, 1); break; }                         \
    case 64 * 16 + 2:   { LAUNCH(64, 2); break; }                         \
    case 64 * 16 + 4:   { LAUNCH(64, 4); break; }                         \
    case 64 * 16 + 8:   { LAUNCH(64, 8); break; }                         \
    case 128 * 16 + 1:  { LAUNCH(128, 1); break; }                        \
    case 128 * 16 + 2:  { LAUNCH(128, 2); break; }                        \
    case 128 * 16 + 4:  { LAUNCH(128, 4); break; }                        \
    case 128 * 16 + 8:  { LAUNCH(128, 8); break; }                        \
    case 256 * 16 + 1:  { LAUNCH(256, 1); break; }                        \
    case 256 * 16 + 2:  { LAUNCH(256, 2); break; }                        \
    case 256 * 16 + 4:  { LAUNCH(256, 4); break; }                        \
    case 256 * 16 + 8:  { LAUNCH(256, 8); break; }                        \
    case 512 * 16 + 1:  { LAUNCH(512, 1); break; }                        \
    case 512 * 16 + 2:  { LAUNCH(512, 2); break; }                        \
    case 512 * 16 + 4:  { LAUNCH(512, 4); break; }                        \
    case 512 * 16 + 8:  { LAUNCH(512, 8); break; }                        \
    case 1024 * 16 + 1: { LAUNCH(1024, 1); break; }                       \
    case 1024 * 16 + 2: { LAUNCH(1024, 2); break; }                       \
    case 1024 * 16 + 4: { LAUNCH(1024, 4); break; }                       \
    case 1024 * 16 + 8: { LAUNCH(1024, 8); break; }                       \
    default: return HEXB_ERR_UNSUPPORTED;                                 \
  }

template <int TPR>
struct CtaThreads {
  static constexpr int value = TPR < 256 ? 256 : TPR;
};

}  // namespace hexb
