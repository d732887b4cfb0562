// Shared host/device helpers for libhexb200 (sm_100a only).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/hexb.h"

namespace hexb {

constexpr int kNumSMsB200 = 148;

// Thread-local text of the last CUDA error seen inside the library.
void set_cuda_error(cudaError_t e, const char *where);
int check_launch(const char *where);  // cudaGetLastError -> status

// Option store behind hexb_set_option / hexb_get_option: one atomic word per option, indexed by an
// enum, so that a launch reads its switches without a lock, a string or an allocation.
// X(name): selectable kernel variants of the shipped library.
#define HEXB_OPTIONS(X)                                                                              \
  X(softmax_vpt_max) X(softmax_force_stream) X(softmax_ring) X(softmax_bulk_store) X(norm_ring)      \
  X(norm_bulk_store) X(ring_bytes_per_warp) X(ring_map) X(norm_vpt_max) X(norm_force_stream)         \
  X(norm_ctas_per_sm) X(norm_affine_f32) X(gemm_bn) X(gemm_tail_split) X(gemm_pair) X(gemm_pair_min_tiles) X(gemm_epi_warps) \
  X(gemm_tma_store) X(gemm_group_m) X(gemm_force_simt) X(attn_force_simt) X(attn_tiles_per_cta) X(attn_kernel)       \
  X(attn_mask_tma) X(attn_f32_tensor) X(scan_force_scalar) X(scan_segments) X(scan_kv) X(decoder_fused_swiglu)          \
  X(host_chunks) X(host_taper) X(pdl) X(tmap_cache)
// Descriptor-field overrides that can mis-describe an operand: compiled in only
// with -DHEXB_DEV, absent from the shipped library's option table.
#define HEXB_DEV_OPTIONS(X) X(gemm_b_lbo) X(gemm_b_sbo) X(attn_v_lbo) X(attn_v_sbo) X(attn_ablate)
enum Opt : int {
#define HEXB_X(n) OPT_##n,
  HEXB_OPTIONS(HEXB_X) HEXB_DEV_OPTIONS(HEXB_X)
#undef HEXB_X
      OPT_COUNT
};
int option(Opt key, int dflt);  // the value set through hexb_set_option, else dflt
#ifdef HEXB_DEV
#define HEXB_DEV_OPTION(key, dflt) ::hexb::option(key, dflt)
#else
#define HEXB_DEV_OPTION(key, dflt) (dflt)
#endif

// One-time set-up per device ordinal (function attributes).  The set-up calls are idempotent, so two
// threads that both find the flag clear may both run them; the flag itself is never torn.
struct PerDeviceOnce {
  std::atomic<bool> done[64];
  bool is_done(int dev) const { return done[dev & 63].load(std::memory_order_acquire); }
  void mark(int dev) { done[dev & 63].store(true, std::memory_order_release); }
};

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

struct DeviceInfo {
  int device = -1;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  size_t smem_optin = 0;
  size_t l2_bytes = 0;
};
// Properties of the current device (cached per device id); status != HEXB_OK if there is none.
int current_device(DeviceInfo *out);

// Stream-ordered scratch for the few kernels that need a small workspace (segment totals of a scan,
// partial sums): allocated from a memory pool the library owns per device, whose release threshold
// keeps freed blocks cached, so a call costs no device allocation after the first and the
// application's own pools are not touched.
int scratch_alloc(void **ptr, size_t bytes, cudaStream_t st);
int scratch_free(void *ptr, cudaStream_t st);

#define HEXB_CUDA_OK(expr)                                   \
  do {                                                       \
    cudaError_t _e = (expr);                                 \
    if (_e != cudaSuccess) {                                 \
      ::hexb::set_cuda_error(_e, #expr);                     \
      return HEXB_ERR_CUDA;                                  \
    }                                                        \
  } while (0)

// ---------------------------------------------------------------- device helpers
#ifdef __CUDACC__
// Programmatic dependent launch: a kernel launched through launch_pdl may become resident while the
// kernel before it in the stream is still draining.  It must call pdl_wait() before its first access
// to global memory (everything before -- index arithmetic, shared-memory and barrier set-up -- overlaps
// the predecessor's tail), and pdl_launch_dependents() lets its own successor do the same.  Both are
// no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = option(OPT_pdl, 1) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// 16-byte vector of T with fp32 unpack/pack.
template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  float4 raw;
  __device__ __forceinline__ void unpack(float (&f)[4]) const {
    f[0] = raw.x; f[1] = raw.y; f[2] = raw.z; f[3] = raw.w;
  }
  __device__ __forceinline__ void pack(const float (&f)[4]) { raw = make_float4(f[0], f[1], f[2], f[3]); }
};
template <>
struct Vec16<__half> {
  static constexpr int N = 8;
  uint4 raw;
  // fp16 -> fp32 by the mixed-precision subtract of +0 (sm_100: sub.rn.f32.f16, exact for every input, -0
  // included): it runs on the FMA pipe at 128 lanes per clock and SM, where cvt.f32.f16 shares the
  // 16-lane unit of the transcendentals and made the fp16 forms of the streaming kernels conversion-bound.
  static __device__ __forceinline__ void widen2(uint32_t w, float &lo, float &hi) {
    asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tsub.rn.f32.f16 %0, l, 0f00000000;\n\tsub.rn.f32.f16 %1, h, 0f00000000;\n\t}"
        : "=f"(lo), "=f"(hi)
        : "r"(w));
  }
  __device__ __forceinline__ void unpack(float (&f)[8]) const {
    widen2(raw.x, f[0], f[1]);
    widen2(raw.y, f[2], f[3]);
    widen2(raw.z, f[4], f[5]);
    widen2(raw.w, f[6], f[7]);
  }
  __device__ __forceinline__ void pack(const float (&f)[8]) {
    __half2 *h = reinterpret_cast<__half2 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
  }
};

// tanh by the special-function unit's own instruction: one operation per value, max relative error 2^-11
// (half an fp16 ulp), against two (ex2 + rcp) for the exponential form.  Used where the result is rounded
// to fp16 anyway.
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) {
  float f;
  asm("sub.rn.f32.f16 %0, %1, 0f00000000;" : "=f"(f) : "h"(__half_as_ushort(v)));
  return f;
}
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// Streaming 16-byte global accesses (read once / write once data).
__device__ __forceinline__ uint4 ld_stream16(const void *p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream16(void *p, uint4 v) {
  asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
// Makes the compiler forget what it knows about a packed 16-byte register vector, so that a later
// unpack is re-materialised from the packed form instead of keeping every unpacked float alive.
__device__ __forceinline__ void opaque(uint4 &v) {
  asm volatile("" : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w));
}
__device__ __forceinline__ void opaque(float4 &v) {
  asm volatile("" : "+f"(v.x), "+f"(v.y), "+f"(v.z), "+f"(v.w));
}

template <typename R>
__device__ __forceinline__ R ld_stream_as(const void *p) {
  uint4 v = ld_stream16(p);
  return *reinterpret_cast<R *>(&v);
}
template <typename R>
__device__ __forceinline__ void st_stream_as(void *p, R r) {
  st_stream16(p, *reinterpret_cast<uint4 *>(&r));
}
#endif  // __CUDACC__

}  // namespace hexb
