// Device helpers shared by the flash-attention kernels (attention.cu, attention_pingpong.cu).
#pragma once
#include "tc_sm100.cuh"

namespace hexb {
namespace attn {

constexpr float kRescaleThreshold = 8.0f;  // log2 units: O and l are rescaled only when a row maximum grows by more

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x on the FMA pipe: x = n + f with n = round(x) taken from the mantissa of x + 1.5*2^23,
// 2^f by a degree-3 polynomial on [-0.5, 0.5] (max relative error 7.5e-5, below the fp16 rounding
// of P), exponent patched in with an integer add.  Kept for reference, not called: routing one exponential
// in 4 through it measured 614 -> 649 us in the 128-key kernel ([4,32,4096,128] causal), and one in
// 32 / 16 / 8 in the default kernel 563 / 568 / 578 us against 563.  The special-function unit is busy
// half of the time only, so the extra FMA-pipe instructions cost more than they free.
__device__ __forceinline__ float ex2_poly(float x) {
  x = fmaxf(x, -126.0f);
  const float t = x + 12582912.0f;
  const float f = x - (t - 12582912.0f);
  float r = fmaf(0.05517161265015602f, f, 0.2426111251115799f);
  r = fmaf(r, f, 0.6932609677314758f);
  r = fmaf(r, f, 0.9999280571937561f);
  return __int_as_float(__float_as_int(r) + (__float_as_int(t) << 23));
}

// Two fp32 lanes per instruction (sm_100 packed arithmetic): halves the issue slots of the scale-and-
// shift and of the row-sum in the softmax loop, which is bound by instruction issue.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(reinterpret_cast<unsigned long long &>(d))
      : "l"(reinterpret_cast<unsigned long long &>(a)), "l"(reinterpret_cast<unsigned long long &>(b)),
        "l"(reinterpret_cast<unsigned long long &>(c)));
  return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  float2 d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<unsigned long long &>(d))
      : "l"(reinterpret_cast<unsigned long long &>(a)), "l"(reinterpret_cast<unsigned long long &>(b)));
  return d;
}

// {lo, hi} -> packed fp16 pair (lo in bits 0..15)
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}


// (s0, s1) <- (s0, s1) * scale + the two fp16 values packed in w, in fp32: the mixed-precision add widens the
// fp16 operand exactly, so no conversion instruction is needed
__device__ __forceinline__ void add_mask_h2(uint32_t w, float scale, uint32_t &s0, uint32_t &s1) {
  float2 t = fma2(make_float2(__uint_as_float(s0), __uint_as_float(s1)), make_float2(scale, scale), make_float2(0.f, 0.f));
  asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tadd.rn.f32.f16 %0, lo, %0;\n\tadd.rn.f32.f16 %1, hi, %1;\n\t}"
      : "+f"(t.x), "+f"(t.y)
      : "r"(w));
  s0 = __float_as_uint(t.x);
  s1 = __float_as_uint(t.y);
}


// Phase timing for development builds (-DHEXB_ATTN_PROFILE): clock64 stamps around the phases of
// one softmax warp and of the MMA thread of the tensor-core kernels, summed into a device buffer that
// hexb_debug_set_attn_profile() registers.  Compiled out otherwise.
#ifdef HEXB_ATTN_PROFILE
#define HEXB_PROF_DECL(n) long long prof_t[n] = {}; long long prof_last = clock64();
#define HEXB_PROF(i) { const long long now_ = clock64(); prof_t[i] += now_ - prof_last; prof_last = now_; }
#define HEXB_PROF_FLUSH(base, n) if (p.prof) { for (int i_ = 0; i_ < n; ++i_) atomicAdd(p.prof + base + i_, (unsigned long long)prof_t[i_]); }
#else
#define HEXB_PROF_DECL(n)
#define HEXB_PROF(i)
#define HEXB_PROF_FLUSH(base, n)
#endif

// Optional parts of a forward call: key length, output type, additive mask.
struct Extra {
  int64_t n_kv;
  int out_f32;
  const void *mask;
  int mask_f32;
  int64_t sm[3];
};

}  // namespace attn

// Two query tiles per CTA taking turns on the tensor pipe (attention_pingpong.cu).  Plain calls only
// (no additive mask, N_KV == N_CTX); returns HEXB_ERR_UNSUPPORTED for anything else.
int attn_pingpong_supported(int64_t Z, int64_t H, int64_t N, int64_t D, int causal, int sm_count);
int attn_pingpong_launch(const __half *Q, const __half *K, const __half *V, void *O, int64_t Z, int64_t H, int64_t N,
                         int64_t D, const int64_t *strides, float scale_log2, int causal, int out_f32, int threads_per_row,
                         cudaStream_t st);
int attn_pingpong_status_fetch_and_clear(int *out);

// One query tile per persistent CTA, 128-key blocks, two score buffers, threads_per_row (2 or 4) softmax
// threads per query row (attention_wide.cu).  Plain calls only.
int attn_wide_launch(const __half *Q, const __half *K, const __half *V, void *O, int64_t Z, int64_t H, int64_t N, int64_t D,
                     const int64_t *strides, float scale_log2, int causal, int out_f32, int threads_per_row, cudaStream_t st);
int attn_wide_status_fetch_and_clear(int *out);

// fp32 tensors on the tensor cores (kind::tf32, attention_tf32.cu): no mask; head size 64 or 128.
int attn_tf32_supported(const void *Q, const void *K, const void *V, int64_t D, const int64_t *strides);
int attn_tf32_launch(const float *Q, const float *K, const float *V, float *O, int64_t Z, int64_t H, int64_t N, int64_t N_KV,
                     int64_t D, const int64_t *strides, float scale_log2, int causal, cudaStream_t st);
int attn_tf32_status_fetch_and_clear(int *out);
#ifdef HEXB_ATTN_PROFILE
unsigned long long *attn_profile_buffer();  // the buffer hexb_debug_set_attn_profile registered
#endif

}  // namespace hexb
