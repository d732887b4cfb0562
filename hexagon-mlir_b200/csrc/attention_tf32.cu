// Flash-attention forward for fp32 tensors on the tensor cores: tcgen05.mma kind::tf32.
//
// fp32 is the dtype of the reference's own Triton test (test/python/triton/test_flash_attention.py:20-27,
// 176-213: [1, 1, 1024, 64] fp32, scale 0.5).  The CUDA-core kernel of attention.cu follows
// _attn_fwd_inner step by step in fp32 and is exact to round-off, but runs at about 1 TFLOP/s.  This kernel
// is the 64-key two-score-buffer design of attention.cu with fp32 tiles: Q, K, V arrive by TMA as fp32
// (128-byte swizzle = 32 floats per row chunk), the tensor cores read them as tf32 (10-bit mantissa,
// fp32 accumulation, K = 8 per instruction), the scores, the online softmax, P and O stay fp32; P is rounded
// to tf32 (to nearest) by the softmax warps before it is stored and summed, so that the row sum matches
// what P.V multiplies.  kind::tf32 takes K-major operands only (a B operand described as MN-major, the way the
// fp16 kernels read V as stored, silently multiplies by zero on B200), so V is transposed once per call into
// scratch memory of the library's stream-ordered pool ([Z, H, D, N_KV], one pass over V at HBM speed) and its
// tiles arrive as D rows x 64 keys.  The tensor cores TRUNCATE fp32 operands to tf32, which shrinks every
// score by about 2^-10 of its size -- a bias the exponential turns into a few 1e-3 of relative error; Q and K are
// therefore copied into the same scratch block rounded to nearest tf32 (V is rounded while it is transposed),
// two more passes at HBM speed that bring the error to a few 1e-4.  Results differ from the fp32 reference by the tf32 rounding of the operands
// (relative error of the output a few 1e-4), inside the benchmark's 1e-3 bar for fp32 kernels but not
// inside torch.allclose's defaults -- the launcher therefore uses this kernel for large problems only
// and keeps the exact CUDA-core kernel for small ones (the reference's test shape among them).
//
//   TMEM (256 columns)  S0 [0,64)  S1 [64,128)  O [128,128+D);  P_b overwrites S_b in place (32-bit elements)
//   warp 0  TMA (Q once per tile; K_j, V^T_j double-buffered)     warp 1  MMA     warps 2-5  softmax / epilogue
// D = 64: two CTAs per SM; D = 128: one (192 KiB of tiles).  No additive mask; separate key length supported.
// Every mbarrier wait is bounded; no load uses cluster multicast.
#include "attn_common.cuh"

namespace hexb {

static __device__ int g_attn32_status = 0;

namespace attn32 {

using namespace attn;

constexpr int BLOCK_M = 128;
constexpr int BN = 64;
constexpr int THREADS = 192;

template <int HD>
struct Cfg {
  static constexpr int CHUNKS = HD / 32;              // 32-float (128-byte) swizzle chunks
  static constexpr int Q_BYTES = 128 * HD * 4;
  static constexpr int Q_CHUNK = 128 * 128;           // 128 rows x 128 bytes
  static constexpr int KV_BYTES = BN * HD * 4;
  static constexpr int KV_CHUNK = BN * 128;           // K tile: 64 rows x 128 bytes per 32-float chunk
  static constexpr int VT_CHUNK = HD * 128;           // V^T tile: HD rows x 128 bytes per 32-key chunk
  static constexpr int NBAR = 18;
  static constexpr int SMEM_BYTES = Q_BYTES + 4 * KV_BYTES + NBAR * 8 + 16 + 1024;
  static constexpr int TMEM_COLS = 256;
  static constexpr int O_COL = 2 * BN;
  static constexpr int CTAS_PER_SM = SMEM_BYTES <= 113 * 1024 ? 2 : 1;
};

struct Params {
  float *out;
  int64_t so_z, so_h, so_n;
  int H, N_CTX, N_KV;
  int out_vec_ok;
  int num_q_tiles, tiles_per_cta, ctas_per_bh;
  float scale_log2;
  int causal;
};

__device__ __forceinline__ float round_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

template <int HD>
__global__ void __launch_bounds__(THREADS, Cfg<HD>::CTAS_PER_SM)
attn_fwd_tf32_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const Params p) {
  using cfg = Cfg<HD>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw_addr = tc::smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
  uint8_t *smem = smem_raw + pad;
  const uint32_t smem_addr = raw_addr + pad;
  const uint32_t sQ = smem_addr;
  const uint32_t sK0 = sQ + cfg::Q_BYTES, sV0 = sK0 + 2 * cfg::KV_BYTES;
  const uint32_t bar0 = sV0 + 2 * cfg::KV_BYTES;
  const uint32_t q_full = bar0, q_empty = bar0 + 8, o_full = bar0 + 16, o_empty = bar0 + 24, pv_done = bar0 + 32;
  auto k_full = [&](uint32_t b) { return bar0 + 40 + 8 * b; };
  auto k_empty = [&](uint32_t b) { return bar0 + 56 + 8 * b; };
  auto v_full = [&](uint32_t b) { return bar0 + 72 + 8 * b; };
  auto v_empty = [&](uint32_t b) { return bar0 + 88 + 8 * b; };
  auto s_full = [&](uint32_t b) { return bar0 + 104 + 8 * b; };
  auto p_full = [&](uint32_t b) { return bar0 + 120 + 8 * b; };   // ends at bar0 + 136 = 17 barriers
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + cfg::Q_BYTES + 4 * cfg::KV_BYTES + 144);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int bh = blockIdx.x / p.ctas_per_bh;
  const int q_rank = blockIdx.x - bh * p.ctas_per_bh;
  const int z = bh / p.H, h = bh - z * p.H;
  const int kv_blocks = (p.N_KV + BN - 1) / BN;
  auto tile_of = [&](int t) {
    if (p.causal && p.tiles_per_cta == 2) return t == 0 ? p.num_q_tiles - 1 - q_rank : q_rank;
    return q_rank * p.tiles_per_cta + t;
  };
  auto nkv_of = [&](int q_tile) {
    const int need = (BLOCK_M / BN) * (q_tile + 1);   // causal: keys 0 .. m0 + 127
    return (p.causal && need < kv_blocks) ? need : kv_blocks;
  };

  if (threadIdx.x == 0) {
    tc::mbar_init(q_full, 1);
    tc::mbar_init(q_empty, 1);
    tc::mbar_init(o_full, 1);
    tc::mbar_init(o_empty, 4);
    tc::mbar_init(pv_done, 1);
    for (uint32_t b = 0; b < 2; ++b) {
      tc::mbar_init(k_full(b), 1);
      tc::mbar_init(k_empty(b), 1);
      tc::mbar_init(v_full(b), 1);
      tc::mbar_init(v_empty(b), 1);
      tc::mbar_init(s_full(b), 1);
      tc::mbar_init(p_full(b), 4);
    }
    *abort_flag = 0;
    tc::fence_barrier_init();
    tc::prefetch_tensormap(&tmQ);
    tc::prefetch_tensormap(&tmK);
    tc::prefetch_tensormap(&tmV);
  }
  if (warp == 1) {
    tc::tmem_alloc(tc::smem_u32(tmem_slot), cfg::TMEM_COLS);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();  // set-up done; global memory is touched from here on
  const uint32_t tO = tmem_base + cfg::O_COL;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = 0; t < p.tiles_per_cta && ok; ++t) {
        const int q_tile = tile_of(t);
        const int n_kv = nkv_of(q_tile);
        if (t > 0 && !tc::mbar_wait(q_empty, (uint32_t)(t - 1) & 1u, abort_flag)) break;
        tc::mbar_arrive_expect_tx(q_full, cfg::Q_BYTES);
#pragma unroll
        for (int c = 0; c < cfg::CHUNKS; ++c)
          tc::tma_load_4d(sQ + c * cfg::Q_CHUNK, &tmQ, c * 32, q_tile * BLOCK_M, h, z, q_full);
        for (int j = 0; j < n_kv; ++j, ++it) {
          const uint32_t b = it & 1u, ph = (it >> 1) & 1u;
          if (!tc::mbar_wait(k_empty(b), ph ^ 1u, abort_flag)) { ok = false; break; }
          tc::mbar_arrive_expect_tx(k_full(b), cfg::KV_BYTES);
#pragma unroll
          for (int c = 0; c < cfg::CHUNKS; ++c)
            tc::tma_load_4d(sK0 + b * cfg::KV_BYTES + c * cfg::KV_CHUNK, &tmK, c * 32, j * BN, h, z, k_full(b));
          if (!tc::mbar_wait(v_empty(b), ph ^ 1u, abort_flag)) { ok = false; break; }
          tc::mbar_arrive_expect_tx(v_full(b), cfg::KV_BYTES);
#pragma unroll
          for (int c = 0; c < BN / 32; ++c)   // V^T: 32 keys (128 bytes) x HD rows per chunk
            tc::tma_load_4d(sV0 + b * cfg::KV_BYTES + c * cfg::VT_CHUNK, &tmV, j * BN + c * 32, 0, h, z, v_full(b));
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = tc::make_idesc_tf32_f32(BLOCK_M, BN, 0, 0);
      constexpr uint32_t idesc_pv = tc::make_idesc_tf32_f32(BLOCK_M, HD, 0, 0);   // both operands K-major
      bool ok = true;
      // S_{blk} = Q . K_{blk}^T into score buffer blk % 2: HD / 8 steps of 8 floats (32 bytes inside a 128-byte chunk)
      auto issue_qk = [&](uint32_t blk, bool last_of_tile) {
        const uint32_t b = blk & 1u, ph = (blk >> 1) & 1u;
        if (!tc::mbar_wait(k_full(b), ph, abort_flag)) { ok = false; return; }
        tc::tc_fence_after();
        const uint32_t sK = sK0 + b * cfg::KV_BYTES;
#pragma unroll
        for (int k = 0; k < HD / 8; ++k) {
          const uint32_t qoff = (uint32_t)((k >> 2) * cfg::Q_CHUNK + (k & 3) * 32);
          const uint32_t koff = (uint32_t)((k >> 2) * cfg::KV_CHUNK + (k & 3) * 32);
          tc::mma_tf32_ss(tmem_base + b * BN, tc::make_smem_desc_sw128(sQ + qoff, 16, 1024),
                          tc::make_smem_desc_sw128(sK + koff, 16, 1024), idesc_qk, k != 0 ? 1u : 0u);
        }
        tc::mma_commit(s_full(b));
        tc::mma_commit(k_empty(b));
        if (last_of_tile) tc::mma_commit(q_empty);
      };
      uint32_t it = 0;
      for (int t = 0; t < p.tiles_per_cta && ok; ++t) {
        const int n_kv = nkv_of(tile_of(t));
        if (!tc::mbar_wait(q_full, (uint32_t)t & 1u, abort_flag)) break;
        issue_qk(it, n_kv == 1);
        for (int j = 0; j < n_kv && ok; ++j, ++it) {
          if (j + 1 < n_kv) issue_qk(it + 1, j + 2 == n_kv);  // run one block ahead of the softmax
          if (!ok) break;
          const uint32_t b = it & 1u, ph = (it >> 1) & 1u;
          if (!tc::mbar_wait(p_full(b), ph, abort_flag)) { ok = false; break; }
          if (!tc::mbar_wait(v_full(b), ph, abort_flag)) { ok = false; break; }
          // the first product of a later tile overwrites O: the previous epilogue must have read it
          if (j == 0 && t > 0 && !tc::mbar_wait(o_empty, (uint32_t)(t - 1) & 1u, abort_flag)) { ok = false; break; }
          tc::tc_fence_after();
          const uint32_t sV = sV0 + b * cfg::KV_BYTES;
#pragma unroll
          for (int k = 0; k < BN / 8; ++k) {
            // A = P rows from TMEM (8 tf32 = 8 columns per step); B = V^T, K-major: 8 keys = 32 bytes inside a chunk
            const uint32_t voff = (uint32_t)((k >> 2) * cfg::VT_CHUNK + (k & 3) * 32);
            tc::mma_tf32_ts(tO, tmem_base + b * BN + (uint32_t)(k * 8), tc::make_smem_desc_sw128(sV + voff, 16, 1024),
                            idesc_pv, (j | k) != 0 ? 1u : 0u);
          }
          tc::mma_commit(v_empty(b));
          tc::mma_commit(pv_done);
          if (j == n_kv - 1) tc::mma_commit(o_full);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / correction / epilogue
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    uint32_t it = 0;
    bool ok = true;
    for (int t = 0; t < p.tiles_per_cta && ok; ++t) {
      const int q_tile = tile_of(t);
      const int n_kv = nkv_of(q_tile);
      const int m0 = q_tile * BLOCK_M;
      const int qi = m0 + r;
      float m_ref = -INFINITY, l = 0.f;
      for (int j = 0; j < n_kv; ++j, ++it) {
        const uint32_t b = it & 1u, ph = (it >> 1) & 1u;
        if (!tc::mbar_wait(s_full(b), ph, abort_flag)) { ok = false; break; }
        tc::tc_fence_after();
        const uint32_t tS = tmem_base + b * BN;
        const int kv0 = j * BN;
        const bool need_mask = (p.causal && kv0 + BN - 1 > m0) || (kv0 + BN > p.N_KV);
        uint32_t sv[BN];
#pragma unroll
        for (int c = 0; c < BN / 32; ++c)
          tc::tmem_ld_32x32(tS + lane_off + (uint32_t)(c * 32), reinterpret_cast<uint32_t(&)[32]>(sv[c * 32]));
        tc::tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int e = 0; e < BN; ++e) {
            const int kv = kv0 + e;
            if ((p.causal && kv > qi) || kv >= p.N_KV) sv[e] = 0xff800000u;  // -inf: exp2 gives 0
          }
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int e = 0; e < BN; e += 8) {
#pragma unroll
          for (int u = 0; u < 4; ++u)
            mx4[u] = max3(mx4[u], __uint_as_float(sv[e + 2 * u]), __uint_as_float(sv[e + 2 * u + 1]));
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
        const float m_new = fmaxf(m_ref, mx);
        if (j == 0) {
          m_ref = m_new;
        } else if (__any_sync(0xffffffffu, m_new - m_ref > kRescaleThreshold)) {
          // O must be quiescent: P_{it-1}.V_{it-1} is the it-th completion of pv_done
          if (!tc::mbar_wait(pv_done, (it - 1u) & 1u, abort_flag)) { ok = false; break; }
          tc::tc_fence_after();
          const float alpha = ex2_approx(m_ref - m_new);
          m_ref = m_new;
          l *= alpha;
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tc::tmem_ld_32x32(tO + lane_off + (uint32_t)(c * 32), o);
            tc::tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tc::tmem_st_32x32(tO + lane_off + (uint32_t)(c * 32), o);
          }
          tc::tmem_st_wait();
        }
        // P = exp2(S*scale - m_ref), rounded to tf32 (what the tensor cores multiply), over S in place
        const float neg_m = -m_ref;
        float l0 = 0.f, l1 = 0.f;
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const float p0 = round_tf32(ex2_approx(fmaf(__uint_as_float(sv[c * 32 + e]), p.scale_log2, neg_m)));
            const float p1 = round_tf32(ex2_approx(fmaf(__uint_as_float(sv[c * 32 + e + 1]), p.scale_log2, neg_m)));
            l0 += p0;
            l1 += p1;
            sv[c * 32 + e] = __float_as_uint(p0);
            sv[c * 32 + e + 1] = __float_as_uint(p1);
          }
          tc::tmem_st_32x32(tS + lane_off + (uint32_t)(c * 32), reinterpret_cast<uint32_t(&)[32]>(sv[c * 32]));
        }
        l += l0 + l1;
        tc::tmem_st_wait();
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(p_full(b));
      }
      if (!ok || !tc::mbar_wait(o_full, (uint32_t)t & 1u, abort_flag)) { ok = false; break; }
      tc::tc_fence_after();
      const float inv = 1.0f / l;
      float *orow = p.out + (int64_t)z * p.so_z + (int64_t)h * p.so_h + (int64_t)qi * p.so_n;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        tc::tmem_ld_32x32(tO + lane_off + (uint32_t)(c * 32), o);
        tc::tmem_ld_wait();
        if (c == HD / 32 - 1) {  // O is in registers: the next tile's first product may overwrite it
          tc::tc_fence_before();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(o_empty);
        }
        if (qi < p.N_CTX) {
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            float4 f = make_float4(__uint_as_float(o[g * 4]) * inv, __uint_as_float(o[g * 4 + 1]) * inv,
                                   __uint_as_float(o[g * 4 + 2]) * inv, __uint_as_float(o[g * 4 + 3]) * inv);
            if (p.out_vec_ok) {
              *reinterpret_cast<float4 *>(orow + c * 32 + g * 4) = f;
            } else {
              orow[c * 32 + g * 4] = f.x; orow[c * 32 + g * 4 + 1] = f.y;
              orow[c * 32 + g * 4 + 2] = f.z; orow[c * 32 + g * 4 + 3] = f.w;
            }
          }
        }
      }
    }
  }

  // ------------------------------------------------------------ teardown
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);  // let copies in flight land before the CTA retires
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, cfg::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&g_attn32_status, (int)HEXB_ERR_TIMEOUT);
}

// V [Z, H, N_KV, D] (strides in elements, D contiguous) -> Vt [Z*H, D, NP] (NP >= N_KV, rows 16-byte aligned).
// x [Z, H, N, D] (strides in elements, D contiguous, D % 4 == 0) -> dense copy rounded to nearest tf32.
__global__ void __launch_bounds__(256) round_copy_kernel(const float *__restrict__ x, float *__restrict__ y, int H, int N, int D,
                                                         int64_t sz, int64_t sh, int64_t sn, int64_t total_vec) {
  const int dv = D / 4;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_vec; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % dv);
    const int64_t row = i / dv;
    const int n = (int)(row % N);
    const int64_t bh = row / N;
    const int h = (int)(bh % H);
    const int64_t z = bh / H;
    float4 v = *reinterpret_cast<const float4 *>(x + z * sz + h * sh + (int64_t)n * sn + 4 * c);
    v.x = round_tf32(v.x); v.y = round_tf32(v.y); v.z = round_tf32(v.z); v.w = round_tf32(v.w);
    reinterpret_cast<float4 *>(y)[i] = v;
  }
}

__global__ void __launch_bounds__(256) transpose_v_kernel(const float *__restrict__ V, float *__restrict__ Vt, int H, int N_KV,
                                                          int D, int NP, int64_t sz, int64_t sh, int64_t sn) {
  __shared__ float tile[32][33];
  const int bh = blockIdx.z, z = bh / H, h = bh - z * H;
  const float *src = V + (int64_t)z * sz + (int64_t)h * sh;
  float *dst = Vt + (int64_t)bh * D * NP;
  const int n0 = blockIdx.x * 32, d0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8 threads
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int n = n0 + ty + 8 * i, d = d0 + tx;
    tile[ty + 8 * i][tx] = (n < N_KV && d < D) ? round_tf32(src[(int64_t)n * sn + d]) : 0.f;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int d = d0 + ty + 8 * i, n = n0 + tx;
    if (d < D && n < NP) dst[(int64_t)d * NP + n] = tile[tx][ty + 8 * i];
  }
}

template <int HD>
static int launch(const float *Q, const float *K, const float *V, float *O, int64_t Z, int64_t H, int64_t N, int64_t N_KV,
                  const int64_t *s, float scale_log2, int causal, cudaStream_t st) {
  using cfg = Cfg<HD>;
  if (Z * H > 65535 || N_KV > (int64_t)32 * 0x7fffffff) return HEXB_ERR_UNSUPPORTED;
  // One scratch block from the library's pool, freed in stream order after the attention kernel:
  // V^T [Z*H][HD][NP] (rounded to tf32), then dense rounded copies of Q [Z*H][N][HD] and K [Z*H][N_KV][HD].
  const int64_t NP = (N_KV + 31) / 32 * 32;
  const size_t vt_elems = (size_t)(Z * H) * HD * NP, q_elems = (size_t)(Z * H) * N * HD, k_elems = (size_t)(Z * H) * N_KV * HD;
  float *Vt = nullptr;
  if (int e = scratch_alloc(reinterpret_cast<void **>(&Vt), (vt_elems + q_elems + k_elems) * sizeof(float), st)) return e;
  float *Qr = Vt + vt_elems, *Kr = Qr + q_elems;
  transpose_v_kernel<<<dim3((unsigned)(NP / 32), HD / 32, (unsigned)(Z * H)), 256, 0, st>>>(V, Vt, (int)H, (int)N_KV, HD, (int)NP,
                                                                                        s[6], s[7], s[8]);
  {
    const int64_t qv = (int64_t)q_elems / 4, kv = (int64_t)k_elems / 4;
    const unsigned gq = (unsigned)((qv + 255) / 256 < 148 * 16 ? (qv + 255) / 256 : 148 * 16);
    const unsigned gk = (unsigned)((kv + 255) / 256 < 148 * 16 ? (kv + 255) / 256 : 148 * 16);
    round_copy_kernel<<<gq, 256, 0, st>>>(Q, Qr, (int)H, (int)N, HD, s[0], s[1], s[2], qv);
    round_copy_kernel<<<gk, 256, 0, st>>>(K, Kr, (int)H, (int)N_KV, HD, s[3], s[4], s[5], kv);
  }
  if (int e = check_launch("attn_tf32_prepare")) { scratch_free(Vt, st); return e; }
  CUtensorMap tm[3];
  const float *base[2] = {Qr, Kr};
  for (int i = 0; i < 2; ++i) {
    const uint64_t rows = (uint64_t)(i == 0 ? N : N_KV);
    const uint64_t dims[4] = {(uint64_t)HD, rows, (uint64_t)H, (uint64_t)Z};
    const uint64_t strides[3] = {(uint64_t)HD * 4, rows * HD * 4, (uint64_t)H * rows * HD * 4};
    const uint32_t box[4] = {32, i == 0 ? 128u : (uint32_t)BN, 1, 1};
    if (int e = encode_tmap_f32_sw128(&tm[i], base[i], 4, dims, strides, box)) { scratch_free(Vt, st); return e; }
  }
  {
    const uint64_t dims[4] = {(uint64_t)N_KV, (uint64_t)HD, (uint64_t)H, (uint64_t)Z};
    const uint64_t strides[3] = {(uint64_t)NP * 4, (uint64_t)HD * NP * 4, (uint64_t)H * HD * NP * 4};
    const uint32_t box[4] = {32, (uint32_t)HD, 1, 1};
    if (int e = encode_tmap_f32_sw128(&tm[2], Vt, 4, dims, strides, box)) { scratch_free(Vt, st); return e; }
  }
  static PerDeviceOnce attr_done;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done.is_done(dev)) {
    HEXB_CUDA_OK(cudaFuncSetAttribute(attn_fwd_tf32_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg::SMEM_BYTES));
    attr_done.mark(dev);
  }
  Params p;
  p.out = O;
  p.so_z = s[9]; p.so_h = s[10]; p.so_n = s[11];
  p.H = (int)H; p.N_CTX = (int)N; p.N_KV = (int)N_KV;
  p.out_vec_ok = aligned16(O) && s[9] % 4 == 0 && s[10] % 4 == 0 && s[11] % 4 == 0;
  p.num_q_tiles = (int)((N + BLOCK_M - 1) / BLOCK_M);
  p.tiles_per_cta = (causal && p.num_q_tiles % 2 == 0) ? 2 : 1;
  p.ctas_per_bh = p.num_q_tiles / p.tiles_per_cta;
  p.scale_log2 = scale_log2;
  p.causal = causal ? 1 : 0;
  const int64_t ctas = (int64_t)p.ctas_per_bh * Z * H;
  if (ctas > 0x7fffffffll) { scratch_free(Vt, st); return HEXB_ERR_UNSUPPORTED; }
  launch_pdl(attn_fwd_tf32_kernel<HD>, dim3((unsigned)ctas), dim3(THREADS), (size_t)cfg::SMEM_BYTES, st, tm[0], tm[1], tm[2],
             p);
  const int status = check_launch("attn_tf32");
  const int freed = scratch_free(Vt, st);
  return status ? status : freed;
}

}  // namespace attn32

// fp32 tensors the TMA path can take: head size 64 or 128, 16-byte aligned bases and strides.
int attn_tf32_supported(const void *Q, const void *K, const void *V, int64_t D, const int64_t *s) {
  if (D != 64 && D != 128) return 0;
  if (!aligned16(Q) || !aligned16(K) || !aligned16(V)) return 0;
  for (int i = 0; i < 9; ++i)
    if (s[i] % 4 != 0 || s[i] <= 0) return 0;
  return 1;
}

int attn_tf32_launch(const float *Q, const float *K, const float *V, float *O, int64_t Z, int64_t H, int64_t N, int64_t N_KV,
                     int64_t D, const int64_t *strides, float scale_log2, int causal, cudaStream_t st) {
  if (D == 128) return attn32::launch<128>(Q, K, V, O, Z, H, N, N_KV, strides, scale_log2, causal, st);
  if (D == 64) return attn32::launch<64>(Q, K, V, O, Z, H, N, N_KV, strides, scale_log2, causal, st);
  return HEXB_ERR_UNSUPPORTED;
}

int attn_tf32_status_fetch_and_clear(int *out) {
  int v = 0, zero = 0;
  HEXB_CUDA_OK(cudaMemcpyFromSymbol(&v, g_attn32_status, sizeof(int)));
  if (v) HEXB_CUDA_OK(cudaMemcpyToSymbol(g_attn32_status, &zero, sizeof(int)));
  *out = v;
  return HEXB_OK;
}

}  // namespace hexb
