// Flash-attention forward on the Blackwell tensor cores (tcgen05 + TMEM + TMA), fp16 in/out.
//
// Reference semantics: attention_fwd_kernel + _attn_fwd_inner
// (test/python/triton/test_flash_attention.py:37-168) and the fp16 MLIR form
// (test/python/mlir/hexkl_attention/input.mlir:5-168) of qualcomm/hexagon-mlir: per block of query
// rows, loop over key/value blocks; qk = Q.K^T; base-2 online softmax with the scale folded in
// (qk_scale = sm_scale * 1.44269504); acc = acc*alpha + P.V with P truncated to fp16 before the
// second product; epilogue acc / l.  The causal flag adds the -inf mask above the diagonal that
// tm_tensor.attention takes as an additive mask (lib/Transforms/LowerTmTensor.cpp:70-235).
//
// One CTA = one 128-row query tile of one (batch, head); 192 threads:
//   warp 0      TMA producer (Q once; K_j, V_j per step; single buffers, refilled as soon as the
//               MMA that read them has completed);
//   warp 1      MMA issuer: S = Q.K_j^T (8 x tcgen05.mma 128x128x16, operands in smem), then
//               O += P_j.V_j (P read from TMEM, V consumed as stored = "MN-major" operand);
//   warps 2..5  one query row per thread: tcgen05.ld S, row max, P = exp2(S*scale - m) written back
//               to TMEM as fp16 over the S columns, running sum; O is rescaled in TMEM only when a
//               row max grows by more than 2^8 (the same reference max is used for P and l, so the
//               final O/l is exact); epilogue O/l -> fp16 -> global.
// Two CTAs share an SM (96 KiB smem and 256 TMEM columns each), so one CTA's softmax overlaps the
// other's MMAs.  Every mbarrier wait is bounded.
//
// A CUDA-core kernel covers fp32 tensors (the dtype of the reference's Triton test) and head
// sizes / strides the TMA path cannot take.
#include "attn_common.cuh"

namespace hexb {

static __device__ int g_attn_status = 0;

namespace attn {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_N = 128;
constexpr int THREADS = 192;

template <int HD>
struct Cfg {
  static constexpr int CHUNKS = HD / 64;             // 64-column (128-byte) swizzle chunks
  static constexpr int TILE_BYTES = 128 * HD * 2;    // Q, K or V tile
  static constexpr int CHUNK_BYTES = 128 * 128;      // 128 rows x 128 bytes
  static constexpr int BAR_BYTES = 10 * 8 + 16;
  static constexpr int NEEDED = 3 * TILE_BYTES + BAR_BYTES + 1024;
  static constexpr int SMEM_BYTES = NEEDED < 100 * 1024 ? 100 * 1024 : NEEDED;  // caps residency at 2 CTAs/SM
  static constexpr int TMEM_COLS = 256;              // S: [0,128)  (P aliases [0,64));  O: [128,128+HD)
  static constexpr int O_COL = 128;
};

struct Params {
#ifdef HEXB_ATTN_PROFILE
  unsigned long long *prof;
#endif
  void *out;           // __half, or float when out_f32
  int64_t so_z, so_h, so_n;
  int Z, H, N_CTX;     // N_CTX: query rows
  int N_KV;            // key/value rows (the 128-key kernel takes N_KV == N_CTX only)
  int out_f32;
  const void *mask;    // additive mask [Z, H, N_CTX, N_KV] (strides below, innermost 1), or null
  int mask_f32;        // mask element type: 1 float, 0 __half
  int mask_vec_ok;     // 16-byte loads of the mask row are aligned
  int mask_tma;        // the mask arrives through the tensor map (fp16, 16-byte aligned strides, one row per query)
  int mask_h_on, mask_z_on;   // 0: that dimension of the mask is broadcast (its tensor-map extent is 1)
  int head_major;             // CTA order: the batches of a head adjacent (mask shared by them), else the heads of a batch
  int64_t sm_z, sm_h, sm_q;
  int num_q_tiles;
  int tiles_per_cta;   // query tiles one CTA walks (1 or 2)
  int ctas_per_bh;     // num_q_tiles / tiles_per_cta
  float scale_log2;
  int causal;
  int out_vec_ok;
  uint32_t v_lbo, v_sbo;
#ifdef HEXB_DEV
  int ablate;          // development builds: 1 = the MMA thread issues no MMAs, 2 = the softmax warps do no arithmetic
#endif
};

template <int HD>
__global__ void __launch_bounds__(THREADS, 2)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const Params p) {
  using cfg = Cfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = tc::smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
  uint8_t *smem = smem_raw + pad;
  const uint32_t smem_addr = raw_addr + pad;
  const uint32_t sQ = smem_addr, sK = sQ + cfg::TILE_BYTES, sV = sK + cfg::TILE_BYTES;
  const uint32_t bar0 = sV + cfg::TILE_BYTES;
  const uint32_t q_full = bar0, k_full = bar0 + 8, k_empty = bar0 + 16, v_full = bar0 + 24,
                 v_empty = bar0 + 32, s_full = bar0 + 40, p_full = bar0 + 48, o_full = bar0 + 56,
                 q_empty = bar0 + 64, o_empty = bar0 + 72;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + 3 * cfg::TILE_BYTES + 80);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Work: the CTAs of one (batch, head) are adjacent in launch order, so its K and V stay in L2
  // while they are re-read.  A CTA walks tiles_per_cta query tiles one after the other; when causal
  // it pairs a heavy (late) tile with a light (early) one so that every CTA does the same number
  // of key/value steps, and heavy tiles come first.
  const int bh = blockIdx.x / p.ctas_per_bh;
  const int q_rank = blockIdx.x - bh * p.ctas_per_bh;
  const int z = bh / p.H, h = bh - z * p.H;
  const int kv_tiles = (p.N_CTX + BLOCK_N - 1) / BLOCK_N;
  auto tile_of = [&](int t) {
    if (p.causal) return t == 0 ? p.num_q_tiles - 1 - q_rank : q_rank;
    return q_rank * p.tiles_per_cta + t;
  };
  auto nkv_of = [&](int q_tile) { return (p.causal && q_tile + 1 < kv_tiles) ? q_tile + 1 : kv_tiles; };

  if (threadIdx.x == 0) {
    tc::mbar_init(q_full, 1);
    tc::mbar_init(k_full, 1);
    tc::mbar_init(k_empty, 1);
    tc::mbar_init(v_full, 1);
    tc::mbar_init(v_empty, 1);
    tc::mbar_init(s_full, 1);
    tc::mbar_init(p_full, 4);
    tc::mbar_init(o_full, 1);
    tc::mbar_init(q_empty, 1);
    tc::mbar_init(o_empty, 4);
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
  const uint32_t tS = tmem_base, tP = tmem_base, tO = tmem_base + cfg::O_COL;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;  // key/value steps so far, across tiles
      bool ok = true;
      for (int t = 0; t < p.tiles_per_cta && ok; ++t) {
        const int q_tile = tile_of(t);
        const int n_kv = nkv_of(q_tile);
        // the previous tile's last Q.K^T has read Q
        if (t > 0 && !tc::mbar_wait(q_empty, (uint32_t)(t - 1) & 1u, abort_flag)) break;
        tc::mbar_arrive_expect_tx(q_full, cfg::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < cfg::CHUNKS; ++c)
          tc::tma_load_4d(sQ + c * cfg::CHUNK_BYTES, &tmQ, c * 64, q_tile * BLOCK_M, h, z, q_full);
        for (int j = 0; j < n_kv; ++j, ++it) {
          const uint32_t ph = it & 1u;
          if (!tc::mbar_wait(k_empty, ph ^ 1u, abort_flag)) { ok = false; break; }
          tc::mbar_arrive_expect_tx(k_full, cfg::TILE_BYTES);
#pragma unroll
          for (int c = 0; c < cfg::CHUNKS; ++c)
            tc::tma_load_4d(sK + c * cfg::CHUNK_BYTES, &tmK, c * 64, j * BLOCK_N, h, z, k_full);
          if (!tc::mbar_wait(v_empty, ph ^ 1u, abort_flag)) { ok = false; break; }
          tc::mbar_arrive_expect_tx(v_full, cfg::TILE_BYTES);
#pragma unroll
          for (int c = 0; c < cfg::CHUNKS; ++c)
            tc::tma_load_4d(sV + c * cfg::CHUNK_BYTES, &tmV, c * 64, j * BLOCK_N, h, z, v_full);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = tc::make_idesc_f16_f32(BLOCK_M, BLOCK_N, 0, 0);
      constexpr uint32_t idesc_pv = tc::make_idesc_f16_f32(BLOCK_M, HD, 0, 1);
      uint32_t it = 0;
      bool ok = true;
      for (int t = 0; t < p.tiles_per_cta && ok; ++t) {
        const int n_kv = nkv_of(tile_of(t));
        if (!tc::mbar_wait(q_full, (uint32_t)t & 1u, abort_flag)) break;
        for (int j = 0; j < n_kv; ++j, ++it) {
          const uint32_t ph = it & 1u;
          if (!tc::mbar_wait(k_full, ph, abort_flag)) { ok = false; break; }
          tc::tc_fence_after();
#pragma unroll
          for (int k = 0; k < HD / 16; ++k) {
            const uint32_t off = (uint32_t)((k >> 2) * cfg::CHUNK_BYTES + (k & 3) * 32);
            tc::mma_f16_ss(tS, tc::make_smem_desc_sw128(sQ + off, 16, 1024),
                           tc::make_smem_desc_sw128(sK + off, 16, 1024), idesc_qk, k != 0 ? 1u : 0u);
          }
          tc::mma_commit(s_full);
          tc::mma_commit(k_empty);
          if (j == n_kv - 1) tc::mma_commit(q_empty);
          if (!tc::mbar_wait(p_full, ph, abort_flag)) { ok = false; break; }
          if (!tc::mbar_wait(v_full, ph, abort_flag)) { ok = false; break; }
          // the first product of a later tile overwrites O: the previous epilogue must have read it
          if (j == 0 && t > 0 && !tc::mbar_wait(o_empty, (uint32_t)(t - 1) & 1u, abort_flag)) { ok = false; break; }
          tc::tc_fence_after();
#pragma unroll
          for (int k = 0; k < BLOCK_N / 16; ++k) {
            // A = P rows from TMEM (16 fp16 = 8 columns per step); B = V: 16 kv rows = 2 swizzle atoms.
            tc::mma_f16_ts(tO, tP + (uint32_t)(k * 8),
                           tc::make_smem_desc_sw128(sV + (uint32_t)(k * 2048), p.v_lbo, p.v_sbo),
                           idesc_pv, (j | k) != 0 ? 1u : 0u);
          }
          tc::mma_commit(v_empty);
          if (j == n_kv - 1) tc::mma_commit(o_full);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / correction / epilogue
    const int q = warp & 3;
    const int r = q * 32 + lane;       // row inside the tile == TMEM lane
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    uint32_t it = 0;
    bool ok = true;
    for (int t = 0; t < p.tiles_per_cta && ok; ++t) {
      const int q_tile = tile_of(t);
      const int n_kv = nkv_of(q_tile);
      const int m0 = q_tile * BLOCK_M;
      const int qi = m0 + r;           // query index
      float m_ref = -INFINITY, l = 0.f;
      for (int j = 0; j < n_kv; ++j, ++it) {
        if (!tc::mbar_wait(s_full, it & 1u, abort_flag)) { ok = false; break; }
        tc::tc_fence_after();
        const int kv0 = j * BLOCK_N;
        const bool need_mask = (p.causal && kv0 + BLOCK_N - 1 > m0) || (kv0 + BLOCK_N > p.N_CTX);
        // The whole score row (128 fp32) comes into registers with one wait.
        uint32_t sv[BLOCK_N];
#pragma unroll
        for (int c = 0; c < BLOCK_N / 32; ++c)
          tc::tmem_ld_32x32(tS + lane_off + (uint32_t)(c * 32), reinterpret_cast<uint32_t(&)[32]>(sv[c * 32]));
        tc::tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int e = 0; e < BLOCK_N; ++e) {
            const int kv = kv0 + e;
            if ((p.causal && kv > qi) || kv >= p.N_CTX) sv[e] = 0xff800000u;  // -inf: exp2 gives 0
          }
        }
        // row maximum: three-input max, four independent chains
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int e = 0; e < BLOCK_N; e += 8) {
#pragma unroll
          for (int u = 0; u < 4; ++u)
            mx4[u] = max3(mx4[u], __uint_as_float(sv[e + 2 * u]), __uint_as_float(sv[e + 2 * u + 1]));
        }
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        mx *= p.scale_log2;  // scale > 0: max commutes with the scaling
        const float m_new = fmaxf(m_ref, mx);
        if (j == 0) {
          m_ref = m_new;
        } else if (__any_sync(0xffffffffu, m_new - m_ref > kRescaleThreshold)) {
          // S_j complete implies P_{j-1}.V_{j-1} complete (MMAs retire in issue order): O is quiescent.
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
        }
        // P = exp2(S*scale - m_ref) as fp16 over the S columns; running row sum in fp32
        const float neg_m = -m_ref;
        float l0 = 0.f, l1 = 0.f;
#pragma unroll
        for (int c = 0; c < BLOCK_N / 32; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const float x0 = fmaf(__uint_as_float(sv[c * 32 + e]), p.scale_log2, neg_m);
            const float x1 = fmaf(__uint_as_float(sv[c * 32 + e + 1]), p.scale_log2, neg_m);
            const float p0 = ex2_approx(x0);
            const float p1 = ex2_approx(x1);
            l0 += p0;
            l1 += p1;
            pk[e >> 1] = pack_f16x2(p0, p1);
          }
          tc::tmem_st_32x16(tP + lane_off + (uint32_t)(c * 16), pk);
        }
        l += l0 + l1;
        tc::tmem_st_wait();
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(p_full);
      }
      if (!ok || !tc::mbar_wait(o_full, (uint32_t)t & 1u, abort_flag)) { ok = false; break; }
      tc::tc_fence_after();
      const float inv = 1.0f / l;
      __half *orow = static_cast<__half *>(p.out) + (int64_t)z * p.so_z + (int64_t)h * p.so_h + (int64_t)qi * p.so_n;
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
          for (int g = 0; g < 4; ++g) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(o[g * 8 + e]) * inv;
            if (p.out_vec_ok) {
              Vec16<__half> ov;
              ov.pack(f);
              *reinterpret_cast<uint4 *>(orow + c * 32 + g * 8) = ov.raw;
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e) orow[c * 32 + g * 8 + e] = __float2half_rn(f[e]);
            }
          }
        }
      }
    }
  }

  // ------------------------------------------------------------ teardown
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, cfg::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&g_attn_status, (int)HEXB_ERR_TIMEOUT);
}

// ---------------------------------------------------------------------------------------------
// Second form of the tensor-core kernel: 64-wide key/value blocks with TWO score buffers.
//
// In the kernel above P aliases S, so Q.K^T of block j+1 cannot start before the softmax of block j
// has finished: every stream is a serial chain MMA -> softmax -> MMA.  Here a block is 64 keys, so
// two S buffers (2 x 64 columns) plus O (128) still fit 256 TMEM columns (two CTAs per SM), and two
// K and two V tiles of 64 rows fit the same 96 KiB of shared memory.  The MMA thread issues
// Q.K_{j+1}^T into the other S buffer before it waits for P_j, so the softmax warps find the next
// scores ready when they finish a block and the tensor pipe works through Q.K^T / P.V while they
// exponentiate.  P_j is written over the first 32 columns of S buffer j%2; Q.K_{j+2}^T, which
// overwrites it, is issued after P_j.V_j (the tensor pipe retires in issue order).
// BN_ = 128 (no mask; option attn_kernel = 5): key blocks twice as wide, so Q is read from shared memory
// once per 128 keys instead of twice; the two score buffers then take 256 TMEM columns and O sits at
// 256: all 512 columns and 160 KiB of shared memory, i.e. one CTA per SM, whose softmax threads hold
// the 128 scores of a row in registers.  Measured slower than two CTAs per SM with 64-key blocks
// ([4,32,4096,128]: 947 vs 1086 TFLOP/s, causal 834 vs 980): with four softmax warps per SM the
// exponentials, not the shared-memory reads, set the pace.  A variant with two query tiles per CTA
// taking turns on the tensor pipe (eight softmax warps, 128-key blocks, one score buffer per tile)
// measured 1070 / 872: the same pace as the default, bounded the same way.
template <int HD, int BN_ = 64>
struct Cfg2 {
  static constexpr int BN = BN_;                      // keys per block
  static constexpr int CHUNKS = HD / 64;
  static constexpr int Q_BYTES = 128 * HD * 2;
  static constexpr int Q_CHUNK = 128 * 128;           // 128 rows x 128 bytes
  static constexpr int KV_BYTES = BN * HD * 2;
  static constexpr int KV_CHUNK = BN * 128;           // 64 rows x 128 bytes
  static constexpr int NBAR = 29;
  static constexpr int NEEDED = Q_BYTES + 4 * KV_BYTES + NBAR * 8 + 16 + 1024;
  static constexpr int SMEM_BYTES = NEEDED < 100 * 1024 ? 100 * 1024 : NEEDED;  // caps residency at 2 CTAs/SM
  // Masked variant: one 32-row x 64-key fp16 mask tile per softmax warp, filled by TMA.  Two CTAs of
  // this size still fit one SM only if the 1024-byte alignment of the buffers costs no padding, which
  // the declared alignment of the dynamic shared array provides; the kernel checks it and reports
  // a status instead of running past its allocation if that ever fails to hold.
  static constexpr int MASK_STAGE = 32 * 128;
  static constexpr int MASK_BYTES = 4 * MASK_STAGE;
  static constexpr int SMEM_BYTES_MASK = Q_BYTES + 4 * KV_BYTES + MASK_BYTES + NBAR * 8 + 16 + 160;
  // P through shared memory (PS form): one more 128-row x 128-byte tile; the 1024-byte alignment of the
  // dynamic shared array is relied upon as in the masked variant (the kernel checks it)
  static constexpr int P_BYTES = 128 * 128;
  static constexpr int SMEM_BYTES_PS = Q_BYTES + 4 * KV_BYTES + P_BYTES + NBAR * 8 + 16 + 160;
  static constexpr int TMEM_COLS = BN == 64 ? 256 : 512;   // S0 [0,BN), S1 [BN,2BN), O [2BN,2BN+HD); P_b over S_b[0,BN/2)
  static constexpr int O_COL = 2 * BN;
};

// MASK: an additive mask tile is read by the softmax warps and the scores are formed as s * scale + mask
// before the running maximum is taken; log2(e) multiplies them where the unmasked kernel applies its scale.
// TPR = 2: two softmax threads per query row (eight softmax warps, 320 threads): warps w and w + 4 own
// the same 32 rows (a warp may only touch its own quarter of the TMEM lanes) and half of a block's score
// columns and of the output columns each; they exchange their row maxima once per block, and their row
// sums once per tile, through shared memory and a named barrier of the two warps.  Every scheduler then
// holds two warps of a CTA that exponentiate together, which is what the special-function unit needs to
// run at its full rate (a warp alone on its scheduler gets 8/11 of it), and the load / mask / max / pack
// work of a block is spread over twice the threads.  Selectable (attn_kernel = 9), not the default: on
// [4, 32, 4096, 128] it measured 583 us causal / 1048 us plain against 552 / 1000 with one thread per row.
// Taking the kernel apart in a development build says why: with the softmax arithmetic skipped the MMAs and
// loads alone take 92 % of the full kernel's time (with the MMAs skipped the softmax alone takes 71 %), so
// the softmax warps are not what the kernel waits for, and the exchange only adds to their share.
// PS = true ("P through shared memory"): the softmax warps write P_j as fp16 into a 16 KiB tile of shared
// memory (128-byte swizzle, the layout of a Q chunk) and P_j.V_j reads both operands from shared memory.
// The score buffer of block j is then free as soon as the softmax warps have loaded it, not only after
// P_j.V_j: Q.K_{j+2}^T is issued then -- while block j is still being exponentiated -- so the scores of
// the next block but one are under way two softmax periods before they are needed, and P_j.V_j goes out
// the moment P_j is there instead of behind a Q.K^T.  K and V get a producer thread each (224 threads), so
// that a K tile is not held back by the V tile queued in front of it.  Selectable (attn_kernel = 10), not the
// default: measured on [4, 32, 4096, 128] 605 us causal / 1095 us plain against 563 / 1020 in the same process.
// The softmax warps alone (MMAs skipped in a development build) get slower by the stores to shared memory
// and the proxy fence (1458 against 1273 clocks per 128 x 128 block and SM), which costs more than the
// earlier scores gain.
// K3 = true: a third K stage (in the 16 KiB the mask tiles or the P tile would take), so that the K tile of
// block j + 2 can be fetched while blocks j and j + 1 are both still unread.  Selectable (attn_kernel = 11);
// it measured level with two stages (551 / 1001 us against 551 / 1000 on [4, 32, 4096, 128] causal / plain):
// the K tiles are not what the MMA thread waits for.
template <int HD, bool MASK, int BN_ = 64, int TPR = 1, bool PS = false, bool K3 = false>
__global__ void __launch_bounds__(64 + 128 * TPR + (PS ? 32 : 0), BN_ == 64 ? 2 : 1)
attn_fwd_tc2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmM,
                    const Params p) {
  using cfg = Cfg2<HD, BN_>;
  constexpr int BN = cfg::BN;
  static_assert(!MASK || BN == 64, "the masked variant stages 64-key mask tiles");
  static_assert(TPR == 1 || (TPR == 2 && !MASK && BN == 64), "two threads per row: plain 64-key blocks only");
  static_assert(!PS || (TPR == 1 && !MASK && BN == 64), "P through shared memory: plain 64-key blocks, one thread per row");
  static_assert(!K3 || (TPR == 1 && !MASK && !PS && BN == 64), "third K stage: the plain 64-key kernel only");
  constexpr int COLS = BN / TPR;     // score columns per softmax thread
  constexpr int OCOLS = HD / TPR;    // output columns per softmax thread
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw_addr = tc::smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
  constexpr uint32_t kMaskBytes = MASK ? cfg::MASK_BYTES : (PS || K3) ? cfg::P_BYTES : 0;   // the P tile or the third K stage sits where the mask tiles would
  if ((MASK && pad + cfg::Q_BYTES + 4 * cfg::KV_BYTES + kMaskBytes + cfg::NBAR * 8 + 16 > (uint32_t)cfg::SMEM_BYTES_MASK) ||
      ((PS || K3) && pad + cfg::Q_BYTES + 4 * cfg::KV_BYTES + kMaskBytes + cfg::NBAR * 8 + 16 > (uint32_t)cfg::SMEM_BYTES_PS)) {
    // the layout would not fit the allocation: every thread leaves before any barrier or TMEM use
    if (threadIdx.x == 0) atomicExch(&g_attn_status, (int)HEXB_ERR_MISALIGNED);
    return;
  }
  uint8_t *smem = smem_raw + pad;
  const uint32_t smem_addr = raw_addr + pad;
  const uint32_t sQ = smem_addr;
  const uint32_t sK0 = sQ + cfg::Q_BYTES, sV0 = sK0 + 2 * cfg::KV_BYTES;
  const uint32_t sM0 = sV0 + 2 * cfg::KV_BYTES;   // mask tiles (masked variant only)
  const uint32_t bar0 = sM0 + kMaskBytes;
  const uint32_t q_full = bar0, q_empty = bar0 + 8, o_full = bar0 + 16, o_empty = bar0 + 24, pv_done = bar0 + 32;
  auto k_full = [&](uint32_t b) { return b < 2 ? bar0 + 40 + 8 * b : bar0 + 216; };    // b == 2: third K stage (K3)
  auto k_empty = [&](uint32_t b) { return b < 2 ? bar0 + 56 + 8 * b : bar0 + 224; };
  auto k_stage = [&](uint32_t b) { return b < 2 ? sQ + cfg::Q_BYTES + b * cfg::KV_BYTES : sQ + cfg::Q_BYTES + 4 * cfg::KV_BYTES; };
  // K stage and phase of block `blk`: two stages alternate with the score buffers, three have their own count
  auto k_slot = [&](uint32_t blk, uint32_t &kb, uint32_t &kph) {
    if (K3) { kb = blk % 3u; kph = (blk / 3u) & 1u; }
    else { kb = blk & 1u; kph = (blk >> 1) & 1u; }
  };
  auto v_full = [&](uint32_t b) { return bar0 + 72 + 8 * b; };
  auto v_empty = [&](uint32_t b) { return bar0 + 88 + 8 * b; };
  auto s_full = [&](uint32_t b) { return bar0 + 104 + 8 * b; };
  // barrier slots: q_full .. pv_done (5), then pairs k_full, k_empty, v_full, v_empty, s_full, p_full (12), then
  // one m_full per softmax warp (4), one x_bar per lane quarter (4; two threads per row only), two s_free (PS), k_full / k_empty of the third K stage (K3): NBAR = 29
  auto p_full = [&](uint32_t b) { return bar0 + 120 + 8 * b; };
  auto m_full = [&](uint32_t w) { return bar0 + 136 + 8 * w; };   // one per softmax warp
  auto x_bar = [&](uint32_t qq) { return bar0 + 168 + 8 * qq; };  // the two warps that share a lane quarter
  auto s_free = [&](uint32_t b) { return bar0 + 200 + 8 * b; };   // PS: score buffer b has been loaded by the softmax warps
  const uint32_t sP = sM0;                                        // PS: the P tile
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + cfg::Q_BYTES + 4 * cfg::KV_BYTES + kMaskBytes + cfg::NBAR * 8);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  // TPR == 2: exchange slots [parity][half][row] for row maxima and row sums (2 KiB behind the flags)
  float *xch = reinterpret_cast<float *>(tmem_slot + 2);
  if (TPR == 2 && pad + cfg::Q_BYTES + 4 * cfg::KV_BYTES + cfg::NBAR * 8 + 8 + 2048 > (uint32_t)cfg::SMEM_BYTES) {  // cannot happen for pad < 1024
    if (threadIdx.x == 0) atomicExch(&g_attn_status, (int)HEXB_ERR_MISALIGNED);
    return;
  }

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int bh = blockIdx.x / p.ctas_per_bh;
  const int q_rank = blockIdx.x - bh * p.ctas_per_bh;
  // (batch, head) of this CTA: batch-major by default; head-major when a mask is shared by the batches of a
  // head, so that the CTAs which read the same mask tiles run next to each other and find them in L2
  const int z = p.head_major ? bh % p.Z : bh / p.H;
  const int h = p.head_major ? bh / p.Z : bh - z * p.H;
  const int kv_blocks = (p.N_KV + BN - 1) / BN;
  auto tile_of = [&](int t) {
    if (p.causal) return t == 0 ? p.num_q_tiles - 1 - q_rank : q_rank;
    return q_rank * p.tiles_per_cta + t;
  };
  // causal: keys 0 .. m0+127 -> (q_tile+1) * 128 / BN blocks
  auto nkv_of = [&](int q_tile) {
    const int need = (BLOCK_M / BN) * (q_tile + 1);
    return (p.causal && need < kv_blocks) ? need : kv_blocks;
  };

  if (threadIdx.x == 0) {
    tc::mbar_init(q_full, 1);
    tc::mbar_init(q_empty, 1);
    tc::mbar_init(o_full, 1);
    tc::mbar_init(o_empty, 4 * TPR);
    tc::mbar_init(pv_done, 1);
    for (uint32_t b = 0; b < 2; ++b) {
      tc::mbar_init(k_full(b), 1);
      tc::mbar_init(k_empty(b), 1);
      tc::mbar_init(v_full(b), 1);
      tc::mbar_init(v_empty(b), 1);
      tc::mbar_init(s_full(b), 1);
      tc::mbar_init(p_full(b), 4 * TPR);
    }
    for (uint32_t w = 0; w < 4; ++w) tc::mbar_init(m_full(w), 1);
    for (uint32_t w = 0; w < 4; ++w) tc::mbar_init(x_bar(w), 2);
    for (uint32_t b = 0; b < 2; ++b) tc::mbar_init(s_free(b), 4);
    tc::mbar_init(k_full(2), 1);
    tc::mbar_init(k_empty(2), 1);
    *abort_flag = 0;
    tc::fence_barrier_init();
    tc::prefetch_tensormap(&tmQ);
    tc::prefetch_tensormap(&tmK);
    tc::prefetch_tensormap(&tmV);
    if (MASK && p.mask_tma) tc::prefetch_tensormap(&tmM);
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

  if (warp == 0 || (PS && warp == 6)) {
    // ------------------------------------------------------------ TMA producer(s)
    // One thread loads Q, K and V in turn; in the PS form warp 0 loads Q and K and warp 6 loads V.
    const bool do_k = !PS || warp == 0, do_v = !PS || warp == 6;
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = 0; t < p.tiles_per_cta && ok; ++t) {
        const int q_tile = tile_of(t);
        const int n_kv = nkv_of(q_tile);
        if (do_k) {
          if (t > 0 && !tc::mbar_wait(q_empty, (uint32_t)(t - 1) & 1u, abort_flag)) break;
          tc::mbar_arrive_expect_tx(q_full, cfg::Q_BYTES);
#pragma unroll
          for (int c = 0; c < cfg::CHUNKS; ++c)
            tc::tma_load_4d(sQ + c * cfg::Q_CHUNK, &tmQ, c * 64, q_tile * BLOCK_M, h, z, q_full);
        }
        for (int j = 0; j < n_kv; ++j, ++it) {
          const uint32_t b = it & 1u, ph = (it >> 1) & 1u;
          if (do_k) {
            uint32_t kb, kph;
            k_slot(it, kb, kph);
            if (!tc::mbar_wait(k_empty(kb), kph ^ 1u, abort_flag)) { ok = false; break; }
            tc::mbar_arrive_expect_tx(k_full(kb), cfg::KV_BYTES);
#pragma unroll
            for (int c = 0; c < cfg::CHUNKS; ++c)
              tc::tma_load_4d(k_stage(kb) + c * cfg::KV_CHUNK, &tmK, c * 64, j * BN, h, z, k_full(kb));
          }
          if (do_v) {
            if (!tc::mbar_wait(v_empty(b), ph ^ 1u, abort_flag)) { ok = false; break; }
            tc::mbar_arrive_expect_tx(v_full(b), cfg::KV_BYTES);
#pragma unroll
            for (int c = 0; c < cfg::CHUNKS; ++c)
              tc::tma_load_4d(sV0 + b * cfg::KV_BYTES + c * cfg::KV_CHUNK, &tmV, c * 64, j * BN, h, z, v_full(b));
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = tc::make_idesc_f16_f32(BLOCK_M, BN, 0, 0);
      constexpr uint32_t idesc_pv = tc::make_idesc_f16_f32(BLOCK_M, HD, 0, 1);
      bool ok = true;
      // S_{blk} = Q . K_{blk}^T into score buffer blk % 2
      HEXB_PROF_DECL(8)
      auto issue_qk = [&](uint32_t blk, bool last_of_tile) {
        const uint32_t b = blk & 1u;
        uint32_t kb, kph;
        k_slot(blk, kb, kph);
        HEXB_PROF(0)  // other
        if (!tc::mbar_wait(k_full(kb), kph, abort_flag)) { ok = false; return; }
        HEXB_PROF(1)  // wait K
        tc::tc_fence_after();
        const uint32_t sK = k_stage(kb);
#ifdef HEXB_DEV
        if (!(p.ablate & 1))
#endif
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t qoff = (uint32_t)((k >> 2) * cfg::Q_CHUNK + (k & 3) * 32);
          const uint32_t koff = (uint32_t)((k >> 2) * cfg::KV_CHUNK + (k & 3) * 32);
          tc::mma_f16_ss(tmem_base + b * BN, tc::make_smem_desc_sw128(sQ + qoff, 16, 1024),
                         tc::make_smem_desc_sw128(sK + koff, 16, 1024), idesc_qk, k != 0 ? 1u : 0u);
        }
        tc::mma_commit(s_full(b));
        tc::mma_commit(k_empty(kb));
        if (last_of_tile) tc::mma_commit(q_empty);
        HEXB_PROF(2)  // issue QK
      };
      uint32_t it = 0;
      if constexpr (PS) {
        // P.V_j: both operands from shared memory (P tile K-major like a Q chunk, V as stored)
        constexpr uint32_t idesc_pv_ss = tc::make_idesc_f16_f32(BLOCK_M, HD, 0, 1);
        for (int t = 0; t < p.tiles_per_cta && ok; ++t) {
          const int n_kv = nkv_of(tile_of(t));
          if (!tc::mbar_wait(q_full, (uint32_t)t & 1u, abort_flag)) break;
          // the first two score blocks of the tile; their buffers were loaded by the softmax warps two blocks ago
          for (int j0 = 0; j0 < 2 && j0 < n_kv && ok; ++j0) {
            const uint32_t blk = it + (uint32_t)j0;
            if (blk >= 2 && !tc::mbar_wait(s_free(blk & 1u), ((blk >> 1) - 1u) & 1u, abort_flag)) { ok = false; break; }
            tc::tc_fence_after();
            issue_qk(blk, j0 + 1 == n_kv);
          }
          for (int j = 0; j < n_kv && ok; ++j, ++it) {
            const uint32_t b = it & 1u, ph = (it >> 1) & 1u;
            // scores of the next block but one go into the buffer of block j as soon as the softmax warps have
            // that block in registers -- before P_j exists, so that P_j.V_j is not queued behind them later
            if (j + 2 < n_kv) {
              if (!tc::mbar_wait(s_free(b), ph, abort_flag)) { ok = false; break; }
              tc::tc_fence_after();
              issue_qk(it + 2u, j + 3 == n_kv);
              if (!ok) break;
            }
            if (!tc::mbar_wait(p_full(0), it & 1u, abort_flag)) { ok = false; break; }
            if (!tc::mbar_wait(v_full(b), ph, abort_flag)) { ok = false; break; }
            if (j == 0 && t > 0 && !tc::mbar_wait(o_empty, (uint32_t)(t - 1) & 1u, abort_flag)) { ok = false; break; }
            tc::tc_fence_after();
            const uint32_t sV = sV0 + b * cfg::KV_BYTES;
#ifdef HEXB_DEV
            if (!(p.ablate & 1))
#endif
#pragma unroll
            for (int k = 0; k < BN / 16; ++k) {
              tc::mma_f16_ss(tO, tc::make_smem_desc_sw128(sP + (uint32_t)(k * 32), 16, 1024),
                             tc::make_smem_desc_sw128(sV + (uint32_t)(k * 2048), cfg::KV_CHUNK, 1024), idesc_pv_ss,
                             (j | k) != 0 ? 1u : 0u);
            }
            tc::mma_commit(v_empty(b));
            tc::mma_commit(pv_done);
            if (j == n_kv - 1) tc::mma_commit(o_full);
          }
        }
      } else {
      for (int t = 0; t < p.tiles_per_cta && ok; ++t) {
        const int n_kv = nkv_of(tile_of(t));
        if (!tc::mbar_wait(q_full, (uint32_t)t & 1u, abort_flag)) break;
        issue_qk(it, n_kv == 1);
        for (int j = 0; j < n_kv && ok; ++j, ++it) {
          if (j + 1 < n_kv) issue_qk(it + 1, j + 2 == n_kv);  // run one block ahead of the softmax
          if (!ok) break;
          const uint32_t b = it & 1u, ph = (it >> 1) & 1u;
          if (!tc::mbar_wait(p_full(b), ph, abort_flag)) { ok = false; break; }
          HEXB_PROF(3)  // wait P
          if (!tc::mbar_wait(v_full(b), ph, abort_flag)) { ok = false; break; }
          HEXB_PROF(4)  // wait V
          // the first product of a later tile overwrites O: the previous epilogue must have read it
          if (j == 0 && t > 0 && !tc::mbar_wait(o_empty, (uint32_t)(t - 1) & 1u, abort_flag)) { ok = false; break; }
          tc::tc_fence_after();
          const uint32_t sV = sV0 + b * cfg::KV_BYTES;
#ifdef HEXB_DEV
          if (!(p.ablate & 1))
#endif
#pragma unroll
          for (int k = 0; k < BN / 16; ++k) {
            tc::mma_f16_ts(tO, tmem_base + b * BN + (uint32_t)(k * 8),
                           tc::make_smem_desc_sw128(sV + (uint32_t)(k * 2048), cfg::KV_CHUNK, 1024), idesc_pv,
                           (j | k) != 0 ? 1u : 0u);
          }
          tc::mma_commit(v_empty(b));
          tc::mma_commit(pv_done);
          if (j == n_kv - 1) tc::mma_commit(o_full);
          HEXB_PROF(5)  // issue PV
        }
      }
      }
      HEXB_PROF_FLUSH(0, 8)
    }
  } else {
    // ------------------------------------------------------------ softmax / correction / epilogue
    const int q = warp & 3;
    const int hsel = TPR == 2 ? ((warp - 2) >> 2) : 0;   // which half of the columns (two threads per row)
    const int c0 = hsel * COLS;                          // first score column of this thread inside a block
    const int r = q * 32 + lane;
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    // Value exchange between the two threads of a row: slot [parity][half][row], parity alternating per
    // exchange so that a thread never overwrites a value its partner may still have to read; the two
    // warps meet at the mbarrier of their lane quarter (a bounded wait, like every other one here).
    uint32_t xc = 0;
    auto exchange = [&](float mine, float &other) -> bool {
      float *slot = xch + (xc & 1u) * 256;
      slot[hsel * 128 + r] = mine;
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(x_bar((uint32_t)q));
      if (!tc::mbar_wait(x_bar((uint32_t)q), xc & 1u, abort_flag)) return false;
      ++xc;
      other = slot[(hsel ^ 1) * 128 + r];
      return true;
    };
    (void)exchange;
    uint32_t it = 0;
    bool ok = true;
    // Mask tiles by TMA: this warp's 32 rows x 64 keys land in its own staging buffer (128-byte
    // swizzle); the copy of the next block's tile is issued as soon as the current one is in registers.
    const uint32_t sM = sM0 + (uint32_t)q * cfg::MASK_STAGE;
    const uint32_t mbar = m_full((uint32_t)q);
    uint32_t mit = 0;
    auto issue_mask = [&](int q_tile, int j) {
      if (lane == 0) {
        tc::mbar_arrive_expect_tx(mbar, cfg::MASK_STAGE);
        tc::tma_load_4d(sM, &tmM, j * BN, q_tile * BLOCK_M + q * 32, p.mask_h_on ? h : 0, p.mask_z_on ? z : 0, mbar);
      }
    };
    if (MASK && p.mask_tma) issue_mask(tile_of(0), 0);
    HEXB_PROF_DECL(8)
    for (int t = 0; t < p.tiles_per_cta && ok; ++t) {
      const int q_tile = tile_of(t);
      const int n_kv = nkv_of(q_tile);
      const int m0 = q_tile * BLOCK_M;
      const int qi = m0 + r;
      float m_ref = -INFINITY, l = 0.f;
      const int64_t mrow_off = (int64_t)z * p.sm_z + (int64_t)h * p.sm_h + (int64_t)qi * p.sm_q;
      const float *mrow_f32 = static_cast<const float *>(p.mask) + mrow_off;
      const __half *mrow_f16 = static_cast<const __half *>(p.mask) + mrow_off;
      (void)mrow_f32; (void)mrow_f16;
      for (int j = 0; j < n_kv; ++j, ++it) {
        const uint32_t b = it & 1u, ph = (it >> 1) & 1u;
        HEXB_PROF(0)  // loop / epilogue of the previous tile
        if (!tc::mbar_wait(s_full(b), ph, abort_flag)) { ok = false; break; }
        HEXB_PROF(1)  // wait S
        tc::tc_fence_after();
#ifdef HEXB_DEV
        if (p.ablate & 2) {  // hand the block straight back
          tc::tc_fence_before();
          __syncwarp();
          if (PS && it > 0 && !tc::mbar_wait(pv_done, (it - 1u) & 1u, abort_flag)) { ok = false; break; }
          if (lane == 0) {
            if (PS) tc::mbar_arrive(s_free(b));
            tc::mbar_arrive(p_full(PS ? 0u : b));
          }
          continue;
        }
#endif
        const uint32_t tS = tmem_base + b * BN, tP = tS;
        const int kv0 = j * BN;
        const bool need_mask = (p.causal && kv0 + BN - 1 > m0) || (kv0 + BN > p.N_KV);
        uint32_t sv[COLS];
#pragma unroll
        for (int c = 0; c < COLS / 32; ++c)
          tc::tmem_ld_32x32(tS + lane_off + (uint32_t)(c0 + c * 32), reinterpret_cast<uint32_t(&)[32]>(sv[c * 32]));
        tc::tmem_ld_wait();
        if constexpr (PS) {  // the scores are in registers: the buffer may take the next block but one
          tc::tc_fence_before();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(s_free(b));
        }
        HEXB_PROF(2)  // TMEM load of S
        if constexpr (MASK) {
          // sv <- s * sm_scale + mask (natural-log domain; log2(e) goes into the exponent's multiply-add below);
          // rows past the end read no mask.  fp16 mask values are widened by the mixed-precision add itself
          // (add.rn.f32.f16: exact), not by a conversion: conversions run on the unit the exponentials need.
          const float sm_nat = p.scale_log2 * 0.69314718056f;
          const bool row_ok = qi < p.N_CTX;
          if (p.mask_tma) {
            if (!tc::mbar_wait(mbar, mit & 1u, abort_flag)) { ok = false; break; }
            HEXB_PROF(7)  // wait for the mask tile
            ++mit;
            const uint8_t *mrow_s = smem + (sM - smem_addr) + lane * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const uint4 raw = *reinterpret_cast<const uint4 *>(mrow_s + ((c ^ (lane & 7)) << 4));
              add_mask_h2(raw.x, sm_nat, sv[c * 8 + 0], sv[c * 8 + 1]);
              add_mask_h2(raw.y, sm_nat, sv[c * 8 + 2], sv[c * 8 + 3]);
              add_mask_h2(raw.z, sm_nat, sv[c * 8 + 4], sv[c * 8 + 5]);
              add_mask_h2(raw.w, sm_nat, sv[c * 8 + 6], sv[c * 8 + 7]);
            }
            // (Reading the whole row into registers first and starting the next copy before the arithmetic
            // measured slower: 1.196 against 1.170 ms on [4, 32, 4096, 128] with a broadcast mask.)
            __syncwarp();  // every lane has read the tile: the buffer may be refilled
            if (j + 1 < n_kv) issue_mask(q_tile, j + 1);
            else if (t + 1 < p.tiles_per_cta) issue_mask(tile_of(t + 1), 0);
          } else if (p.mask_f32) {
            const float *mp = mrow_f32 + kv0;
            if (j + 1 < n_kv && row_ok) {  // the next block of this row starts inside the row
              asm volatile("prefetch.global.L2 [%0];" ::"l"(mp + BN));
              if (kv0 + BN + 32 < p.N_KV) asm volatile("prefetch.global.L2 [%0];" ::"l"(mp + BN + 32));
            }
            if (row_ok && p.mask_vec_ok && kv0 + BN <= p.N_KV) {
#pragma unroll
              for (int e = 0; e < BN; e += 4) {
                const float4 mv = __ldg(reinterpret_cast<const float4 *>(mp + e));
                sv[e + 0] = __float_as_uint(fmaf(__uint_as_float(sv[e + 0]), sm_nat, mv.x));
                sv[e + 1] = __float_as_uint(fmaf(__uint_as_float(sv[e + 1]), sm_nat, mv.y));
                sv[e + 2] = __float_as_uint(fmaf(__uint_as_float(sv[e + 2]), sm_nat, mv.z));
                sv[e + 3] = __float_as_uint(fmaf(__uint_as_float(sv[e + 3]), sm_nat, mv.w));
              }
            } else {
#pragma unroll
              for (int e = 0; e < BN; ++e) {
                const float mv = (row_ok && kv0 + e < p.N_KV) ? __ldg(mp + e) : 0.f;
                sv[e] = __float_as_uint(fmaf(__uint_as_float(sv[e]), sm_nat, mv));
              }
            }
          } else {
            const __half *mp = mrow_f16 + kv0;
            if (j + 1 < n_kv && row_ok) asm volatile("prefetch.global.L2 [%0];" ::"l"(mp + BN));
            if (row_ok && p.mask_vec_ok && kv0 + BN <= p.N_KV) {
#pragma unroll
              for (int e = 0; e < BN; e += 8) {
                const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(mp + e));
                add_mask_h2(raw.x, sm_nat, sv[e + 0], sv[e + 1]);
                add_mask_h2(raw.y, sm_nat, sv[e + 2], sv[e + 3]);
                add_mask_h2(raw.z, sm_nat, sv[e + 4], sv[e + 5]);
                add_mask_h2(raw.w, sm_nat, sv[e + 6], sv[e + 7]);
              }
            } else {
#pragma unroll
              for (int e = 0; e < BN; ++e) {
                const float mv = (row_ok && kv0 + e < p.N_KV) ? __half2float(__ldg(mp + e)) : 0.f;
                sv[e] = __float_as_uint(fmaf(__uint_as_float(sv[e]), sm_nat, mv));
              }
            }
          }
        }
        if (need_mask) {
#pragma unroll
          for (int e = 0; e < COLS; ++e) {
            const int kv = kv0 + c0 + e;
            if ((p.causal && kv > qi) || kv >= p.N_KV) sv[e] = 0xff800000u;
          }
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int e = 0; e < COLS; e += 8) {
#pragma unroll
          for (int u = 0; u < 4; ++u)
            mx4[u] = max3(mx4[u], __uint_as_float(sv[e + 2 * u]), __uint_as_float(sv[e + 2 * u + 1]));
        }
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * (MASK ? 1.44269504f : p.scale_log2);
        if (TPR == 2) {  // both threads of the row end up with the same maximum
          float other;
          if (!exchange(mx, other)) { ok = false; break; }
          mx = fmaxf(mx, other);
        }
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
          for (int c = 0; c < OCOLS / 32; ++c) {
            uint32_t o[32];
            tc::tmem_ld_32x32(tO + lane_off + (uint32_t)(hsel * OCOLS + c * 32), o);
            tc::tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tc::tmem_st_32x32(tO + lane_off + (uint32_t)(hsel * OCOLS + c * 32), o);
          }
        }
        HEXB_PROF(3)  // mask, max, rescale
        // a row whose keys so far are all masked to -inf keeps m_ref = -inf: its weights must come out 0, not NaN
        const float neg_m = (MASK && m_ref == -INFINITY) ? 0.f : -m_ref;
        const float mul = MASK ? 1.44269504f : p.scale_log2;
        const float2 mul2 = make_float2(mul, mul), neg_m2 = make_float2(neg_m, neg_m);
        float2 lacc0 = make_float2(0.f, 0.f), lacc1 = make_float2(0.f, 0.f);
        if constexpr (PS) {  // the P tile is single: P_{it-1}.V_{it-1} must have read it
          if (it > 0 && !tc::mbar_wait(pv_done, (it - 1u) & 1u, abort_flag)) { ok = false; break; }
        }
#pragma unroll
        for (int c = 0; c < COLS / 32; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            const float2 xa = fma2(make_float2(__uint_as_float(sv[c * 32 + e]), __uint_as_float(sv[c * 32 + e + 1])), mul2, neg_m2);
            const float2 xb = fma2(make_float2(__uint_as_float(sv[c * 32 + e + 2]), __uint_as_float(sv[c * 32 + e + 3])), mul2, neg_m2);
            const float2 pa = make_float2(ex2_approx(xa.x), ex2_approx(xa.y));
            const float2 pb = make_float2(ex2_approx(xb.x), ex2_approx(xb.y));
            lacc0 = add2(lacc0, pa);
            lacc1 = add2(lacc1, pb);
            pk[e >> 1] = pack_f16x2(pa.x, pa.y);
            pk[(e >> 1) + 1] = pack_f16x2(pb.x, pb.y);
          }
          if constexpr (PS) {
            // row r of the P tile: 128 bytes = eight 16-byte pieces, piece i stored at (i ^ (r & 7)) (128-byte swizzle)
            const uint32_t prow = sP + (uint32_t)r * 128u;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t addr = prow + ((uint32_t)((4 * c + i) ^ (r & 7)) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[4 * i]), "r"(pk[4 * i + 1]),
                           "r"(pk[4 * i + 2]), "r"(pk[4 * i + 3])
                           : "memory");
            }
          } else {
            tc::tmem_st_32x16(tP + lane_off + (uint32_t)(c0 / 2 + c * 16), pk);
          }
        }
        l += (lacc0.x + lacc0.y) + (lacc1.x + lacc1.y);
        HEXB_PROF(4)  // exp, pack, TMEM store issue
        if constexpr (PS) {
          tc::fence_proxy_async_smem();   // the tensor pipe reads the tile through the async proxy
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(p_full(0));
        } else {
        tc::tmem_st_wait();
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(p_full(b));
        }
        HEXB_PROF(5)  // store wait + arrive
      }
      if (!ok || !tc::mbar_wait(o_full, (uint32_t)t & 1u, abort_flag)) { ok = false; break; }
      tc::tc_fence_after();
      if (TPR == 2) {  // the two halves of the row sum
        float other;
        if (!exchange(l, other)) { ok = false; break; }
        l += other;
      }
      const float inv = 1.0f / l;
      const int64_t orow_off = (int64_t)z * p.so_z + (int64_t)h * p.so_h + (int64_t)qi * p.so_n + hsel * OCOLS;
      __half *orow = static_cast<__half *>(p.out) + orow_off;
      float *orow32 = static_cast<float *>(p.out) + orow_off;
#pragma unroll 1
      for (int c = 0; c < OCOLS / 32; ++c) {
        uint32_t o[32];
        tc::tmem_ld_32x32(tO + lane_off + (uint32_t)(hsel * OCOLS + c * 32), o);
        tc::tmem_ld_wait();
        if (c == OCOLS / 32 - 1) {
          tc::tc_fence_before();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(o_empty);
        }
        if (qi < p.N_CTX && p.out_f32) {
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            float4 f = make_float4(__uint_as_float(o[g * 4]) * inv, __uint_as_float(o[g * 4 + 1]) * inv,
                                   __uint_as_float(o[g * 4 + 2]) * inv, __uint_as_float(o[g * 4 + 3]) * inv);
            if (p.out_vec_ok) {
              *reinterpret_cast<float4 *>(orow32 + c * 32 + g * 4) = f;
            } else {
              orow32[c * 32 + g * 4] = f.x; orow32[c * 32 + g * 4 + 1] = f.y;
              orow32[c * 32 + g * 4 + 2] = f.z; orow32[c * 32 + g * 4 + 3] = f.w;
            }
          }
        } else if (qi < p.N_CTX) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(o[g * 8 + e]) * inv;
            if (p.out_vec_ok) {
              Vec16<__half> ov;
              ov.pack(f);
              *reinterpret_cast<uint4 *>(orow + c * 32 + g * 8) = ov.raw;
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e) orow[c * 32 + g * 8 + e] = __float2half_rn(f[e]);
            }
          }
        }
      }
      HEXB_PROF(6)  // epilogue
    }
    if (threadIdx.x == 64) { HEXB_PROF_FLUSH(8, 8) }
  }

  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, cfg::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&g_attn_status, (int)HEXB_ERR_TIMEOUT);
}

#ifdef HEXB_ATTN_PROFILE
static unsigned long long *g_attn_prof = nullptr;
extern "C" void hexb_debug_set_attn_profile(void *dev_buf) { g_attn_prof = (unsigned long long *)dev_buf; }
}  // namespace attn
unsigned long long *attn_profile_buffer() { return attn::g_attn_prof; }
namespace attn {
#endif

// CUDA-core forward for fp32 tensors and for shapes the TMA path cannot take: one warp per query
// row, 32 keys per step (one per lane), base-2 online softmax exactly as _attn_fwd_inner writes it
// (running max of scaled scores, alpha = exp2(m_old - m_new)); each lane owns D/32 output columns.
template <typename T, int MAXD>
__global__ void __launch_bounds__(128)
attn_fwd_simt_kernel(const T *__restrict__ Q, const T *__restrict__ K, const T *__restrict__ V,
                     T *__restrict__ O, int Z, int H, int N_CTX, int D, const int64_t sq_z,
                     const int64_t sq_h, const int64_t sq_n, const int64_t sk_z, const int64_t sk_h,
                     const int64_t sk_n, const int64_t sv_z, const int64_t sv_h, const int64_t sv_n,
                     const int64_t so_z, const int64_t so_h, const int64_t so_n, float scale_log2,
                     int causal, int N_KV, int out_f32, const void *__restrict__ mask, int mask_f32,
                     const int64_t sm_z, const int64_t sm_h, const int64_t sm_q) {
  constexpr int DPL = MAXD / 32;  // output columns per lane
  __shared__ float qs[4][MAXD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row_id = (int64_t)blockIdx.x * 4 + warp;
  const int64_t total = (int64_t)Z * H * N_CTX;
  if (row_id >= total) return;
  const int qi = (int)(row_id % N_CTX);
  const int h = (int)((row_id / N_CTX) % H);
  const int z = (int)(row_id / ((int64_t)N_CTX * H));
  const T *qp = Q + z * sq_z + h * sq_h + (int64_t)qi * sq_n;
  const T *kp = K + z * sk_z + h * sk_h;
  const T *vp = V + z * sv_z + h * sv_h;
  for (int d = lane; d < D; d += 32) qs[warp][d] = to_f32<T>(qp[d]);
  __syncwarp();
  float acc[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  const int kv_end = (causal && qi + 1 < N_KV) ? qi + 1 : N_KV;
  const int64_t mrow = z * sm_z + h * sm_h + (int64_t)qi * sm_q;
  for (int kv0 = 0; kv0 < kv_end; kv0 += 32) {
    const int kv = kv0 + lane;
    float s = -INFINITY;
    if (kv < kv_end) {
      const T *kr = kp + (int64_t)kv * sk_n;
      float dot = 0.f;
      for (int d = 0; d < D; ++d) dot = fmaf(qs[warp][d], to_f32<T>(kr[d]), dot);
      s = dot * scale_log2;
      if (mask) {
        const float mv = mask_f32 ? static_cast<const float *>(mask)[mrow + kv]
                                  : __half2float(static_cast<const __half *>(mask)[mrow + kv]);
        s = fmaf(mv, 1.44269504f, s);
      }
    }
    const float m_raw = fmaxf(m, warp_max(s));
    // every key so far masked out: this step's weights are 0, not NaN.  A row whose keys are ALL masked
    // ends with l == 0 and the final acc * (1 / l) = 0 * inf is NaN, as on the tensor-core path and as the
    // reference's exp(-inf - -inf).
    const float m_new = m_raw == -INFINITY ? 0.f : m_raw;
    const float pe = (kv < kv_end) ? exp2f(s - m_new) : 0.f;
    const float alpha = exp2f(m - m_new);  // m == -inf on the first step: alpha = 0, acc and l are 0
    l = l * alpha + warp_sum(pe);
    m = m_raw;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] *= alpha;
    const int nvalid = kv_end - kv0 < 32 ? kv_end - kv0 : 32;
    for (int t = 0; t < nvalid; ++t) {
      const float pt = __shfl_sync(0xffffffffu, pe, t);
      const T *vr = vp + (int64_t)(kv0 + t) * sv_n;
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const int d = lane + i * 32;
        if (d < D) acc[i] = fmaf(pt, to_f32<T>(vr[d]), acc[i]);
      }
    }
  }
  const int64_t ooff = z * so_z + h * so_h + (int64_t)qi * so_n;
  const float inv = 1.0f / l;
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int d = lane + i * 32;
    if (d < D) {
      if (out_f32) reinterpret_cast<float *>(O)[ooff + d] = acc[i] * inv;
      else O[ooff + d] = from_f32<T>(acc[i] * inv);
    }
  }
}

template <typename T>
static int launch_simt(const T *Q, const T *K, const T *V, void *O, int64_t Z, int64_t H, int64_t N,
                       int64_t D, const int64_t *s, float scale_log2, int causal, const Extra &x,
                       cudaStream_t st) {
  if (D > 256) return HEXB_ERR_UNSUPPORTED;
  const int64_t rows = Z * H * N;
  const int64_t ctas = (rows + 3) / 4;
  if (ctas > 0x7fffffffll) return HEXB_ERR_UNSUPPORTED;
  const int of32 = (sizeof(T) == 4) ? 1 : x.out_f32;
#define HEXB_SIMT_LAUNCH(MAXD)                                                                              \
  attn_fwd_simt_kernel<T, MAXD><<<(unsigned)ctas, 128, 0, st>>>(                                            \
      Q, K, V, static_cast<T *>(O), (int)Z, (int)H, (int)N, (int)D, s[0], s[1], s[2], s[3], s[4], s[5], s[6], \
      s[7], s[8], s[9], s[10], s[11], scale_log2, causal, (int)x.n_kv, of32, x.mask, x.mask_f32, x.sm[0],    \
      x.sm[1], x.sm[2])
  if (D <= 64) HEXB_SIMT_LAUNCH(64);
  else if (D <= 128) HEXB_SIMT_LAUNCH(128);
  else HEXB_SIMT_LAUNCH(256);
#undef HEXB_SIMT_LAUNCH
  return check_launch("attn_simt");
}

template <int HD>
static int launch_tc(const __half *Q, const __half *K, const __half *V, void *O, int64_t Z, int64_t H,
                     int64_t N, const int64_t *s, float scale_log2, int causal, const Extra &x, cudaStream_t st) {
  using cfg = Cfg<HD>;
  // 2: 64-key blocks, two score buffers; 1: 128-key blocks (plain calls only)
  const bool plain = !x.mask && !x.out_f32 && x.n_kv == N;
  const int which = (int)option(OPT_attn_kernel, 0);
  const bool two_buffers = !plain || which != 1;
  const bool wide = two_buffers && !x.mask && which == 5;  // 128-key blocks, one CTA per SM
  const bool two_per_row = two_buffers && !x.mask && which == 9;  // 64-key blocks, two softmax threads per row
  const bool p_smem = two_buffers && !x.mask && which == 10;      // 64-key blocks, P through shared memory
  const bool k3 = two_buffers && !x.mask && which == 11;          // 64-key blocks, three K stages
  CUtensorMap tm[4];
  const __half *base[3] = {Q, K, V};
  for (int i = 0; i < 3; ++i) {
    const uint64_t dims[4] = {(uint64_t)HD, (uint64_t)(i == 0 ? N : x.n_kv), (uint64_t)H, (uint64_t)Z};
    const uint64_t strides[3] = {(uint64_t)s[3 * i + 2] * 2, (uint64_t)s[3 * i + 1] * 2,
                                 (uint64_t)s[3 * i + 0] * 2};
    const uint32_t box[4] = {64, (i > 0 && two_buffers && !wide) ? 64u : 128u, 1, 1};  // rows per K/V load
    if (int e = encode_tmap_f16_sw128(&tm[i], base[i], 4, dims, strides, box)) return e;
  }
  static PerDeviceOnce attr_done;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done.is_done(dev)) {
    HEXB_CUDA_OK(cudaFuncSetAttribute(attn_fwd_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg::SMEM_BYTES));
    HEXB_CUDA_OK(cudaFuncSetAttribute(attn_fwd_tc2_kernel<HD, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Cfg2<HD>::SMEM_BYTES));
    HEXB_CUDA_OK(cudaFuncSetAttribute(attn_fwd_tc2_kernel<HD, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Cfg2<HD>::SMEM_BYTES_MASK));
    HEXB_CUDA_OK(cudaFuncSetAttribute(attn_fwd_tc2_kernel<HD, false, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Cfg2<HD, 128>::SMEM_BYTES));
    HEXB_CUDA_OK(cudaFuncSetAttribute(attn_fwd_tc2_kernel<HD, false, 64, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Cfg2<HD>::SMEM_BYTES));
    HEXB_CUDA_OK(cudaFuncSetAttribute(attn_fwd_tc2_kernel<HD, false, 64, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Cfg2<HD>::SMEM_BYTES_PS));
    HEXB_CUDA_OK(cudaFuncSetAttribute(attn_fwd_tc2_kernel<HD, false, 64, 1, false, true>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg2<HD>::SMEM_BYTES_PS));
    attr_done.mark(dev);
  }
  Params p;
#ifdef HEXB_ATTN_PROFILE
  p.prof = g_attn_prof;
#endif
  p.out = O;
  p.so_z = s[9]; p.so_h = s[10]; p.so_n = s[11];
  p.Z = (int)Z; p.H = (int)H; p.N_CTX = (int)N;
  p.N_KV = (int)x.n_kv;
  p.out_f32 = x.out_f32;
  p.mask = x.mask;
  p.mask_f32 = x.mask_f32;
  p.sm_z = x.sm[0]; p.sm_h = x.sm[1]; p.sm_q = x.sm[2];
  {
    const int per16 = x.mask_f32 ? 4 : 8;  // mask elements per 16 bytes
    p.mask_vec_ok = x.mask && aligned16(x.mask) && x.sm[0] % per16 == 0 && x.sm[1] % per16 == 0 && x.sm[2] % per16 == 0;
  }
  p.mask_h_on = x.sm[1] != 0;
  p.mask_z_on = x.sm[0] != 0;
  p.head_major = (x.mask && p.mask_h_on && !p.mask_z_on && Z > 1) ? 1 : 0;
  p.mask_tma = p.mask_vec_ok && !x.mask_f32 && x.sm[2] >= x.n_kv && option(OPT_attn_mask_tma, 1);
  tm[3] = tm[0];
  if (p.mask_tma) {
    // a broadcast dimension becomes an extent of 1 (its stride is then never applied)
    const uint64_t row = (uint64_t)x.sm[2] * 2;
    const uint64_t dims[4] = {(uint64_t)x.n_kv, (uint64_t)N, (uint64_t)(p.mask_h_on ? H : 1),
                              (uint64_t)(p.mask_z_on ? Z : 1)};
    const uint64_t strides[3] = {row, p.mask_h_on ? (uint64_t)x.sm[1] * 2 : row * (uint64_t)N,
                                 p.mask_z_on ? (uint64_t)x.sm[0] * 2 : row * (uint64_t)N};
    const uint32_t box[4] = {64, 32, 1, 1};
    if (encode_tmap_f16_sw128(&tm[3], x.mask, 4, dims, strides, box) != HEXB_OK) {
      p.mask_tma = 0;  // a layout the tensor map cannot describe: the softmax warps load the mask themselves
      tm[3] = tm[0];
    }
  }
  p.num_q_tiles = (int)((N + BLOCK_M - 1) / BLOCK_M);
  p.scale_log2 = scale_log2;
  p.causal = causal ? 1 : 0;
  {
    const int per16 = x.out_f32 ? 4 : 8;
    p.out_vec_ok = aligned16(O) && s[9] % per16 == 0 && s[10] % per16 == 0 && s[11] % per16 == 0;
  }
  p.v_lbo = (uint32_t)HEXB_DEV_OPTION(OPT_attn_v_lbo, cfg::CHUNK_BYTES);
  p.v_sbo = (uint32_t)HEXB_DEV_OPTION(OPT_attn_v_sbo, 1024);
#ifdef HEXB_DEV
  p.ablate = (int)option(OPT_attn_ablate, 0);
#endif
  // Pairing a long and a short tile pays when the tiles differ in length (causal) and the pairs still
  // give every SM a CTA; equal tiles run slightly faster one per CTA, and a grid of fewer pairs than SMs
  // is better off with twice as many CTAs ([1, 16, 1024, 128] causal: 30.6 us paired, 23.9 us unpaired).
  // attn_tiles_per_cta = 1 or 2 forces one or the other.
  {
    DeviceInfo di;
    if (int e = current_device(&di)) return e;
    const int64_t pairs = (int64_t)(p.num_q_tiles / 2) * Z * H;
    const int want = option(OPT_attn_tiles_per_cta, 0);
    const bool pair = want == 2 || (want != 1 && causal && pairs >= di.sm_count);
    p.tiles_per_cta = (p.num_q_tiles % 2 == 0 && pair) ? 2 : 1;
  }
  p.ctas_per_bh = p.num_q_tiles / p.tiles_per_cta;
  const int64_t ctas = (int64_t)p.ctas_per_bh * Z * H;
  if (ctas > 0x7fffffffll) return HEXB_ERR_UNSUPPORTED;
  if (wide)
    launch_pdl(attn_fwd_tc2_kernel<HD, false, 128>, dim3((unsigned)ctas), dim3(THREADS), (size_t)Cfg2<HD, 128>::SMEM_BYTES, st,
               tm[0], tm[1], tm[2], tm[3], p);
  else if (k3)
    launch_pdl(attn_fwd_tc2_kernel<HD, false, 64, 1, false, true>, dim3((unsigned)ctas), dim3(THREADS), (size_t)Cfg2<HD>::SMEM_BYTES_PS,
               st, tm[0], tm[1], tm[2], tm[3], p);
  else if (p_smem)
    launch_pdl(attn_fwd_tc2_kernel<HD, false, 64, 1, true>, dim3((unsigned)ctas), dim3(224), (size_t)Cfg2<HD>::SMEM_BYTES_PS, st,
               tm[0], tm[1], tm[2], tm[3], p);
  else if (two_per_row)
    launch_pdl(attn_fwd_tc2_kernel<HD, false, 64, 2>, dim3((unsigned)ctas), dim3(64 + 128 * 2), (size_t)Cfg2<HD>::SMEM_BYTES, st,
               tm[0], tm[1], tm[2], tm[3], p);
  else if (two_buffers && x.mask)
    launch_pdl(attn_fwd_tc2_kernel<HD, true>, dim3((unsigned)ctas), dim3(THREADS), (size_t)Cfg2<HD>::SMEM_BYTES_MASK, st,
               tm[0], tm[1], tm[2], tm[3], p);
  else if (two_buffers)
    launch_pdl(attn_fwd_tc2_kernel<HD, false>, dim3((unsigned)ctas), dim3(THREADS), (size_t)Cfg2<HD>::SMEM_BYTES, st, tm[0],
               tm[1], tm[2], tm[3], p);
  else
    attn_fwd_tc_kernel<HD><<<(unsigned)ctas, THREADS, cfg::SMEM_BYTES, st>>>(tm[0], tm[1], tm[2], p);
  return check_launch("attn_tc");
}

}  // namespace attn

int attn_device_status_fetch_and_clear(int *out) {
  int v = 0, zero = 0, v3 = 0;
  HEXB_CUDA_OK(cudaMemcpyFromSymbol(&v, g_attn_status, sizeof(int)));
  if (v) HEXB_CUDA_OK(cudaMemcpyToSymbol(g_attn_status, &zero, sizeof(int)));
  if (int e = attn_pingpong_status_fetch_and_clear(&v3)) return e;
  int v4 = 0, v5 = 0;
  if (int e = attn_wide_status_fetch_and_clear(&v4)) return e;
  if (int e = attn_tf32_status_fetch_and_clear(&v5)) return e;
  if (!v3) v3 = v4 ? v4 : v5;
  *out = v ? v : v3;
  return HEXB_OK;
}

static int attn_check(const void *Q, const void *K, const void *V, void *O, int64_t Z, int64_t H,
                      int64_t N, int64_t D, const int64_t *s, float scale) {
  if (Z < 0 || H < 0 || N < 0 || D < 0) return HEXB_ERR_BAD_ARG;
  if (Z == 0 || H == 0 || N == 0 || D == 0) return 1;  // nothing to do
  if (!Q || !K || !V || !O || !s) return HEXB_ERR_BAD_ARG;
  if (!(scale > 0.f)) return HEXB_ERR_BAD_ARG;
  for (int i = 0; i < 12; ++i)
    if (s[i] < 0) return HEXB_ERR_BAD_ARG;
  for (int t = 0; t < 4; ++t)
    if (s[3 * t + 2] < D) return HEXB_ERR_BAD_ARG;
  if (N >= (1ll << 31) || H >= (1ll << 31) || Z >= (1ll << 31)) return HEXB_ERR_UNSUPPORTED;
  return HEXB_OK;
}

}  // namespace hexb

namespace hexb {
// fp32 tensors.  The tensor-core kernel (kind::tf32) rounds the operands to 10 mantissa bits: its result is
// inside the benchmark's 1e-3 bar for fp32 kernels but not inside the reference test's torch.allclose defaults,
// and the CUDA-core kernel is exact but runs at about 1 TFLOP/s.  Option attn_f32_tensor: 0 = the tensor
// cores from 2^30 multiply-adds on (where the exact kernel would take milliseconds), 1 = never, 2 = always.
static int attention_f32_dispatch(const float *Q, const float *K, const float *V, float *Out, int64_t Z, int64_t H,
                                  int64_t N, int64_t D, const int64_t *s, float sm_scale, int causal, const attn::Extra &x,
                                  cudaStream_t st) {
  DeviceInfo di;
  if (int e = current_device(&di)) return e;
  const int mode = option(OPT_attn_f32_tensor, 0);
  const double macs = (double)Z * H * N * x.n_kv * D * (causal ? 0.5 : 1.0);
  if (!x.mask && mode != 1 && (mode == 2 || macs >= 1073741824.0) && !option(OPT_attn_force_simt, 0) &&
      aligned16(Out) && attn_tf32_supported(Q, K, V, D, s))
    return attn_tf32_launch(Q, K, V, Out, Z, H, N, x.n_kv, D, s, sm_scale * 1.44269504f, causal, st);
  return attn::launch_simt<float>(Q, K, V, Out, Z, H, N, D, s, sm_scale * 1.44269504f, causal, x, st);
}

// Shared body of the fp16-input entry points.
static int attention_f16_dispatch(const void *Q, const void *K, const void *V, void *Out, int64_t Z, int64_t H,
                                  int64_t N, int64_t D, const int64_t *s, float sm_scale, int causal,
                                  const attn::Extra &x, cudaStream_t st) {
  DeviceInfo di;
  if (int e = current_device(&di)) return e;
  const float scale_log2 = sm_scale * 1.44269504f;
  bool tma_ok = (D == 64 || D == 128) && !option(OPT_attn_force_simt, 0) && aligned16(Q) && aligned16(K) &&
                aligned16(V);
  for (int i = 0; i < 9 && tma_ok; ++i) tma_ok = s[i] % 8 == 0 && s[i] > 0;
  // attn_kernel: 0 or 2 = 64-key blocks with two score buffers (the default), 1 = 128-key blocks / one score
  // buffer, 3 / 4 = two query tiles per persistent CTA taking turns with one / two softmax threads per row
  // (attention_pingpong.cu), 5 = 128-key blocks / two score buffers / one CTA per SM, 6-8 = attention_wide.cu,
  // 9 = the default with two softmax threads per row, 10 = the default with P handed over through shared memory,
  // 11 = the default with three K stages
  const int which = (int)option(OPT_attn_kernel, 0);
  const bool plain = !x.mask && x.n_kv == N;
  if (tma_ok && plain && (which == 6 || which == 7 || which == 8))   // attention_wide.cu: 2 or 4 softmax threads per row (6, 7),
    return attn_wide_launch((const __half *)Q, (const __half *)K, (const __half *)V, Out, Z, H, N, D, s, scale_log2, causal,
                            x.out_f32, which == 6 ? 2 : which == 7 ? 4 : 1, st);       // or two warpgroups taking turns on the blocks (8)
  if (tma_ok && plain && (which == 3 || which == 4) && attn_pingpong_supported(Z, H, N, D, causal, di.sm_count))
    return attn_pingpong_launch((const __half *)Q, (const __half *)K, (const __half *)V, Out, Z, H, N, D, s, scale_log2,
                                causal, x.out_f32, which == 4 ? 2 : 1, st);
  if (tma_ok) {
    if (D == 128)
      return attn::launch_tc<128>((const __half *)Q, (const __half *)K, (const __half *)V, Out, Z, H, N, s,
                                  scale_log2, causal, x, st);
    return attn::launch_tc<64>((const __half *)Q, (const __half *)K, (const __half *)V, Out, Z, H, N, s,
                               scale_log2, causal, x, st);
  }
  return attn::launch_simt<__half>((const __half *)Q, (const __half *)K, (const __half *)V, Out, Z, H, N, D, s,
                                   scale_log2, causal, x, st);
}
}  // namespace hexb

extern "C" int hexb_attention_fwd_f16(const void *Q, const void *K, const void *V, void *Out, int64_t Z,
                                      int64_t H, int64_t N, int64_t D, const int64_t *s, float sm_scale,
                                      int causal, void *stream) {
  using namespace hexb;
  const int c = attn_check(Q, K, V, Out, Z, H, N, D, s, sm_scale);
  if (c == 1) return HEXB_OK;
  if (c) return c;
  const attn::Extra x = {N, 0, nullptr, 0, {0, 0, 0}};
  return attention_f16_dispatch(Q, K, V, Out, Z, H, N, D, s, sm_scale, causal, x, (cudaStream_t)stream);
}

extern "C" int hexb_attention_fwd_f32(const float *Q, const float *K, const float *V, float *Out,
                                      int64_t Z, int64_t H, int64_t N, int64_t D, const int64_t *s,
                                      float sm_scale, int causal, void *stream) {
  using namespace hexb;
  const int c = attn_check(Q, K, V, Out, Z, H, N, D, s, sm_scale);
  if (c == 1) return HEXB_OK;
  if (c) return c;
  const attn::Extra x = {N, 1, nullptr, 0, {0, 0, 0}};
  return attention_f32_dispatch(Q, K, V, Out, Z, H, N, D, s, sm_scale, causal, x, (cudaStream_t)stream);
}

extern "C" int hexb_attention_fwd_ex(const hexb_attention_desc *d, void *stream) {
  using namespace hexb;
  if (!d) return HEXB_ERR_BAD_ARG;
  if (d->in_dtype != HEXB_DT_F16 && d->in_dtype != HEXB_DT_F32) return HEXB_ERR_UNSUPPORTED;
  if (d->out_dtype != HEXB_DT_F16 && d->out_dtype != HEXB_DT_F32) return HEXB_ERR_UNSUPPORTED;
  if (d->in_dtype == HEXB_DT_F32 && d->out_dtype != HEXB_DT_F32) return HEXB_ERR_UNSUPPORTED;
  if (d->mask && d->mask_dtype != HEXB_DT_F16 && d->mask_dtype != HEXB_DT_F32) return HEXB_ERR_UNSUPPORTED;
  if (d->N_KV < 0) return HEXB_ERR_BAD_ARG;
  const int c = attn_check(d->Q, d->K, d->V, d->Out, d->Z, d->H, d->N_Q, d->D, d->strides, d->sm_scale);
  if (c == 1) return HEXB_OK;
  if (c) return c;
  if (d->N_KV == 0) return HEXB_ERR_BAD_ARG;  // a softmax over no keys has no value
  if (d->N_KV >= (1ll << 31)) return HEXB_ERR_UNSUPPORTED;
  attn::Extra x = {d->N_KV, d->out_dtype == HEXB_DT_F32 ? 1 : 0, d->mask, d->mask_dtype == HEXB_DT_F32 ? 1 : 0,
                   {d->mask_strides[0], d->mask_strides[1], d->mask_strides[2]}};
  if (d->mask) {
    for (int i = 0; i < 3; ++i)
      if (x.sm[i] < 0) return HEXB_ERR_BAD_ARG;
    if (d->N_Q > 1 && x.sm[2] != 0 && x.sm[2] < d->N_KV) return HEXB_ERR_BAD_ARG;
  }
  cudaStream_t st = (cudaStream_t)stream;
  if (d->in_dtype == HEXB_DT_F16)
    return attention_f16_dispatch(d->Q, d->K, d->V, d->Out, d->Z, d->H, d->N_Q, d->D, d->strides, d->sm_scale,
                                  d->causal, x, st);
  return attention_f32_dispatch((const float *)d->Q, (const float *)d->K, (const float *)d->V, (float *)d->Out, d->Z, d->H,
                                d->N_Q, d->D, d->strides, d->sm_scale, d->causal, x, st);
}
