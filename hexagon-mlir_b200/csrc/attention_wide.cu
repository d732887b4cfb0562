// Flash-attention forward, fourth form: one 128-row query tile per persistent CTA, 128-key blocks, two
// score buffers, and SEVERAL threads per query row in the softmax.
//
// Reference semantics as in attention.cu: attention_fwd_kernel + _attn_fwd_inner
// (test/python/triton/test_flash_attention.py:37-168), the fp16 MLIR form
// (test/python/mlir/hexkl_attention/input.mlir:5-168, P truncated to fp16 before P.V), causal = the
// -inf mask of tm_tensor.attention (lib/Transforms/LowerTmTensor.cpp:70-235).
//
// What the measurements of the other forms say (B200, clock counters inside the kernels):
//   * a 128x64x16 Q.K^T MMA takes 48.7 clocks instead of 32 because it re-reads 4 KiB of Q for 2 KiB of
//     K from shared memory; 128x128x16 runs at the full 64 -- so key blocks should be 128 wide;
//   * with ONE score buffer per tile (P aliases S) every block pays the hand-off chain
//     Q.K^T -> softmax -> P.V -> Q.K^T, about 250 clocks from tcgen05.commit to the waiting thread each
//     way, which two tiles per SM do not hide -- so the scores should be double-buffered;
//   * two 128-key score buffers (256 TMEM columns) plus O (128) leave room for one tile per SM, and with
//     one thread per row its four softmax warps -- one per scheduler, each row 128 exponentials deep --
//     set the pace (947 TFLOP/s on [4, 32, 4096, 128]).
// Here the row is split over TPR threads (warps w, w+4, ... share a TMEM lane quarter and take BN / TPR
// columns each), so the load, the row maximum, the packing and the stores shrink by TPR while the
// exponentials stay bound by the special-function unit.  The threads of a row agree on the running maximum
// through shared memory and an mbarrier per lane quarter; each keeps a partial row sum that is
// combined in the epilogue.
//
//   TMEM (512 columns allocated)  S0 [0,128)  S1 [128,256)  [S2 [256,384)]  O behind them;  P_b = fp16 over S_b[0,64)
//   warp 0   TMA: Q per tile; K_j and V_j through rings of three and two 128-row stages, K ahead of V
//   warp 1   MMA: S_{j+1} = Q.K_{j+1}^T is issued before P_j is waited for, then O += P_j.V_j
//   warps 2 .. 2+4*TPR-1   softmax / correction / epilogue
// The CTA is persistent (one per SM) and walks work items; a causal item is a late and an early tile so
// that all items cost the same.  Plain calls only (no additive mask, equal query and key lengths).
// Every mbarrier wait is bounded; no load uses cluster multicast.
#include "attn_common.cuh"

namespace hexb {

static __device__ int g_attn4_status = 0;

namespace attn4 {

using namespace attn;

constexpr int BLOCK_M = 128;
constexpr int BN = 128;
constexpr int KSTAGES = 3;     // K tiles in flight (Q.K^T runs up to two blocks ahead of P.V)
constexpr int VSTAGES = 2;     // V tiles in flight
constexpr int STAGES = KSTAGES + VSTAGES;

template <int HD, int TPR>
struct Cfg {
  static constexpr int THREADS = 64 + 128 * TPR;
  static constexpr int CHUNKS = HD / 64;
  static constexpr int TILE_BYTES = 128 * HD * 2;   // the Q tile, or one K / V stage
  static constexpr int CHUNK_BYTES = 128 * 128;
  static constexpr int XCHG_BYTES = 4 * TPR * 128 * 4;   // row maxima [block parity][column group][row], then row sums [column group][row]
  static constexpr int NBAR = 32;
  static constexpr int SMEM_BYTES = (1 + STAGES) * TILE_BYTES + XCHG_BYTES + NBAR * 8 + 16 + 1024;
  static constexpr int TMEM_COLS = 512;
  static constexpr int O_COL = 256;
  static constexpr int COLS = BN / TPR;             // score columns per thread
  static constexpr int OCOLS = HD / TPR;            // output columns per thread
};

struct Params {
#ifdef HEXB_ATTN_PROFILE
  unsigned long long *prof;
#endif
  void *out;
  int64_t so_z, so_h, so_n;
  int H, N_CTX;
  int out_f32, out_vec_ok;
  int num_q_tiles;
  int tiles_per_item;   // 1, or 2 (causal: a late and an early tile)
  int items_per_bh;
  int num_items;
  float scale_log2;
  int causal;
};


template <int HD, int TPR, bool ALT>
__global__ void __launch_bounds__(Cfg<HD, TPR>::THREADS, 1)
attn_fwd_wide_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const Params p) {
  using cfg = Cfg<HD, TPR>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw_addr = tc::smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
  uint8_t *smem = smem_raw + pad;
  const uint32_t smem_addr = raw_addr + pad;
  const uint32_t sQ = smem_addr;
  const uint32_t sKV0 = sQ + cfg::TILE_BYTES;
  float *xchg = reinterpret_cast<float *>(smem + (1 + STAGES) * cfg::TILE_BYTES);
  const uint32_t bar0 = sKV0 + STAGES * cfg::TILE_BYTES + cfg::XCHG_BYTES;
  const uint32_t q_full = bar0, q_empty = bar0 + 8, o_full = bar0 + 16, o_empty = bar0 + 24, pv_done = bar0 + 32;
  // score buffers: two (the softmax of block j runs while Q.K^T of block j+1 is in the pipe), or three when two
  // warpgroups take turns on the blocks -- each then needs its NEXT block's scores, two blocks ahead, while it
  // works, so the MMA thread runs two blocks ahead of the softmax
  constexpr uint32_t NSB = ALT ? 3 : 2;
  auto s_full = [&](uint32_t b) { return bar0 + 40 + 8u * b; };
  auto p_full = [&](uint32_t b) { return bar0 + 64 + 8u * b; };
  // K and V have rings of their own (stages 0 .. KSTAGES-1 and KSTAGES .. STAGES-1): a K tile is needed up to two
  // blocks before the V tile of the same block, and in one ring its load would queue behind V loads that wait
  // for earlier products to retire
  auto kv_full = [&](uint32_t s) { return bar0 + 88 + 8u * s; };
  auto kv_empty = [&](uint32_t s) { return bar0 + 128 + 8u * s; };
  auto x_bar = [&](int q) { return bar0 + 168 + 8u * (uint32_t)q; };
  auto l_bar = [&](int q) { return bar0 + 200 + 8u * (uint32_t)q; };   // ends at bar0 + 232 = 29 barriers
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + (1 + STAGES) * cfg::TILE_BYTES + cfg::XCHG_BYTES + 240);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kv_blocks = (p.N_CTX + BN - 1) / BN;
  // item w: (batch, head) w / items_per_bh, rank w % items_per_bh; its i-th tile
  auto tile_of = [&](int rank, int i) {
    if (p.tiles_per_item == 2) return i == 0 ? p.num_q_tiles - 1 - rank : rank;
    return rank;
  };
  auto nkv_of = [&](int q_tile) { return (p.causal && q_tile + 1 < kv_blocks) ? q_tile + 1 : kv_blocks; };

  if (threadIdx.x == 0) {
    tc::mbar_init(q_full, 1);
    tc::mbar_init(q_empty, 1);
    tc::mbar_init(o_full, 1);
    tc::mbar_init(o_empty, 4 * TPR);
    tc::mbar_init(pv_done, 1);
    for (uint32_t b = 0; b < NSB; ++b) {
      tc::mbar_init(s_full(b), 1);
      tc::mbar_init(p_full(b), ALT ? 4 : 4 * TPR);
    }
    for (uint32_t s = 0; s < STAGES; ++s) {
      tc::mbar_init(kv_full(s), 1);
      tc::mbar_init(kv_empty(s), 1);
    }
    for (int q = 0; q < 4; ++q) {
      tc::mbar_init(x_bar(q), ALT ? 1 : TPR);   // column split: one arrival per warp of the lane quarter; alternating: the block's warp
      tc::mbar_init(l_bar(q), 2);
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
  const uint32_t tO = tmem_base + NSB * BN;   // O sits behind the score buffers

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t kc = 0, vc = 0, tiles_done = 0;   // K and V tiles loaded so far
      bool ok = true;
      constexpr int LA = ALT ? 2 : 1;            // K runs this many blocks ahead of V, as the MMA thread consumes them
      for (int w = blockIdx.x; w < p.num_items && ok; w += gridDim.x) {
        const int bh = w / p.items_per_bh, rank = w - bh * p.items_per_bh;
        const int z = bh / p.H, h = bh - z * p.H;
        auto load_k = [&](int j) {
          const uint32_t s = kc % KSTAGES, ph = (kc / KSTAGES) & 1u;
          ++kc;
          if (!tc::mbar_wait(kv_empty(s), ph ^ 1u, abort_flag)) return false;
          tc::mbar_arrive_expect_tx(kv_full(s), cfg::TILE_BYTES);
#pragma unroll
          for (int c = 0; c < cfg::CHUNKS; ++c)
            tc::tma_load_4d(sKV0 + s * cfg::TILE_BYTES + c * cfg::CHUNK_BYTES, &tmK, c * 64, j * BN, h, z, kv_full(s));
          return true;
        };
        auto load_v = [&](int j) {
          const uint32_t s = KSTAGES + vc % VSTAGES, ph = (vc / VSTAGES) & 1u;
          ++vc;
          if (!tc::mbar_wait(kv_empty(s), ph ^ 1u, abort_flag)) return false;
          tc::mbar_arrive_expect_tx(kv_full(s), cfg::TILE_BYTES);
#pragma unroll
          for (int c = 0; c < cfg::CHUNKS; ++c)
            tc::tma_load_4d(sKV0 + s * cfg::TILE_BYTES + c * cfg::CHUNK_BYTES, &tmV, c * 64, j * BN, h, z, kv_full(s));
          return true;
        };
        for (int i = 0; i < p.tiles_per_item && ok; ++i, ++tiles_done) {
          const int q_tile = tile_of(rank, i);
          const int n_kv = nkv_of(q_tile);
          // the previous tile's last Q.K^T has read Q
          if (tiles_done > 0 && !tc::mbar_wait(q_empty, (tiles_done - 1u) & 1u, abort_flag)) { ok = false; break; }
          tc::mbar_arrive_expect_tx(q_full, cfg::TILE_BYTES);
#pragma unroll
          for (int c = 0; c < cfg::CHUNKS; ++c)
            tc::tma_load_4d(sQ + c * cfg::CHUNK_BYTES, &tmQ, c * 64, q_tile * BLOCK_M, h, z, q_full);
          for (int a = 0; a < LA && a < n_kv && ok; ++a) ok = load_k(a);
          for (int j = 0; j < n_kv && ok; ++j) {
            if (j + LA < n_kv) ok = load_k(j + LA);
            if (ok) ok = load_v(j);
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
      uint32_t kbase = 0;       // K tiles (= V tiles = key blocks) of the tiles before the current one
      uint32_t blk = 0;         // key blocks issued so far (score buffer = blk % NSB)
      uint32_t tiles_done = 0;
      auto k_stage = [&](uint32_t kc) { return kc % KSTAGES; };
      auto v_stage = [&](uint32_t vc) { return KSTAGES + vc % VSTAGES; };
      auto wait_k = [&](uint32_t kc) { return tc::mbar_wait(kv_full(k_stage(kc)), (kc / KSTAGES) & 1u, abort_flag); };
      auto wait_v = [&](uint32_t vc) { return tc::mbar_wait(kv_full(v_stage(vc)), (vc / VSTAGES) & 1u, abort_flag); };
      // S_b = Q . K^T with K tile number kc
      auto issue_qk = [&](uint32_t b, uint32_t kc, bool last_of_tile) {
        const uint32_t sK = sKV0 + k_stage(kc) * cfg::TILE_BYTES;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (uint32_t)((k >> 2) * cfg::CHUNK_BYTES + (k & 3) * 32);
          tc::mma_f16_ss(tmem_base + b * BN, tc::make_smem_desc_sw128(sQ + off, 16, 1024),
                         tc::make_smem_desc_sw128(sK + off, 16, 1024), idesc_qk, k != 0 ? 1u : 0u);
        }
        tc::mma_commit(s_full(b));
        tc::mma_commit(kv_empty(k_stage(kc)));
        if (last_of_tile) tc::mma_commit(q_empty);
      };
      for (int w = blockIdx.x; w < p.num_items && ok; w += gridDim.x) {
        const int rank = w % p.items_per_bh;
        for (int i = 0; i < p.tiles_per_item && ok; ++i, ++tiles_done) {
          const int n_kv = nkv_of(tile_of(rank, i));
          if (!tc::mbar_wait(q_full, tiles_done & 1u, abort_flag)) { ok = false; break; }
          constexpr int LA = (int)NSB - 1;   // key blocks the scores run ahead of the softmax
          for (int a = 0; a < LA && a < n_kv && ok; ++a) {
            if (!wait_k(kbase + (uint32_t)a)) { ok = false; break; }
            tc::tc_fence_after();
            issue_qk((blk + (uint32_t)a) % NSB, kbase + (uint32_t)a, a + 1 == n_kv);
          }
          for (int j = 0; j < n_kv && ok; ++j, ++blk) {
            if (j + LA < n_kv) {
              if (!wait_k(kbase + (uint32_t)(j + LA))) { ok = false; break; }
              tc::tc_fence_after();
              issue_qk((blk + (uint32_t)LA) % NSB, kbase + (uint32_t)(j + LA), j + LA + 1 == n_kv);
            }
            const uint32_t b = blk % NSB, ph = (blk / NSB) & 1u;
            const uint32_t vc = kbase + (uint32_t)j;
            if (!tc::mbar_wait(p_full(b), ph, abort_flag)) { ok = false; break; }
            if (!wait_v(vc)) { ok = false; break; }
            // the first product of a later tile overwrites O: the previous epilogue must have read it
            if (j == 0 && tiles_done > 0 && !tc::mbar_wait(o_empty, (tiles_done - 1u) & 1u, abort_flag)) { ok = false; break; }
            tc::tc_fence_after();
            const uint32_t sV = sKV0 + v_stage(vc) * cfg::TILE_BYTES;
#pragma unroll
            for (int k = 0; k < BN / 16; ++k) {
              // A = P rows from TMEM (16 fp16 = 8 columns per step); B = V: 16 key rows = 2 swizzle atoms
              tc::mma_f16_ts(tO, tmem_base + b * BN + (uint32_t)(k * 8),
                             tc::make_smem_desc_sw128(sV + (uint32_t)(k * 2048), cfg::CHUNK_BYTES, 1024), idesc_pv,
                             (j | k) != 0 ? 1u : 0u);
            }
            tc::mma_commit(kv_empty(v_stage(vc)));
            tc::mma_commit(pv_done);
            if (j == n_kv - 1) tc::mma_commit(o_full);
          }
          kbase += (uint32_t)n_kv;
        }
      }
    }
  } else if constexpr (ALT) {
    // ------------------------------------------------------------ softmax, two warpgroups taking turns on the blocks
    // Warpgroup g (warps 2-5: g = 0, warps 6-9: g = 1) handles the key blocks whose running index has parity g
    // (score buffer = running index mod 3), one query row per thread over all 128 keys.  While one warpgroup
    // exponentiates, the other loads and reduces the next block, so the special-function unit and the
    // rest of the loop overlap.  The online-softmax state crosses between them once per block: the row's
    // reference maximum after block j goes through shared memory (two slots by block parity) with one
    // mbarrier per lane quarter, published before the exponentials and before the rare rescale of O so that
    // the other warpgroup is not held up.  Each warpgroup keeps its own partial row sum at the scale it last saw;
    // the epilogue brings both to the final scale and adds them.
    const int q = warp & 3;
    const int g = (warp - 2) >> 2;
    const int r = q * 32 + lane;
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    constexpr int OCOLS = HD / 2;
    float *mref_sh = xchg;                  // [2][128]: reference maximum after block bg, slot bg & 1
    float *l_sh = xchg + 2 * 128;           // [2 tile parities][2 warpgroups][128]
    uint32_t blk_base = 0, tiles_done = 0;
    bool ok = true;
    HEXB_PROF_DECL(8)
    for (int w = blockIdx.x; w < p.num_items && ok; w += gridDim.x) {
      const int bh = w / p.items_per_bh, rank = w - bh * p.items_per_bh;
      const int z = bh / p.H, h = bh - z * p.H;
      for (int i = 0; i < p.tiles_per_item && ok; ++i, ++tiles_done) {
        const int q_tile = tile_of(rank, i);
        const int n_kv = nkv_of(q_tile);
        const int m0 = q_tile * BLOCK_M;
        const int qi = m0 + r;
        float m_known = -INFINITY, l = 0.f;
        for (int j = 0; j < n_kv; ++j) {
          const uint32_t bg = blk_base + (uint32_t)j;    // running block index: buffer and warpgroup = bg & 1
          if ((int)(bg & 1u) != g) continue;
          const uint32_t b = bg % NSB;
          const uint32_t tS = tmem_base + b * BN, tP = tS;
          HEXB_PROF(0)  // loop / epilogue
          if (!tc::mbar_wait(s_full(b), (bg / NSB) & 1u, abort_flag)) { ok = false; break; }
          HEXB_PROF(1)  // wait S
          tc::tc_fence_after();
          const int kv0 = j * BN;
          const bool need_mask = (p.causal && kv0 + BN - 1 > m0) || (kv0 + BN > p.N_CTX);
          uint32_t sv[BN];
#pragma unroll
          for (int c = 0; c < BN / 32; ++c)
            tc::tmem_ld_32x32(tS + lane_off + (uint32_t)(c * 32), reinterpret_cast<uint32_t(&)[32]>(sv[c * 32]));
          tc::tmem_ld_wait();
          HEXB_PROF(2)  // TMEM load of S
          if (need_mask) {
#pragma unroll
            for (int e = 0; e < BN; ++e) {
              const int kv = kv0 + e;
              if ((p.causal && kv > qi) || kv >= p.N_CTX) sv[e] = 0xff800000u;  // -inf: exp2 gives 0
            }
          }
          float mx8[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) mx8[u] = -INFINITY;
#pragma unroll
          for (int e = 0; e < BN; e += 16) {
#pragma unroll
            for (int u = 0; u < 8; ++u)
              mx8[u] = max3(mx8[u], __uint_as_float(sv[e + 2 * u]), __uint_as_float(sv[e + 2 * u + 1]));
          }
          const float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])),
                                 fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7]))) * p.scale_log2;
          HEXB_PROF(3)  // mask, max
          // the reference maximum the previous block of this tile left (the other warpgroup's block)
          float m_prev = -INFINITY;
          if (j > 0) {
            if (!tc::mbar_wait(x_bar(q), (bg - 1u) & 1u, abort_flag)) { ok = false; break; }
            m_prev = mref_sh[((bg - 1u) & 1u) * 128 + r];
          }
          HEXB_PROF(4)  // wait for the other warpgroup's maximum
          if (m_prev != m_known) {   // the other warpgroup moved the reference: bring the own partial sum along
            l *= ex2_approx(m_known - m_prev);
            m_known = m_prev;
          }
          const float m_new = fmaxf(m_prev, mx);
          const bool grow = j > 0 && __any_sync(0xffffffffu, m_new - m_prev > kRescaleThreshold);
          const float m_ref = (j == 0 || grow) ? m_new : m_prev;
          // published before the exponentials (and before the rare rescale of O): the other warpgroup can go on.
          // Publishing after them instead, so that the two warpgroups take strict turns on the special-function
          // unit, measured the same -- one warp per scheduler cannot saturate that unit by itself
          // (11 clocks per element against 8 with two warps).
          mref_sh[(bg & 1u) * 128 + r] = m_ref;
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(x_bar(q));
          if (grow) {
            // O must be quiescent: P.V of block bg - 1 is the bg-th completion of pv_done
            if (!tc::mbar_wait(pv_done, (bg - 1u) & 1u, abort_flag)) { ok = false; break; }
            tc::tc_fence_after();
            const float alpha = ex2_approx(m_prev - m_new);
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
          m_known = m_ref;
          // P = exp2(S*scale - m_ref) as fp16; partial row sum in fp32 from the fp32 exponentials
          const float neg_m = -m_ref;
          const float2 mul2 = make_float2(p.scale_log2, p.scale_log2), neg_m2 = make_float2(neg_m, neg_m);
          float2 lacc0 = make_float2(0.f, 0.f), lacc1 = make_float2(0.f, 0.f);
#pragma unroll
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < 32; e += 4) {
              const float2 xa = fma2(make_float2(__uint_as_float(sv[c * 32 + e]), __uint_as_float(sv[c * 32 + e + 1])), mul2, neg_m2);
              const float2 xb2 = fma2(make_float2(__uint_as_float(sv[c * 32 + e + 2]), __uint_as_float(sv[c * 32 + e + 3])), mul2, neg_m2);
              const float2 pa = make_float2(ex2_approx(xa.x), ex2_approx(xa.y));
              const float2 pb = make_float2(ex2_approx(xb2.x), ex2_approx(xb2.y));
              lacc0 = add2(lacc0, pa);
              lacc1 = add2(lacc1, pb);
              pk[e >> 1] = pack_f16x2(pa.x, pa.y);
              pk[(e >> 1) + 1] = pack_f16x2(pb.x, pb.y);
            }
            tc::tmem_st_32x16(tP + lane_off + (uint32_t)(c * 16), pk);
          }
          l += (lacc0.x + lacc0.y) + (lacc1.x + lacc1.y);
          HEXB_PROF(5)  // exp, pack, TMEM store issue
          tc::tmem_st_wait();
          tc::tc_fence_before();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(p_full(b));
          HEXB_PROF(6)  // store wait + arrive
        }
        if (!ok) break;
        // ---- epilogue: final scale, row sum of both warpgroups, then each writes half of the columns
        const uint32_t bg_last = blk_base + (uint32_t)n_kv - 1u;
        if (!tc::mbar_wait(x_bar(q), bg_last & 1u, abort_flag)) { ok = false; break; }
        const float m_fin = mref_sh[(bg_last & 1u) * 128 + r];
        float *lt = l_sh + (tiles_done & 1u) * 256;
        lt[g * 128 + r] = l * ex2_approx(m_known - m_fin);   // a warpgroup that had no block of this tile holds l = 0
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(l_bar(q));
        if (!tc::mbar_wait(l_bar(q), tiles_done & 1u, abort_flag)) { ok = false; break; }
        const float lsum = lt[r] + lt[128 + r];
        if (!tc::mbar_wait(o_full, tiles_done & 1u, abort_flag)) { ok = false; break; }
        tc::tc_fence_after();
        const float inv = 1.0f / lsum;
        const int64_t orow_off = (int64_t)z * p.so_z + (int64_t)h * p.so_h + (int64_t)qi * p.so_n + g * OCOLS;
        __half *orow = static_cast<__half *>(p.out) + orow_off;
        float *orow32 = static_cast<float *>(p.out) + orow_off;
#pragma unroll 1
        for (int c = 0; c < OCOLS / 32; ++c) {
          uint32_t o[32];
          tc::tmem_ld_32x32(tO + lane_off + (uint32_t)(g * OCOLS + c * 32), o);
          tc::tmem_ld_wait();
          if (c == OCOLS / 32 - 1) {  // O is in registers: the next tile's first product may overwrite it
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(o_empty);
          }
          if (qi < p.N_CTX && p.out_f32) {
#pragma unroll
            for (int gq = 0; gq < 8; ++gq) {
              float4 f = make_float4(__uint_as_float(o[gq * 4]) * inv, __uint_as_float(o[gq * 4 + 1]) * inv,
                                     __uint_as_float(o[gq * 4 + 2]) * inv, __uint_as_float(o[gq * 4 + 3]) * inv);
              if (p.out_vec_ok) {
                *reinterpret_cast<float4 *>(orow32 + c * 32 + gq * 4) = f;
              } else {
                orow32[c * 32 + gq * 4] = f.x; orow32[c * 32 + gq * 4 + 1] = f.y;
                orow32[c * 32 + gq * 4 + 2] = f.z; orow32[c * 32 + gq * 4 + 3] = f.w;
              }
            }
          } else if (qi < p.N_CTX) {
#pragma unroll
            for (int gq = 0; gq < 4; ++gq) {
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(o[gq * 8 + e]) * inv;
              if (p.out_vec_ok) {
                Vec16<__half> ov;
                ov.pack(f);
                *reinterpret_cast<uint4 *>(orow + c * 32 + gq * 8) = ov.raw;
              } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) orow[c * 32 + gq * 8 + e] = __float2half_rn(f[e]);
              }
            }
          }
        }
        blk_base += (uint32_t)n_kv;
      }
    }
    if (lane == 0 && q == 2) { HEXB_PROF_FLUSH(8 * g, 8) }
  } else {
    // ------------------------------------------------------------ softmax / correction / epilogue
    const int q = warp & 3;                 // TMEM lane quarter this warp may touch
    const int g = (warp - 2) >> 2;          // column group of the row this thread works on
    const int r = q * 32 + lane;            // row inside the tile == TMEM lane
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    constexpr int COLS = cfg::COLS, OCOLS = cfg::OCOLS;
    uint32_t blk = 0, tiles_done = 0, xphase = 0;
    bool ok = true;
    HEXB_PROF_DECL(8)
    // Meeting point of the TPR warps that share this lane quarter: every lane has written its value to the
    // exchange buffer, lane 0 arrives for the warp, and all wait for the phase (a bounded wait, like every
    // other wait of the kernel -- a named barrier would hang the partners of a warp that gave up).
    auto quarter_sync = [&]() {
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(x_bar(q));
      const bool done = tc::mbar_wait(x_bar(q), xphase & 1u, abort_flag);
      ++xphase;
      return done;
    };
    for (int w = blockIdx.x; w < p.num_items && ok; w += gridDim.x) {
      const int bh = w / p.items_per_bh, rank = w - bh * p.items_per_bh;
      const int z = bh / p.H, h = bh - z * p.H;
      for (int i = 0; i < p.tiles_per_item && ok; ++i, ++tiles_done) {
        const int q_tile = tile_of(rank, i);
        const int n_kv = nkv_of(q_tile);
        const int m0 = q_tile * BLOCK_M;
        const int qi = m0 + r;
        float m_ref = -INFINITY, l = 0.f;
        for (int j = 0; j < n_kv; ++j, ++blk) {
          const uint32_t b = blk & 1u, ph = (blk >> 1) & 1u;
          HEXB_PROF(0)  // loop / epilogue
          if (!tc::mbar_wait(s_full(b), ph, abort_flag)) { ok = false; break; }
          HEXB_PROF(1)  // wait S
          tc::tc_fence_after();
          const uint32_t tS = tmem_base + b * BN + (uint32_t)(g * COLS);      // this thread's score columns
          const uint32_t tP = tmem_base + b * BN + (uint32_t)(g * COLS / 2);  // and where their fp16 pairs go
          const int kv0 = j * BN + g * COLS;
          const bool need_mask = (p.causal && j * BN + BN - 1 > m0) || (j * BN + BN > p.N_CTX);
          uint32_t sv[COLS];
#pragma unroll
          for (int c = 0; c < COLS / 32; ++c)
            tc::tmem_ld_32x32(tS + lane_off + (uint32_t)(c * 32), reinterpret_cast<uint32_t(&)[32]>(sv[c * 32]));
          tc::tmem_ld_wait();
          HEXB_PROF(2)  // TMEM load of S
          if (need_mask) {
#pragma unroll
            for (int e = 0; e < COLS; ++e) {
              const int kv = kv0 + e;
              if ((p.causal && kv > qi) || kv >= p.N_CTX) sv[e] = 0xff800000u;  // -inf: exp2 gives 0
            }
          }
          float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int e = 0; e < COLS; e += 8) {
#pragma unroll
            for (int u = 0; u < 4; ++u)
              mx4[u] = max3(mx4[u], __uint_as_float(sv[e + 2 * u]), __uint_as_float(sv[e + 2 * u + 1]));
          }
          float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
          // the threads of a row agree on the block maximum: own part to shared memory, barrier of the TPR warps
          // of this lane quarter, read all parts (two buffers by block parity, so one barrier per block suffices)
          float *xb = xchg + (size_t)(blk & 1u) * (TPR * 128);
          xb[g * 128 + r] = mx;
          HEXB_PROF(3)  // mask, own max
          if (!quarter_sync()) { ok = false; break; }
          HEXB_PROF(4)  // meeting point
#pragma unroll
          for (int gg = 0; gg < TPR; ++gg) mx = fmaxf(mx, xb[gg * 128 + r]);
          mx *= p.scale_log2;   // scale > 0: max commutes with the scaling
          const float m_new = fmaxf(m_ref, mx);
          if (j == 0) {
            m_ref = m_new;
          } else if (__any_sync(0xffffffffu, m_new - m_ref > kRescaleThreshold)) {
            // every warp of the lane quarter sees the same maxima, hence takes this branch together.
            // O must be quiescent: P.V of the previous block is the blk-th completion of pv_done
            if (!tc::mbar_wait(pv_done, (blk - 1u) & 1u, abort_flag)) { ok = false; break; }
            tc::tc_fence_after();
            const float alpha = ex2_approx(m_ref - m_new);
            m_ref = m_new;
            l *= alpha;
#pragma unroll 1
            for (int c = 0; c < OCOLS / 16; ++c) {
              uint32_t o[16];
              tc::tmem_ld_32x16(tO + lane_off + (uint32_t)(g * OCOLS + c * 16), o);
              tc::tmem_ld_wait();
#pragma unroll
              for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
              tc::tmem_st_32x16(tO + lane_off + (uint32_t)(g * OCOLS + c * 16), o);
            }
            tc::tmem_st_wait();
          }
          HEXB_PROF(3)
          // P = exp2(S*scale - m_ref) as fp16; partial row sum in fp32 from the fp32 exponentials
          const float neg_m = -m_ref;
          const float2 mul2 = make_float2(p.scale_log2, p.scale_log2), neg_m2 = make_float2(neg_m, neg_m);
          float2 lacc0 = make_float2(0.f, 0.f), lacc1 = make_float2(0.f, 0.f);
#pragma unroll
          for (int c = 0; c < COLS / 32; ++c) {
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < 32; e += 4) {
              const float2 xa = fma2(make_float2(__uint_as_float(sv[c * 32 + e]), __uint_as_float(sv[c * 32 + e + 1])), mul2, neg_m2);
              const float2 xb2 = fma2(make_float2(__uint_as_float(sv[c * 32 + e + 2]), __uint_as_float(sv[c * 32 + e + 3])), mul2, neg_m2);
              const float2 pa = make_float2(ex2_approx(xa.x), ex2_approx(xa.y));
              const float2 pb = make_float2(ex2_approx(xb2.x), ex2_approx(xb2.y));
              lacc0 = add2(lacc0, pa);
              lacc1 = add2(lacc1, pb);
              pk[e >> 1] = pack_f16x2(pa.x, pa.y);
              pk[(e >> 1) + 1] = pack_f16x2(pb.x, pb.y);
            }
            tc::tmem_st_32x16(tP + lane_off + (uint32_t)(c * 16), pk);
          }
          l += (lacc0.x + lacc0.y) + (lacc1.x + lacc1.y);
          HEXB_PROF(5)  // exp, pack, TMEM store issue
          tc::tmem_st_wait();
          tc::tc_fence_before();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(p_full(b));
          HEXB_PROF(6)  // store wait + arrive
        }
        if (!ok) break;
        // the row sum: partial sums of the TPR threads of the row through their own part of the exchange buffer
        // (written once per tile; the partners read it right after the meeting point, a whole tile of meeting
        // points before it is written again)
        float *xl = xchg + 2 * TPR * 128;
        xl[g * 128 + r] = l;
        if (!quarter_sync()) { ok = false; break; }
        float lsum = 0.f;
#pragma unroll
        for (int gg = 0; gg < TPR; ++gg) lsum += xl[gg * 128 + r];
        if (!tc::mbar_wait(o_full, tiles_done & 1u, abort_flag)) { ok = false; break; }
        tc::tc_fence_after();
        const float inv = 1.0f / lsum;
        const int64_t orow_off = (int64_t)z * p.so_z + (int64_t)h * p.so_h + (int64_t)qi * p.so_n + g * OCOLS;
        __half *orow = static_cast<__half *>(p.out) + orow_off;
        float *orow32 = static_cast<float *>(p.out) + orow_off;
#pragma unroll 1
        for (int c = 0; c < OCOLS / 16; ++c) {
          uint32_t o[16];
          tc::tmem_ld_32x16(tO + lane_off + (uint32_t)(g * OCOLS + c * 16), o);
          tc::tmem_ld_wait();
          if (c == OCOLS / 16 - 1) {  // O is in registers: the next tile's first product may overwrite it
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(o_empty);
          }
          if (qi < p.N_CTX && p.out_f32) {
#pragma unroll
            for (int gq = 0; gq < 4; ++gq) {
              float4 f = make_float4(__uint_as_float(o[gq * 4]) * inv, __uint_as_float(o[gq * 4 + 1]) * inv,
                                     __uint_as_float(o[gq * 4 + 2]) * inv, __uint_as_float(o[gq * 4 + 3]) * inv);
              if (p.out_vec_ok) {
                *reinterpret_cast<float4 *>(orow32 + c * 16 + gq * 4) = f;
              } else {
                orow32[c * 16 + gq * 4] = f.x; orow32[c * 16 + gq * 4 + 1] = f.y;
                orow32[c * 16 + gq * 4 + 2] = f.z; orow32[c * 16 + gq * 4 + 3] = f.w;
              }
            }
          } else if (qi < p.N_CTX) {
#pragma unroll
            for (int gq = 0; gq < 2; ++gq) {
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(o[gq * 8 + e]) * inv;
              if (p.out_vec_ok) {
                Vec16<__half> ov;
                ov.pack(f);
                *reinterpret_cast<uint4 *>(orow + c * 16 + gq * 8) = ov.raw;
              } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) orow[c * 16 + gq * 8 + e] = __float2half_rn(f[e]);
              }
            }
          }
        }
      }
    }
    if (lane == 0 && q == 2) { HEXB_PROF_FLUSH(8 * g, 8) }
  }

  // ------------------------------------------------------------ teardown
#ifdef HEXB_ATTN_PROFILE
  // (development builds: the phase timers of one softmax warp per column group are flushed inside its role)
#endif
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);  // let copies in flight land before the CTA retires
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, cfg::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&g_attn4_status, (int)HEXB_ERR_TIMEOUT);
}

template <int HD, int TPR, bool ALT = false>
static int launch(const __half *Q, const __half *K, const __half *V, void *O, int64_t Z, int64_t H, int64_t N,
                  const int64_t *s, float scale_log2, int causal, int out_f32, int sm_count, cudaStream_t st) {
  using cfg = Cfg<HD, TPR>;
  CUtensorMap tm[3];
  const __half *base[3] = {Q, K, V};
  for (int i = 0; i < 3; ++i) {
    const uint64_t dims[4] = {(uint64_t)HD, (uint64_t)N, (uint64_t)H, (uint64_t)Z};
    const uint64_t strides[3] = {(uint64_t)s[3 * i + 2] * 2, (uint64_t)s[3 * i + 1] * 2, (uint64_t)s[3 * i + 0] * 2};
    const uint32_t box[4] = {64, 128, 1, 1};
    if (int e = encode_tmap_f16_sw128(&tm[i], base[i], 4, dims, strides, box)) return e;
  }
  static PerDeviceOnce attr_done;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done.is_done(dev)) {
    HEXB_CUDA_OK(cudaFuncSetAttribute(attn_fwd_wide_kernel<HD, TPR, ALT>, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg::SMEM_BYTES));
    attr_done.mark(dev);
  }
  Params p;
#ifdef HEXB_ATTN_PROFILE
  p.prof = attn_profile_buffer();
#endif
  p.out = O;
  p.so_z = s[9]; p.so_h = s[10]; p.so_n = s[11];
  p.H = (int)H; p.N_CTX = (int)N;
  p.out_f32 = out_f32;
  {
    const int per16 = out_f32 ? 4 : 8;
    p.out_vec_ok = aligned16(O) && s[9] % per16 == 0 && s[10] % per16 == 0 && s[11] % per16 == 0;
  }
  p.num_q_tiles = (int)((N + BLOCK_M - 1) / BLOCK_M);
  p.tiles_per_item = (causal && p.num_q_tiles % 2 == 0) ? 2 : 1;
  p.items_per_bh = p.num_q_tiles / p.tiles_per_item;
  p.scale_log2 = scale_log2;
  p.causal = causal ? 1 : 0;
  const int64_t items = (int64_t)p.items_per_bh * Z * H;
  if (items > 0x7fffffffll) return HEXB_ERR_UNSUPPORTED;
  p.num_items = (int)items;
  const int64_t ctas = items < sm_count ? items : sm_count;
  launch_pdl(attn_fwd_wide_kernel<HD, TPR, ALT>, dim3((unsigned)ctas), dim3(cfg::THREADS), (size_t)cfg::SMEM_BYTES, st, tm[0],
             tm[1], tm[2], p);
  return check_launch("attn_wide");
}

}  // namespace attn4

int attn_wide_launch(const __half *Q, const __half *K, const __half *V, void *O, int64_t Z, int64_t H, int64_t N, int64_t D,
                     const int64_t *strides, float scale_log2, int causal, int out_f32, int threads_per_row, cudaStream_t st) {
  DeviceInfo di;
  if (int e = current_device(&di)) return e;
#define HEXB_WIDE(HD_, TPR_) \
  return attn4::launch<HD_, TPR_>(Q, K, V, O, Z, H, N, strides, scale_log2, causal, out_f32, di.sm_count, st)
  if (D == 128 && threads_per_row == 1)
    return attn4::launch<128, 2, true>(Q, K, V, O, Z, H, N, strides, scale_log2, causal, out_f32, di.sm_count, st);
  if (D == 64 && threads_per_row == 1)
    return attn4::launch<64, 2, true>(Q, K, V, O, Z, H, N, strides, scale_log2, causal, out_f32, di.sm_count, st);
  if (D == 128 && threads_per_row == 4) HEXB_WIDE(128, 4);
  if (D == 128) HEXB_WIDE(128, 2);
  if (D == 64 && threads_per_row == 4) HEXB_WIDE(64, 4);
  if (D == 64) HEXB_WIDE(64, 2);
#undef HEXB_WIDE
  return HEXB_ERR_UNSUPPORTED;
}

int attn_wide_status_fetch_and_clear(int *out) {
  int v = 0, zero = 0;
  HEXB_CUDA_OK(cudaMemcpyFromSymbol(&v, g_attn4_status, sizeof(int)));
  if (v) HEXB_CUDA_OK(cudaMemcpyToSymbol(g_attn4_status, &zero, sizeof(int)));
  *out = v;
  return HEXB_OK;
}

}  // namespace hexb
