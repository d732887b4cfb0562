// Flash-attention forward, third form: TWO 128-row query tiles per CTA taking turns on the tensor
// pipe, 128-key blocks, one CTA per SM.
//
// Reference semantics as in attention.cu: attention_fwd_kernel + _attn_fwd_inner
// (test/python/triton/test_flash_attention.py:37-168), the fp16 MLIR form
// (test/python/mlir/hexkl_attention/input.mlir:5-168, P truncated to fp16 before P.V), causal = the
// -inf mask of tm_tensor.attention (lib/Transforms/LowerTmTensor.cpp:70-235).
//
// Why a third form.  With 64-key blocks the Q.K^T MMAs are 128x64x16: every one of them re-reads 4 KiB
// of Q and 2 KiB of K from shared memory for 32 tensor clocks of work, more than shared memory
// delivers, and the tensor pipe stalls on its operands.  A 128x128x16 MMA reads 8 KiB per 64 clocks,
// which shared memory sustains -- but its score tile takes 128 TMEM columns, so a query tile cannot
// double-buffer its scores next to a 128-column output accumulator and a second resident CTA.  Here
// the two things that overlap are two query tiles of one CTA instead:
//
//   TMEM (512 columns)  S0 [0,128)  S1 [128,256)  O0 [256,256+D)  O1 [384,384+D);  P_t = fp16 over S_t[0,64)
//   warp 0      TMA: Q0, Q1 once per tile pair; K_j, V_j through a ring of four 128-row stages
//   warp 1      MMA: S_t = Q_t.K_j^T (operands in shared memory), O_t += P_t.V_j (P from TMEM, V as
//               stored); order  P0V, Q0K', P1V, Q1K', ...  so that while the softmax of tile t runs, the
//               pipe works on the other tile.  (One issuing thread per tile instead -- tried: the products
//               alone then run 18 % faster, the queue in front of the pipe being only a few instructions
//               deep, but nothing keeps the two tiles out of step any more and the whole kernel ran 25 % slower.)
//   warps 2-5   softmax of tile 0, warps 6-9 softmax of tile 1 (one query row per thread; twice as many
//               warps with two threads per row): tcgen05.ld
//               the 128 scores, row max, P = exp2(S*scale - m) -> fp16 -> TMEM in two halves (the
//               first 64 keys are handed to the MMA thread while the second 64 are exponentiated),
//               lazy rescale of O (only when a maximum grows by more than 2^8), epilogue O/l.
// K and V tiles are read once for 256 query rows.  Causal: a tile's last block is the diagonal one;
// a CTA walks a late (long) and an early (short) tile pair so that all CTAs do the same work.
// Plain calls only (no additive mask, equal query and key lengths); everything else stays on the
// kernels of attention.cu.  Every mbarrier wait is bounded; no load uses cluster multicast.
#include "attn_common.cuh"

namespace hexb {

static __device__ int g_attn3_status = 0;

namespace attn3 {

using namespace attn;

constexpr int BLOCK_M = 128;
constexpr int BN = 128;
constexpr int STAGES = 4;

template <int HD>
struct Cfg {
  static constexpr int CHUNKS = HD / 64;            // 64-column (128-byte) swizzle chunks
  static constexpr int TILE_BYTES = 128 * HD * 2;   // one Q tile, or one K / V stage
  static constexpr int CHUNK_BYTES = 128 * 128;     // 128 rows x 128 bytes
  static constexpr int NBAR = 32;                   // 24 pipeline barriers + 8 exchange barriers (tile x lane quarter)
  static constexpr int XCH_BYTES = 2 * 2 * 2 * 128 * 4;   // exchange slots [tile][parity][half][row] (two threads per row)
  static constexpr int SMEM_BYTES = (2 + STAGES) * TILE_BYTES + NBAR * 8 + 16 + XCH_BYTES + 1024;
  static constexpr int TMEM_COLS = 512;
  static constexpr int O_COL = 256;                 // O_t at O_COL + t * 128
};

struct Params {
#ifdef HEXB_ATTN_PROFILE
  unsigned long long *prof;
#endif
  void *out;
  int64_t so_z, so_h, so_n;
  int H, N_CTX;
  int out_f32, out_vec_ok;
  int num_pairs;        // tile pairs (256 query rows) per (batch, head)
  int pairs_per_cta;    // 1, or 2 (causal: a late and an early pair)
  int ctas_per_bh;      // work items per (batch, head)
  int num_items;        // work items in the launch; CTA c walks items c, c + gridDim.x, ...
  float scale_log2;
  int causal;
#ifdef HEXB_DEV
  int ablate;           // development builds: 1 = no MMAs are issued, 2 = the softmax warps do no arithmetic
#endif
};

// TPR = 2: two softmax threads per query row (sixteen softmax warps, 576 threads).  Warps w and w + 4 of a
// tile own the same 32 rows and, of every 64-key half of a block, 32 columns each (so both halves of P
// are still handed over one after the other); they exchange row maxima once per block and row sums once
// per tile through shared memory and an mbarrier of their own.  With one thread per row the four warps of
// a tile sit alone on their schedulers while the other tile is in its MMA phase, and a lone warp gets
// 8/11 of the special-function unit; the softmax of a block is in this kernel's critical chain.
template <int HD, int TPR>
__global__ void __launch_bounds__(64 + 256 * TPR, 1)
attn_fwd_pingpong_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmV, const Params p) {
  using cfg = Cfg<HD>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw_addr = tc::smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
  uint8_t *smem = smem_raw + pad;
  const uint32_t smem_addr = raw_addr + pad;
  const uint32_t sQ0 = smem_addr;                                  // Q_t at sQ0 + t * TILE_BYTES
  const uint32_t sKV0 = sQ0 + 2 * cfg::TILE_BYTES;                 // stage s at sKV0 + s * TILE_BYTES
  const uint32_t bar0 = sKV0 + STAGES * cfg::TILE_BYTES;
  auto q_full = [&](int t) { return bar0 + 8u * (uint32_t)t; };
  auto q_empty = [&](int t) { return bar0 + 16 + 8u * (uint32_t)t; };
  auto s_full = [&](int t) { return bar0 + 32 + 8u * (uint32_t)t; };
  auto p_full = [&](int t, int h) { return bar0 + 48 + 8u * (uint32_t)(2 * t + h); };
  auto pv_done = [&](int t) { return bar0 + 80 + 8u * (uint32_t)t; };
  auto o_full = [&](int t) { return bar0 + 96 + 8u * (uint32_t)t; };
  auto o_empty = [&](int t) { return bar0 + 112 + 8u * (uint32_t)t; };
  auto kv_full = [&](uint32_t s) { return bar0 + 128 + 8u * s; };
  auto kv_empty = [&](uint32_t s) { return bar0 + 160 + 8u * s; };   // ends at bar0 + 192 = 24 barriers
  auto x_bar = [&](int t, int qq) { return bar0 + 192 + 8u * (uint32_t)(4 * t + qq); };   // ends at bar0 + 256
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + (2 + STAGES) * cfg::TILE_BYTES + cfg::NBAR * 8);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  float *xch = reinterpret_cast<float *>(tmem_slot + 4);   // 16 bytes behind the slot
  constexpr int PART = 64 / TPR;     // score columns per thread in each 64-key half of a block
  constexpr int OCOLS = HD / TPR;    // output columns per thread

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kv_blocks = (p.N_CTX + BN - 1) / BN;
  // Work items: item w = (batch, head) w / ctas_per_bh, rank w % ctas_per_bh inside it; the items of one
  // (batch, head) are adjacent so that its K and V stay in L2 while the CTAs that share them run.  A
  // causal item is a late (long) tile pair followed by an early (short) one, so all items cost the same.
  // The CTA is persistent: every role walks the same item sequence, and the hand-offs run across item
  // boundaries (the next item's Q, K, V are fetched and its first scores issued while the softmax warps
  // finish the current one).
  auto pair_of = [&](int q_rank, int i) {
    if (p.pairs_per_cta == 2) return i == 0 ? p.num_pairs - 1 - q_rank : q_rank;
    return q_rank;
  };
  // key blocks tile t of pair T walks (0: the tile lies past the last query row)
  auto nkv_of = [&](int T, int t) {
    const int m0 = (2 * T + t) * BLOCK_M;
    if (m0 >= p.N_CTX) return 0;
    const int need = 2 * T + t + 1;     // causal: keys 0 .. m0 + 127
    return (p.causal && need < kv_blocks) ? need : kv_blocks;
  };

  if (threadIdx.x == 0) {
    for (int t = 0; t < 2; ++t) {
      tc::mbar_init(q_full(t), 1);
      tc::mbar_init(q_empty(t), 1);
      tc::mbar_init(s_full(t), 1);
      tc::mbar_init(p_full(t, 0), 4 * TPR);
      tc::mbar_init(p_full(t, 1), 4 * TPR);
      tc::mbar_init(pv_done(t), 1);
      tc::mbar_init(o_full(t), 1);
      tc::mbar_init(o_empty(t), 4 * TPR);
      for (int qq = 0; qq < 4; ++qq) tc::mbar_init(x_bar(t, qq), 2);
    }
    for (uint32_t s = 0; s < STAGES; ++s) {
      tc::mbar_init(kv_full(s), 1);
      tc::mbar_init(kv_empty(s), 1);
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

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t item = 0;           // K/V tiles loaded so far (K_0, V_0, K_1, V_1, ...), across tile pairs
      uint32_t rounds[2] = {0, 0}; // tile pairs in which tile t was active so far
      bool ok = true;
      for (int w = blockIdx.x; w < p.num_items && ok; w += gridDim.x) {
      const int bh = w / p.ctas_per_bh, q_rank = w - bh * p.ctas_per_bh;
      const int z = bh / p.H, h = bh - z * p.H;
      for (int i = 0; i < p.pairs_per_cta && ok; ++i) {
        const int T = pair_of(q_rank, i);
        const int n0 = nkv_of(T, 0), n1 = nkv_of(T, 1);
        const int nmax = n0 > n1 ? n0 : n1;
        for (int t = 0; t < 2; ++t) {
          if (nkv_of(T, t) == 0) continue;
          // the previous pair's last Q.K^T of this tile has read Q_t
          if (rounds[t] > 0 && !tc::mbar_wait(q_empty(t), (rounds[t] - 1u) & 1u, abort_flag)) { ok = false; break; }
          ++rounds[t];
          tc::mbar_arrive_expect_tx(q_full(t), cfg::TILE_BYTES);
#pragma unroll
          for (int c = 0; c < cfg::CHUNKS; ++c)
            tc::tma_load_4d(sQ0 + t * cfg::TILE_BYTES + c * cfg::CHUNK_BYTES, &tmQ, c * 64, (2 * T + t) * BLOCK_M, h, z,
                            q_full(t));
        }
        for (int j = 0; j < nmax && ok; ++j) {
#pragma unroll
          for (int kind = 0; kind < 2; ++kind, ++item) {
            const uint32_t s = item % STAGES, ph = (item / STAGES) & 1u;
            if (!tc::mbar_wait(kv_empty(s), ph ^ 1u, abort_flag)) { ok = false; break; }
            tc::mbar_arrive_expect_tx(kv_full(s), cfg::TILE_BYTES);
#pragma unroll
            for (int c = 0; c < cfg::CHUNKS; ++c)
              tc::tma_load_4d(sKV0 + s * cfg::TILE_BYTES + c * cfg::CHUNK_BYTES, kind == 0 ? &tmK : &tmV, c * 64, j * BN, h,
                              z, kv_full(s));
          }
        }
      }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = tc::make_idesc_f16_f32(BLOCK_M, BN, 0, 0);
      constexpr uint32_t idesc_pv = tc::make_idesc_f16_f32(BLOCK_M, HD, 0, 1);
      uint32_t item_base = 0;       // index of K_0 of the current pair in the K/V item sequence
      uint32_t blk[2] = {0, 0};     // blocks of tile t issued so far (phase counters of s_full / p_full / pv_done)
      uint32_t rounds[2] = {0, 0};
      bool ok = true;
      HEXB_PROF_DECL(8)
      auto wait_kv = [&](uint32_t item) {
        return tc::mbar_wait(kv_full(item % STAGES), (item / STAGES) & 1u, abort_flag);
      };
      // S_t = Q_t . K^T with K in the stage of `item`
      auto issue_qk = [&](int t, uint32_t item, bool last_of_tile) {
        const uint32_t sQ = sQ0 + t * cfg::TILE_BYTES, sK = sKV0 + (item % STAGES) * cfg::TILE_BYTES;
#ifdef HEXB_DEV
        if (!(p.ablate & 1))
#endif
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (uint32_t)((k >> 2) * cfg::CHUNK_BYTES + (k & 3) * 32);
          tc::mma_f16_ss(tmem_base + (uint32_t)t * 128u, tc::make_smem_desc_sw128(sQ + off, 16, 1024),
                         tc::make_smem_desc_sw128(sK + off, 16, 1024), idesc_qk, k != 0 ? 1u : 0u);
        }
        tc::mma_commit(s_full(t));
        if (last_of_tile) tc::mma_commit(q_empty(t));
      };
      for (int w = blockIdx.x; w < p.num_items && ok; w += gridDim.x) {
      const int q_rank = w % p.ctas_per_bh;
      for (int i = 0; i < p.pairs_per_cta && ok; ++i) {
        const int T = pair_of(q_rank, i);
        int n[2] = {nkv_of(T, 0), nkv_of(T, 1)};
        const int nmax = n[0] > n[1] ? n[0] : n[1];
        // first scores of both tiles
        if (!wait_kv(item_base)) { ok = false; break; }
        tc::tc_fence_after();
        for (int t = 0; t < 2 && ok; ++t) {
          if (n[t] == 0) continue;
          if (!tc::mbar_wait(q_full(t), rounds[t] & 1u, abort_flag)) { ok = false; break; }
          tc::tc_fence_after();
          issue_qk(t, item_base, n[t] == 1);
        }
        if (!ok) break;
        tc::mma_commit(kv_empty(item_base % STAGES));
        for (int j = 0; j < nmax && ok; ++j) {
          const uint32_t item_v = item_base + 2u * (uint32_t)j + 1u, item_k1 = item_v + 1u;
          HEXB_PROF(0)  // other
          if (!wait_kv(item_v)) { ok = false; break; }
          HEXB_PROF(1)  // wait V
          bool k1_ready = false;
          for (int t = 0; t < 2 && ok; ++t) {
            if (j >= n[t]) continue;
            // the first product of a later pair overwrites O_t: the previous epilogue must have read it
            if (j == 0 && rounds[t] > 0 && !tc::mbar_wait(o_empty(t), (rounds[t] - 1u) & 1u, abort_flag)) { ok = false; break; }
            const uint32_t ph = blk[t] & 1u;
            const uint32_t sV = sKV0 + (item_v % STAGES) * cfg::TILE_BYTES;
            const uint32_t tP = tmem_base + (uint32_t)t * 128u, tO = tmem_base + cfg::O_COL + (uint32_t)t * 128u;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              HEXB_PROF(0)
              if (!tc::mbar_wait(p_full(t, half), ph, abort_flag)) { ok = false; break; }
              HEXB_PROF(2 + half)  // wait P first half / second half
              tc::tc_fence_after();
#ifdef HEXB_DEV
              if (!(p.ablate & 1))
#endif
#pragma unroll
              for (int k = 4 * half; k < 4 * half + 4; ++k) {
                // A = P rows from TMEM (16 fp16 = 8 columns per step); B = V: 16 key rows = 2 swizzle atoms
                tc::mma_f16_ts(tO, tP + (uint32_t)(k * 8),
                               tc::make_smem_desc_sw128(sV + (uint32_t)(k * 2048), cfg::CHUNK_BYTES, 1024), idesc_pv,
                               (j | k) != 0 ? 1u : 0u);
              }
              HEXB_PROF(4)  // issue P.V
            }
            if (!ok) break;
            tc::mma_commit(pv_done(t));
            if (j == n[t] - 1) tc::mma_commit(o_full(t));
            ++blk[t];
            // next scores of this tile go out right behind its P.V, before the other tile's P is waited for
            if (j + 1 < n[t]) {
              if (!k1_ready) {
                HEXB_PROF(0)
                if (!wait_kv(item_k1)) { ok = false; break; }
                HEXB_PROF(5)  // wait K
                tc::tc_fence_after();
                k1_ready = true;
              }
              HEXB_PROF(0)
              issue_qk(t, item_k1, j + 2 == n[t]);
              HEXB_PROF(6)  // issue Q.K^T
            }
          }
          if (!ok) break;
          tc::mma_commit(kv_empty(item_v % STAGES));                      // both tiles' P.V_j are issued
          if (j + 1 < nmax) tc::mma_commit(kv_empty(item_k1 % STAGES));   // and both tiles' Q.K_{j+1}^T
        }
        for (int t = 0; t < 2; ++t)
          if (n[t] > 0) ++rounds[t];
        item_base += 2u * (uint32_t)nmax;
      }
      }
      HEXB_PROF_FLUSH(0, 8)
    }
  } else {
    // ------------------------------------------------------------ softmax / correction / epilogue
    const int t = (warp - 2) / (4 * TPR);   // tile of this warpgroup
    const int hsel = TPR == 2 ? (((warp - 2) >> 2) & 1) : 0;   // which columns of a half (two threads per row)
    const int q = warp & 3;                 // TMEM lane quarter this warp may touch
    const int r = q * 32 + lane;            // row inside the tile == TMEM lane
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    // value exchange between the two threads of a row (see the kernel's head comment); bounded like every wait
    uint32_t xc = 0;
    auto exchange = [&](float mine, float &other) -> bool {
      float *slot = xch + (t * 2 + (int)(xc & 1u)) * 256;
      slot[hsel * 128 + r] = mine;
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(x_bar(t, q));
      if (!tc::mbar_wait(x_bar(t, q), xc & 1u, abort_flag)) return false;
      ++xc;
      other = slot[(hsel ^ 1) * 128 + r];
      return true;
    };
    (void)exchange;
    const uint32_t tS = tmem_base + (uint32_t)t * 128u, tP = tS, tO = tmem_base + cfg::O_COL + (uint32_t)t * 128u;
    uint32_t blk = 0, rounds = 0;
    bool ok = true;
    HEXB_PROF_DECL(8)
    for (int w = blockIdx.x; w < p.num_items && ok; w += gridDim.x) {
    const int bh = w / p.ctas_per_bh, q_rank = w - bh * p.ctas_per_bh;
    const int z = bh / p.H, h = bh - z * p.H;
    for (int i = 0; i < p.pairs_per_cta && ok; ++i) {
      const int T = pair_of(q_rank, i);
      const int n_kv = nkv_of(T, t);
      if (n_kv == 0) continue;
      const int m0 = (2 * T + t) * BLOCK_M;
      const int qi = m0 + r;
      float m_ref = -INFINITY, l = 0.f;
      for (int j = 0; j < n_kv; ++j, ++blk) {
        HEXB_PROF(0)  // loop / epilogue of the previous pair
        if (!tc::mbar_wait(s_full(t), blk & 1u, abort_flag)) { ok = false; break; }
        HEXB_PROF(1)  // wait S
        tc::tc_fence_after();
#ifdef HEXB_DEV
        if (p.ablate & 2) {  // hand the block straight back
          tc::tc_fence_before();
          __syncwarp();
          if (lane == 0) { tc::mbar_arrive(p_full(t, 0)); tc::mbar_arrive(p_full(t, 1)); }
          continue;
        }
#endif
        const int kv0 = j * BN;
        const bool need_mask = (p.causal && kv0 + BN - 1 > m0) || (kv0 + BN > p.N_CTX);
        // Element e of half h2 is key kv0 + 64 * h2 + PART * hsel + e.  One thread per row: all 128 scores
        // stay in registers (sv[h2 * 64 + e]).  Two threads per row: 64 scores per thread do not fit the 96
        // registers a CTA of 18 warps leaves, so the part of the second half is read for the maximum,
        // dropped, and read again before it is exponentiated; the part of the first half stays in sv.
        // (P of the first half lands on score columns 0..31, which both threads have read by the time
        // they have exchanged their maxima; P of the second half on columns 32..63, likewise.)
        uint32_t sv[TPR == 1 ? 128 : 32];
        auto mask_part = [&](uint32_t(&v)[32], int h2, int c) {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int kv = kv0 + 64 * h2 + PART * hsel + c * 32 + e;
            if ((p.causal && kv > qi) || kv >= p.N_CTX) v[e] = 0xff800000u;  // -inf: exp2 gives 0
          }
        };
        float mx8[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) mx8[u] = -INFINITY;
        auto max_part = [&](const uint32_t(&v)[32]) {
#pragma unroll
          for (int e = 0; e < 32; e += 16)
#pragma unroll
            for (int u = 0; u < 8; ++u) mx8[u] = max3(mx8[u], __uint_as_float(v[e + 2 * u]), __uint_as_float(v[e + 2 * u + 1]));
        };
        if constexpr (TPR == 1) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
            tc::tmem_ld_32x32(tS + lane_off + (uint32_t)(c * 32), reinterpret_cast<uint32_t(&)[32]>(sv[c * 32]));
          tc::tmem_ld_wait();
          HEXB_PROF(2)  // TMEM load of S
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (need_mask) mask_part(reinterpret_cast<uint32_t(&)[32]>(sv[c * 32]), c >> 1, c & 1);
            max_part(reinterpret_cast<uint32_t(&)[32]>(sv[c * 32]));
          }
        } else {
          uint32_t second[32];
          tc::tmem_ld_32x32(tS + lane_off + (uint32_t)(64 + PART * hsel), second);
          tc::tmem_ld_32x32(tS + lane_off + (uint32_t)(PART * hsel), reinterpret_cast<uint32_t(&)[32]>(sv[0]));
          tc::tmem_ld_wait();
          HEXB_PROF(2)  // TMEM load of S
          if (need_mask) {
            mask_part(second, 1, 0);
            mask_part(reinterpret_cast<uint32_t(&)[32]>(sv[0]), 0, 0);
          }
          max_part(second);
          max_part(reinterpret_cast<uint32_t(&)[32]>(sv[0]));
        }
        float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])),
                         fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7]))) * p.scale_log2;
        if (TPR == 2) {  // both threads of the row end up with the same maximum
          float other;
          if (!exchange(mx, other)) { ok = false; break; }
          mx = fmaxf(mx, other);
        }
        const float m_new = fmaxf(m_ref, mx);   // scale > 0: max commutes with the scaling
        if (j == 0) {
          m_ref = m_new;
        } else if (__any_sync(0xffffffffu, m_new - m_ref > kRescaleThreshold)) {
          // O_t must be quiescent: P.V of the previous block of this tile is the blk-th completion of pv_done
          if (!tc::mbar_wait(pv_done(t), (blk - 1u) & 1u, abort_flag)) { ok = false; break; }
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
          tc::tmem_st_wait();
        }
        HEXB_PROF(3)  // mask, max, rescale
        // P = exp2(S*scale - m_ref) as fp16 over the first 64 columns of S_t, in two halves of 64 keys;
        // running row sum in fp32 from the fp32 exponentials
        const float neg_m = -m_ref;
        const float2 mul2 = make_float2(p.scale_log2, p.scale_log2), neg_m2 = make_float2(neg_m, neg_m);
        float2 lacc0 = make_float2(0.f, 0.f), lacc1 = make_float2(0.f, 0.f);
        // 32 scores -> 32 weights: packed fp16 into 16 columns of P starting at column pcol
        auto exp_part = [&](const uint32_t(&v)[32], uint32_t pcol) {
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            const float2 xa = fma2(make_float2(__uint_as_float(v[e]), __uint_as_float(v[e + 1])), mul2, neg_m2);
            const float2 xb = fma2(make_float2(__uint_as_float(v[e + 2]), __uint_as_float(v[e + 3])), mul2, neg_m2);
            const float2 pa = make_float2(ex2_approx(xa.x), ex2_approx(xa.y));
            const float2 pb = make_float2(ex2_approx(xb.x), ex2_approx(xb.y));
            lacc0 = add2(lacc0, pa);
            lacc1 = add2(lacc1, pb);
            pk[e >> 1] = pack_f16x2(pa.x, pa.y);
            pk[(e >> 1) + 1] = pack_f16x2(pb.x, pb.y);
          }
          tc::tmem_st_32x16(tP + lane_off + pcol, pk);
        };
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          if constexpr (TPR == 1) {
#pragma unroll
            for (int c = 2 * half; c < 2 * half + 2; ++c)
              exp_part(reinterpret_cast<uint32_t(&)[32]>(sv[c * 32]), (uint32_t)(c * 16));   // key k -> P column k / 2
          } else {
            if (half == 1) {  // the part of the second half comes back from TMEM
              tc::tmem_ld_32x32(tS + lane_off + (uint32_t)(64 + PART * hsel), reinterpret_cast<uint32_t(&)[32]>(sv[0]));
              tc::tmem_ld_wait();
              if (need_mask) mask_part(reinterpret_cast<uint32_t(&)[32]>(sv[0]), 1, 0);
            }
            exp_part(reinterpret_cast<uint32_t(&)[32]>(sv[0]), (uint32_t)(32 * half + 16 * hsel));
          }
          HEXB_PROF(4)  // exp, pack, TMEM store issue
          tc::tmem_st_wait();
          tc::tc_fence_before();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(p_full(t, half));
          HEXB_PROF(5)  // store wait + arrive
        }
        l += (lacc0.x + lacc0.y) + (lacc1.x + lacc1.y);
      }
      if (!ok || !tc::mbar_wait(o_full(t), rounds & 1u, abort_flag)) { ok = false; break; }
      ++rounds;
      tc::tc_fence_after();
      if (TPR == 2) {  // the two parts of the row sum
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
        if (c == OCOLS / 32 - 1) {  // O_t is in registers: the next pair's first product may overwrite it
          tc::tc_fence_before();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(o_empty(t));
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
    }
    if (threadIdx.x == 64 || threadIdx.x == 64 + 128 * TPR) { HEXB_PROF_FLUSH(8 + 8 * t, 8) }
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
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&g_attn3_status, (int)HEXB_ERR_TIMEOUT);
}

template <int HD, int TPR>
static int launch(const __half *Q, const __half *K, const __half *V, void *O, int64_t Z, int64_t H, int64_t N,
                  const int64_t *s, float scale_log2, int causal, int out_f32, int sm_count, cudaStream_t st) {
  using cfg = Cfg<HD>;
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
    HEXB_CUDA_OK(cudaFuncSetAttribute(attn_fwd_pingpong_kernel<HD, TPR>, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg::SMEM_BYTES));
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
  const int q_tiles = (int)((N + BLOCK_M - 1) / BLOCK_M);
  p.num_pairs = (q_tiles + 1) / 2;
  // pairing a late and an early tile pair equalises the CTAs when the tiles differ in length (causal)
  p.pairs_per_cta = (causal && p.num_pairs % 2 == 0) ? 2 : 1;
  p.ctas_per_bh = p.num_pairs / p.pairs_per_cta;
  p.scale_log2 = scale_log2;
  p.causal = causal ? 1 : 0;
#ifdef HEXB_DEV
  p.ablate = (int)option(OPT_attn_ablate, 0);
#endif
  const int64_t items = (int64_t)p.ctas_per_bh * Z * H;
  if (items > 0x7fffffffll) return HEXB_ERR_UNSUPPORTED;
  p.num_items = (int)items;
  const int64_t ctas = items < sm_count ? items : sm_count;   // persistent: one CTA per SM
  launch_pdl(attn_fwd_pingpong_kernel<HD, TPR>, dim3((unsigned)ctas), dim3(64 + 256 * TPR), (size_t)cfg::SMEM_BYTES, st, tm[0],
             tm[1], tm[2], p);
  return check_launch("attn_pingpong");
}

}  // namespace attn3

// Shapes the kernel takes (head sizes 64 and 128).  It is selectable (option attn_kernel = 3, or 4 for two
// softmax threads per row), not the default: measured on B200 it runs behind the 64-key two-buffer kernel
// ([4, 32, 4096, 128]: 597-608 us causal and 1015-1030 us plain against 543-552 and 980; with two threads
// per row 586-592 and 1003-1018).  With one score buffer per tile a block's period is the sum of its
// softmax, its two products and the hand-offs between them (about 250 clocks from tcgen05.commit to the
// waiting thread each way); the exponentials of one tile cannot take less than 1024 clocks (16 per clock
// and SM) whatever the number of threads, so the second thread per row shortens only the load / max part.
int attn_pingpong_supported(int64_t Z, int64_t H, int64_t N, int64_t D, int causal, int sm_count) {
  (void)Z; (void)H; (void)N; (void)causal; (void)sm_count;
  return (D == 64 || D == 128) ? 1 : 0;
}

int attn_pingpong_launch(const __half *Q, const __half *K, const __half *V, void *O, int64_t Z, int64_t H, int64_t N,
                         int64_t D, const int64_t *strides, float scale_log2, int causal, int out_f32, int threads_per_row,
                         cudaStream_t st) {
  DeviceInfo di;
  if (int e = current_device(&di)) return e;
#define HEXB_PP(HD_, TPR_) \
  return attn3::launch<HD_, TPR_>(Q, K, V, O, Z, H, N, strides, scale_log2, causal, out_f32, di.sm_count, st)
  if (D == 128 && threads_per_row == 2) HEXB_PP(128, 2);
  if (D == 128) HEXB_PP(128, 1);
  if (D == 64 && threads_per_row == 2) HEXB_PP(64, 2);
  if (D == 64) HEXB_PP(64, 1);
#undef HEXB_PP
  return HEXB_ERR_UNSUPPORTED;
}

int attn_pingpong_status_fetch_and_clear(int *out) {
  int v = 0, zero = 0;
  HEXB_CUDA_OK(cudaMemcpyFromSymbol(&v, g_attn3_status, sizeof(int)));
  if (v) HEXB_CUDA_OK(cudaMemcpyToSymbol(g_attn3_status, &zero, sizeof(int)));
  *out = v;
  return HEXB_OK;
}

}  // namespace hexb
