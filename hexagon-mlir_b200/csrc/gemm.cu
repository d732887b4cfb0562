// fp16 matmul with fp32 accumulation on the Blackwell tensor cores (tcgen05 + TMEM + TMA).
//
// Reference semantics: matmul(A, B, C, N_ROWS, N_COLUMNS, N_INNER)
// (test/python/triton/test_matmul.py:35-70) and the HexKL runtime call
// hexkl_matmul_f16f16_f32 (qcom_hexagon_backend/bin/runtime/src/HexKLAPI.cpp:15-141) of
// qualcomm/hexagon-mlir: C[M,N] = A[M,K] @ B[K,N], everything row-major.  The HexKL loop re-lays
// out one 32x32 weight tile from DDR per (row tile, col tile, k tile) and accumulates in the fp16
// HMX accumulator; this kernel accumulates in fp32 (TMEM) and rounds once.
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: A tile [128 x 64] (K-major, 128-byte swizzle) and BN/64 B boxes
//               [64 k x 64 n] (N-major, 128-byte swizzle) per k-block into a STAGES-deep smem ring;
//   warp 1      MMA issuer: one thread issues 4 tcgen05.mma (128 x BN x 16) per k-block; the
//               accumulator lives in TMEM and is double-buffered (2 x BN columns) so the epilogue of
//               tile i overlaps the main loop of tile i+1;
//   warps 2..5  epilogue: tcgen05.ld -> (+ residual) -> fp16/fp32 -> 16-byte global stores.
// B is consumed as stored ([K, N] row-major = the "MN-major" operand form), no transpose pass.
// Every mbarrier wait is bounded; on a timeout the CTA sets the status word and tears down.
#include "tc_sm100.cuh"

namespace hexb {

static __device__ int g_gemm_status = 0;

// ---- tile order.  Tiles are walked in groups of `group_m` row-tiles: inside a group the row-tile index
// runs fastest, then the column-tile index, then the next group.  The tiles that run at the same time
// then share `group_m` row-blocks of A and about (concurrent tiles / group_m) column-blocks of B.
// group_m == tiles_m is the plain column-tile-major order: right when A and B both stay in L2 anyway.
__host__ __device__ __forceinline__ void tile_to_mn(int tile, int tiles_m, int tiles_n, int group_m, int *tm, int *tn) {
  const int per_group = group_m * tiles_n;
  const int g = tile / per_group, r = tile - g * per_group;
  const int first = g * group_m;
  const int gsize = tiles_m - first < group_m ? tiles_m - first : group_m;
  *tn = r / gsize;
  *tm = first + (r - *tn * gsize);
}

// Chooses group_m so that the operand blocks of the tiles in flight (`concurrent` of them, each reading
// a_tile_bytes of A and b_tile_bytes of B over the whole K) fit L2: minimise
// group_m * a_tile + ceil(concurrent / group_m) * b_tile.  When all of A and B fit anyway the plain order
// is kept.  Measured on [8192 x 8192] x [8192 x 2048] (the decoder's down projection: A is 128 MiB, more
// than L2): the plain order re-reads A from DRAM in every wave.
static int choose_group_m(int tiles_m, int tiles_n, int concurrent, double a_tile_bytes, double b_tile_bytes, size_t l2_bytes) {
  const int forced = option(OPT_gemm_group_m, 0);
  if (forced > 0) return forced < tiles_m ? forced : tiles_m;
  const double l2 = l2_bytes ? (double)l2_bytes : 100e6;
  if (tiles_m * a_tile_bytes + tiles_n * b_tile_bytes <= 0.85 * l2) return tiles_m;
  int best = tiles_m;
  double best_ws = 1e30;
  for (int g = 1; g <= tiles_m; ++g) {
    const int cols = (concurrent + g - 1) / g;
    const double ws = g * a_tile_bytes + (cols < tiles_n ? cols : tiles_n) * b_tile_bytes;
    if (ws < best_ws) { best_ws = ws; best = g; }
  }
  return best;
}


namespace gemm {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int A_BYTES = BM * BK * 2;  // 16 KiB
constexpr int THREADS = 192;      // TMA warp, MMA warp, four epilogue warps
constexpr int MAX_THREADS = 320;  // ... or eight epilogue warps: two per TMEM lane quarter, each taking half the columns
// Eight pay when the epilogue is the longer stage of a tile or sits in the tail: short K, an activation
// to evaluate, or so few tiles that the last epilogue is exposed (measured with the TMA-store epilogue:
// 8192 x 2304 x 768 808 -> 1034 TFLOP/s, with GELU 562 -> 766, 8192 x 768 x 3072 900 -> 971); long-K
// products with many tiles run 1-2 % faster with four.
static inline int launch_threads(int64_t M, int64_t N, int64_t K, int act, int sm_count) {
  const int64_t forced = option(OPT_gemm_epi_warps, 0);
  if (forced) return forced == 8 ? MAX_THREADS : THREADS;
  const int64_t tiles = ((M + 255) / 256) * ((N + 255) / 256);
  return (act != 0 || K <= 1536 || tiles <= sm_count) ? MAX_THREADS : THREADS;
}

// Output staging for the TMA-store epilogue: 32 KiB shared by the epilogue warps, in 4 KiB slots of
// 32 rows x 128 bytes (two slots per warp with four epilogue warps, one with eight).
constexpr int STAGING_BYTES = 32 * 1024;
constexpr int SLOT_BYTES = 4096;

template <int BN, int STAGES>
struct Cfg {
  static constexpr int B_BYTES = BK * BN * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 16;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + BAR_BYTES + 1024;
  static constexpr int TMEM_COLS = 2 * BN;
};

template <typename OutT>
__device__ __forceinline__ void store_row_chunk(OutT *crow, const __half *rrow, const uint32_t (&acc)[32],
                                                int col0, int N, bool vec_ok);

template <>
__device__ __forceinline__ void store_row_chunk<__half>(__half *crow, const __half *rrow,
                                                        const uint32_t (&acc)[32], int col0, int N,
                                                        bool vec_ok) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const int c = col0 + g * 8;
    float f[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(acc[g * 8 + e]);
    if (vec_ok && c + 8 <= N) {
      if (rrow) {
        Vec16<__half> r;
        r.raw = *reinterpret_cast<const uint4 *>(rrow + c);
        float rf[8];
        r.unpack(rf);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] += rf[e];
      }
      Vec16<__half> o;
      o.pack(f);
      *reinterpret_cast<uint4 *>(crow + c) = o.raw;
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (c + e < N) crow[c + e] = __float2half_rn(f[e] + (rrow ? __half2float(rrow[c + e]) : 0.f));
    }
  }
}

template <>
__device__ __forceinline__ void store_row_chunk<float>(float *crow, const __half *rrow,
                                                       const uint32_t (&acc)[32], int col0, int N,
                                                       bool vec_ok) {
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    const int c = col0 + g * 4;
    float f[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) f[e] = __uint_as_float(acc[g * 4 + e]);
    if (rrow) {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (c + e < N) f[e] += __half2float(rrow[c + e]);
    }
    if (vec_ok && c + 4 <= N) {
      *reinterpret_cast<float4 *>(crow + c) = make_float4(f[0], f[1], f[2], f[3]);
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (c + e < N) crow[c + e] = f[e];
    }
  }
}

// Optional per-column bias and activation applied to the accumulators before the residual is added:
// C = act(A.B + bias) + residual.  act 1: GELU in its tanh form, 0.5 x (1 + tanh(0.797885 x + 0.035677 x^3))
// (the constants of gelu_kernel, test/python/triton/test_gelu.py:25-54; GPT-2's "gelu_new").
struct EpiArgs {
  const __half *bias;  // [N] or null
  int act;             // 0 none, 1 GELU (tanh form)
};

__device__ __forceinline__ float gelu_tanh_f32(float x) {
  const float u = 0.797885f * x + 0.035677f * x * x * x;
  // 1 + tanh(u) = 2 - 2 / (1 + e^{2u}); the fast division (2 ulp) keeps the epilogue off the slow path the
  // IEEE one takes once e^{2u} overflows
  return 0.5f * x * (2.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * u)));
}

// For fp16 outputs: tanh as one special-function instruction (absolute error ~5e-4, the size of the
// output's own rounding step); fp32 outputs keep the exp-based form above.
__device__ __forceinline__ float gelu_tanh_fast(float x) {
  const float u = 0.797885f * x + 0.035677f * x * x * x;
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  const float hx = 0.5f * x;
  return fmaf(hx, t, hx);
}

template <bool FAST>
__device__ __forceinline__ void apply_bias_act(uint32_t (&acc)[32], const EpiArgs &epi, int col0, int N) {
  if (epi.bias) {
    if (col0 + 32 <= N && (reinterpret_cast<uintptr_t>(epi.bias + col0) & 15u) == 0) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        Vec16<__half> b;
        b.raw = __ldg(reinterpret_cast<const uint4 *>(epi.bias + col0 + g * 8));
        float bf[8];
        b.unpack(bf);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g * 8 + e] = __float_as_uint(__uint_as_float(acc[g * 8 + e]) + bf[e]);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 32; ++e)
        if (col0 + e < N) acc[e] = __float_as_uint(__uint_as_float(acc[e]) + __half2float(__ldg(epi.bias + col0 + e)));
    }
  }
  if (epi.act == 1) {
#pragma unroll
    for (int e = 0; e < 32; ++e)
      acc[e] = __float_as_uint(FAST ? gelu_tanh_fast(__uint_as_float(acc[e])) : gelu_tanh_f32(__uint_as_float(acc[e])));
  }
}

// TMA-store epilogue.  A warp converts its 32 accumulator rows to the output type, writes them into a
// 4 KiB slot of shared memory in the 128-byte-swizzle layout (row r, 16-byte chunk c at chunk c ^ (r & 7):
// conflict-free for one row per lane) and lane 0 issues one tiled bulk store for the slot: 64 fp16 or
// 32 fp32 columns x 32 rows.  The store engine writes whole 128-byte row segments and clips at the
// matrix edges, where the direct path has each lane write 16-byte pieces of its own row.
template <typename OutT>
struct StoreStager {
  uint32_t buf0;            // shared address of this warp's first slot (1024-aligned)
  uint8_t *gen0;            // the same slot through a generic pointer
  int nbuf;                 // slots this warp owns: 1 or 2
  int n;                    // stores issued so far
  const CUtensorMap *tm;
  int lane;

  __device__ __forceinline__ uint32_t off() const { return (uint32_t)(n & (nbuf - 1)) * SLOT_BYTES; }
  // the bulk store that last used the slot has finished reading it
  __device__ __forceinline__ void acquire() {
    if (lane == 0) {
      if (nbuf == 2) tc::bulk_wait_group_read<1>();
      else tc::bulk_wait_group_read<0>();
    }
    __syncwarp();
  }
  __device__ __forceinline__ void release(int x, int y) {
    tc::fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tc::tma_store_2d(tm, buf0 + off(), x, y);
      tc::bulk_commit_group();
    }
    ++n;
  }
  __device__ __forceinline__ void drain() {
    if (lane == 0) tc::bulk_wait_group_read<0>();
    __syncwarp();
  }
  // 32 accumulator columns [col0, col0 + 32) of this lane's row; rrow: residual row or null
  __device__ __forceinline__ void put32(const uint32_t (&acc)[32], const __half *rrow, int r_vec, int col0, int row0w,
                                        int N);
};

template <>
__device__ __forceinline__ void StoreStager<__half>::put32(const uint32_t (&acc)[32], const __half *rrow, int r_vec,
                                                           int col0, int row0w, int N) {
  const int h = (col0 >> 5) & 1;  // which half of the 64-column slot
  if (h == 0) acquire();
  uint8_t *row = gen0 + off() + lane * 128;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const int c = col0 + g * 8;
    float f[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(acc[g * 8 + e]);
    if (rrow) {
      if (r_vec && c + 8 <= N) {
        Vec16<__half> r;
        r.raw = *reinterpret_cast<const uint4 *>(rrow + c);
        float rf[8];
        r.unpack(rf);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] += rf[e];
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (c + e < N) f[e] += __half2float(rrow[c + e]);
      }
    }
    Vec16<__half> o;
    o.pack(f);
    *reinterpret_cast<uint4 *>(row + (((h * 4 + g) ^ (lane & 7)) << 4)) = o.raw;
  }
  if (h == 1) release(col0 - 32, row0w);
}

template <>
__device__ __forceinline__ void StoreStager<float>::put32(const uint32_t (&acc)[32], const __half *rrow, int r_vec,
                                                          int col0, int row0w, int N) {
  (void)r_vec;
  acquire();
  uint8_t *row = gen0 + off() + lane * 128;
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    const int c = col0 + g * 4;
    float f[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) f[e] = __uint_as_float(acc[g * 4 + e]);
    if (rrow) {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (c + e < N) f[e] += __half2float(rrow[c + e]);
    }
    *reinterpret_cast<float4 *>(row + ((g ^ (lane & 7)) << 4)) = make_float4(f[0], f[1], f[2], f[3]);
  }
  release(col0, row0w);
}

template <typename OutT>
__device__ __forceinline__ StoreStager<OutT> make_stager(uint8_t *staging, uint32_t staging_addr, const CUtensorMap *tm,
                                                         int warp, int lane) {
  const int n_epi = (blockDim.x >> 5) - 2;           // 4 or 8 epilogue warps
  const int per_warp = STAGING_BYTES / n_epi;        // 8 KiB or 4 KiB
  StoreStager<OutT> st;
  st.buf0 = staging_addr + (uint32_t)((warp - 2) * per_warp);
  st.gen0 = staging + (warp - 2) * per_warp;
  st.nbuf = per_warp / SLOT_BYTES;
  st.n = 0;
  st.tm = tm;
  st.lane = lane;
  return st;
}

// Drains this warp's share of one accumulator buffer.  taddr: TMEM address of the warp's lane quarter at
// the buffer's first column; `width` output columns starting at col_base.  With two warps per lane
// quarter (halves == 2) the columns are split in units of 64 so that a slot is always filled by one warp.
template <typename OutT, int EPI, int BN>
__device__ __forceinline__ void drain_accumulator(uint32_t taddr, int width, int col_base, int row, int row0w, int M,
                                                  int N, OutT *C, int64_t ldc, const __half *R, int64_t ldr, int vec_ok,
                                                  const EpiArgs &epi, int halves, int half, StoreStager<OutT> &st,
                                                  int use_tma, int r_vec) {
  const int units = (EPI == 1 ? BN / 2 : width) / 64;
  const int mid = halves == 1 ? units : (units + 1) / 2;
  const int ubeg = half == 0 ? 0 : mid, uend = half == 0 ? mid : units;
  OutT *crow = C + (int64_t)row * ldc;
  const __half *rrow = (R && row < M) ? R + (int64_t)row * ldr : nullptr;
#pragma unroll 1
  for (int c = 2 * ubeg; c < 2 * uend; ++c) {
    uint32_t v[32];
    if constexpr (EPI == 1) {
      uint32_t u[32];
      tc::tmem_ld_32x32(taddr + (uint32_t)(c * 32), v);
      tc::tmem_ld_32x32(taddr + (uint32_t)(BN / 2 + c * 32), u);
      tc::tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const float gv = __uint_as_float(v[e]);
        v[e] = __float_as_uint(__fdividef(gv, 1.0f + __expf(-gv)) * __uint_as_float(u[e]));
      }
    } else {
      tc::tmem_ld_32x32(taddr + (uint32_t)(c * 32), v);
      tc::tmem_ld_wait();
    }
    const int col0 = col_base + c * 32;
    if constexpr (EPI == 2) apply_bias_act<sizeof(OutT) == 2>(v, epi, col0, N);
    if (use_tma) st.put32(v, rrow, r_vec, col0, row0w, N);
    else if (row < M && col0 < N) store_row_chunk<OutT>(crow, rrow, v, col0, N, vec_ok != 0);
  }
}

// EPI == 1 (SwiGLU, BN = 256, fp16 out): B is a [K, 2*N] gate|up matrix; a tile's B operand is made
// of 128 gate columns [col0, col0+128) and the 128 up columns [N+col0, N+col0+128), so accumulator
// columns c and 128+c belong to output column col0+c and the epilogue writes silu(gate) * up.
// BT: B is given transposed, Bt[N, K] row-major (C = A @ Bt^T): it is then the K-major operand form,
// loaded as 128-row x 64-k boxes like A.
template <int BN, int STAGES, typename OutT, int EPI = 0, bool BT = false>
__global__ void __launch_bounds__(MAX_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               OutT *__restrict__ C, const __half *__restrict__ R, int M, int N, int K, int64_t ldc,
               int64_t ldr, int tiles_m, int tiles_n, int group_m, int vec_ok, uint32_t b_lbo, uint32_t b_sbo,
               int full_items, int split, const EpiArgs epi, const __grid_constant__ CUtensorMap tmC, int use_tma,
               int r_vec) {
  using cfg = Cfg<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = tc::smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
  uint8_t *smem = smem_raw + pad;
  const uint32_t smem_addr = raw_addr + pad;

  uint8_t *staging = smem + STAGES * cfg::STAGE_BYTES;
  const uint32_t staging_addr = smem_addr + STAGES * cfg::STAGE_BYTES;
  uint64_t *bars = reinterpret_cast<uint64_t *>(staging + STAGING_BYTES);
  const uint32_t bar0 = staging_addr + STAGING_BYTES;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tc::mbar_init(full_bar(s), 1);
      tc::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      tc::mbar_init(tfull_bar(a), 1);
      tc::mbar_init(tempty_bar(a), (blockDim.x >> 5) - 2);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    tc::fence_barrier_init();
    tc::prefetch_tensormap(&tmA);
    tc::prefetch_tensormap(&tmB);
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
  pdl_wait();  // barriers and TMEM are set up; global memory is touched from here on

  // Work items.  Items [0, full_items) are whole 128 x BN tiles; each remaining tile -- the ones of
  // the last, partial wave over the SMs -- is cut into `split` column slices of BN/split, so that
  // wave finishes in 1/split of a tile time instead of leaving most SMs idle for a whole one.
  const int num_tiles = tiles_m * tiles_n;
  const int num_items = full_items + (num_tiles - full_items) * split;
  const int num_kb = (K + BK - 1) / BK;
  struct Item { int tm, col0, width; };
  auto item_of = [&](int i) {
    Item it;
    int tile = i, sub = 0;
    it.width = BN;
    if (i >= full_items) {
      const int k = i - full_items;
      tile = full_items + k / split;
      sub = k - (k / split) * split;
      it.width = BN / split;
    }
    int tn;
    tile_to_mn(tile, tiles_m, tiles_n, group_m, &it.tm, &tn);
    it.col0 = tn * (EPI == 1 ? BN / 2 : BN) + sub * it.width;
    return it;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        const Item w = item_of(item);
        const int chunks = w.width / 64;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!tc::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t sa = smem_addr + stage * cfg::STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          tc::mbar_arrive_expect_tx(full_bar(stage), (uint32_t)(A_BYTES + (BT ? BN * 128 : chunks * BK * 128)));
          tc::tma_load_2d(sa, &tmA, kb * BK, w.tm * BM, full_bar(stage));
          if constexpr (BT) {
            // rows of Bt = output columns; boxes of 128 rows x 64 k (the whole BN is always loaded)
#pragma unroll
            for (int j = 0; j < BN / 128; ++j) {
              int n0 = w.col0 + j * 128;
              if (EPI == 1 && j >= 1) n0 = N + w.col0;  // the matching up rows
              tc::tma_load_2d(sb + j * (128 * 128), &tmB, kb * BK, n0, full_bar(stage));
            }
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) {
              int x = w.col0 + j * 64;
              if (EPI == 1 && j >= BN / 128) x = N + w.col0 + (j - BN / 128) * 64;  // the matching up columns
              if (j < chunks) tc::tma_load_2d(sb + j * (BK * 128), &tmB, x, kb * BK, full_bar(stage));
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int t = 0;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++t) {
        const uint32_t idesc = tc::make_idesc_f16_f32(BM, item_of(item).width, 0, BT ? 0 : 1);
        const int acc = t & 1;
        if (!tc::mbar_wait(tempty_bar(acc), ((uint32_t)(t >> 1) & 1u) ^ 1u, abort_flag)) break;
        tc::tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!tc::mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
          tc::tc_fence_after();
          const uint32_t sa = smem_addr + stage * cfg::STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          const uint64_t adesc = tc::make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t bdesc = BT ? tc::make_smem_desc_sw128(sb, 16, 1024) : tc::make_smem_desc_sw128(sb, b_lbo, b_sbo);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // A (and a K-major B): +32 bytes inside the 128-byte swizzle row; N-major B: +16 k-rows = 2 atoms.
            tc::mma_f16_ss(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(BT ? k * 2 : k * 128), idesc,
                           (kb | k) != 0 ? 1u : 0u);
          }
          tc::mma_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) tc::mma_commit(tfull_bar(acc));
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5 or 2..9)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    const int halves = ((blockDim.x >> 5) - 2) >> 2, half = (warp - 2) >> 2;  // column share of this warp
    StoreStager<OutT> st = make_stager<OutT>(staging, staging_addr, &tmC, warp, lane);
    int t = 0;
    for (int item = blockIdx.x; item < num_items; item += gridDim.x, ++t) {
      const Item w = item_of(item);
      const int acc = t & 1;
      if (!tc::mbar_wait(tfull_bar(acc), (uint32_t)(t >> 1) & 1u, abort_flag)) break;
      tc::tc_fence_after();
      const int row0w = w.tm * BM + q * 32;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
      drain_accumulator<OutT, EPI, BN>(taddr, w.width, w.col0, row0w + lane, row0w, M, N, C, ldc, R, ldr, vec_ok, epi,
                                       halves, half, st, use_tma, r_vec);
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(tempty_bar(acc));
    }
    if (use_tma) st.drain();  // shared memory stays allocated until the last store has read it
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
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&g_gemm_status, (int)HEXB_ERR_TIMEOUT);
}

// Any shape / alignment / K == 0: plain CUDA-core tiles.  Only the shapes the tensor-core path
// cannot take (leading dimensions or pointers that break the 16-byte TMA rule) land here.
template <typename OutT>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const __half *__restrict__ A, const __half *__restrict__ B, OutT *__restrict__ C,
                 const __half *__restrict__ R, int64_t M, int64_t N, int64_t K, int64_t lda,
                 int64_t ldb, int64_t ldc, int64_t ldr, int bt, const EpiArgs epi) {
  __shared__ float As[16][17], Bs[16][17];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t row = (int64_t)blockIdx.y * 16 + ty, col = (int64_t)blockIdx.x * 16 + tx;
  float acc = 0.f;
  for (int64_t k0 = 0; k0 < K; k0 += 16) {
    As[ty][tx] = (row < M && k0 + tx < K) ? __half2float(A[row * lda + k0 + tx]) : 0.f;
    Bs[ty][tx] = (k0 + ty < K && col < N) ? __half2float(bt ? B[col * ldb + k0 + ty] : B[(k0 + ty) * ldb + col]) : 0.f;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) acc = fmaf(As[ty][k], Bs[k][tx], acc);
    __syncthreads();
  }
  if (row < M && col < N) {
    if (epi.bias) acc += __half2float(epi.bias[col]);
    if (epi.act == 1) acc = gelu_tanh_f32(acc);
    if (R) acc += __half2float(R[row * ldr + col]);
    C[row * ldc + col] = from_f32<OutT>(acc);
  }
}


// ---------------------------------------------------------------------------------------------
// CTA-pair form (cta_group::2): a cluster of two CTAs computes a 256 x 256 tile.  Each CTA loads
// its own 128 rows of A and its own half (128 columns) of the B tile, so per k-block a CTA writes
// 32 KiB into shared memory instead of 48 and the tensor cores read each B half once for both CTAs;
// six pipeline stages fit.  The leader CTA (cluster rank 0) issues the 256 x 256 x 16 MMAs; their
// completion is multicast to the stage barriers of both CTAs; each CTA's epilogue warps drain their
// own 128 accumulator rows and signal the leader when the buffer is free.  Every wait is bounded
// and both CTAs meet at a cluster barrier before they exit.
namespace pair {
constexpr int STAGES = 6;
constexpr int BN = 256;
constexpr int B_HALF_BYTES = BK * 128 * 2;             // this CTA's 128 columns of the B tile: 16 KiB
constexpr int STAGE_BYTES = A_BYTES + B_HALF_BYTES;    // 32 KiB
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + (2 * STAGES + 4) * 8 + 16 + 1024;
constexpr int TMEM_COLS = 512;
}  // namespace pair

template <typename OutT, int EPI, bool BT = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(MAX_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    OutT *__restrict__ C, const __half *__restrict__ R, int M, int N, int K, int64_t ldc,
                    int64_t ldr, int tiles_m, int tiles_n, int group_m, int vec_ok, const EpiArgs epi,
                    const __grid_constant__ CUtensorMap tmC, int use_tma, int r_vec, int full_items, int split) {
  using namespace pair;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = tc::smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
  uint8_t *smem = smem_raw + pad;
  const uint32_t smem_addr = raw_addr + pad;
  uint8_t *staging = smem + STAGES * STAGE_BYTES;
  const uint32_t staging_addr = smem_addr + STAGES * STAGE_BYTES;
  uint64_t *bars = reinterpret_cast<uint64_t *>(staging + STAGING_BYTES);
  const uint32_t bar0 = staging_addr + STAGING_BYTES;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };                   // used in the leader only
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };       // one per CTA
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };   // one per CTA
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };  // used in the leader only
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = tc::cluster_ctarank();
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tc::mbar_init(full_bar(s), 1);
      tc::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      tc::mbar_init(tfull_bar(a), 1);
      tc::mbar_init(tempty_bar(a), 2 * ((blockDim.x >> 5) - 2));  // the epilogue warps of both CTAs of the pair
    }
    *abort_flag = 0;
    tc::fence_barrier_init();
    tc::prefetch_tensormap(&tmA);
    tc::prefetch_tensormap(&tmB);
  }
  if (warp == 1) {
    tc::tmem_alloc_pair(tc::smem_u32(tmem_slot), TMEM_COLS);
    tc::tmem_relinquish_pair();
  }
  tc::tc_fence_before();
  tc::cluster_sync_all();  // barriers of both CTAs are initialised before anything signals them
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();  // barriers and TMEM are set up; global memory is touched from here on

  constexpr int OUT_COLS = EPI == 1 ? BN / 2 : BN;
  const int num_tiles = tiles_m * tiles_n;       // tiles of 256 rows x OUT_COLS output columns
  const int num_kb = (K + BK - 1) / BK;
  // Work items: the tiles of the full waves, then the tiles of the last, partial wave cut into `split`
  // column slices (256 x 128 with split == 2) so that the tail occupies the clusters for half a tile time.
  const int num_items = full_items + (num_tiles - full_items) * split;
  struct Item { int tm, col0, width; };
  auto item_of = [&](int i) {
    Item it;
    int tile = i, sub = 0;
    it.width = BN;
    if (i >= full_items) {
      const int k = i - full_items;
      tile = full_items + k / split;
      sub = k - (k / split) * split;
      it.width = BN / split;
    }
    int tn;
    tile_to_mn(tile, tiles_m, tiles_n, group_m, &it.tm, &tn);
    it.col0 = tn * OUT_COLS + sub * it.width;
    return it;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = cluster_id; item < num_items && ok; item += num_clusters) {
        const Item w = item_of(item);
        const int col0 = w.col0;
        const int row0 = w.tm * 256 + (int)rank * BM;
        const int half_w = w.width / 2;  // columns of B this CTA supplies: 128, or 64 for a slice
        // this CTA's half of the B tile: plain = columns [col0 + half_w*rank, +half_w);
        // SwiGLU = rank 0 the gate columns [col0, +128), rank 1 the matching up columns [N + col0, +128)
        const int bx = EPI == 1 ? (rank == 0 ? col0 : N + col0) : col0 + (int)rank * half_w;
        // bytes per CTA and stage: A, plus the B boxes actually loaded (the K-major form always loads its 128-row box)
        const uint32_t stage_tx = (uint32_t)A_BYTES + (BT ? (uint32_t)B_HALF_BYTES : (uint32_t)half_w * BK * 2u);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!tc::mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t sa = smem_addr + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          const uint32_t leader_full = tc::map_to_rank(full_bar(stage), 0);
          if (rank == 0) tc::mbar_arrive_expect_tx(full_bar(stage), 2u * stage_tx);  // both CTAs' bytes
          tc::tma_load_2d_pair(sa, &tmA, kb * BK, row0, leader_full);
          if constexpr (BT) {
            tc::tma_load_2d_pair(sb, &tmB, kb * BK, bx, leader_full);  // 128 rows of Bt x 64 k (a slice uses the first 64)
          } else {
            tc::tma_load_2d_pair(sb, &tmB, bx, kb * BK, leader_full);
            if (half_w > 64) tc::tma_load_2d_pair(sb + BK * 128, &tmB, bx + 64, kb * BK, leader_full);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int t = 0;
      for (int item = cluster_id; item < num_items && ok; item += num_clusters, ++t) {
        const uint32_t idesc = tc::make_idesc_f16_f32(256, item_of(item).width, 0, BT ? 0 : 1);
        const int acc = t & 1;
        if (!tc::mbar_wait(tempty_bar(acc), ((uint32_t)(t >> 1) & 1u) ^ 1u, abort_flag)) break;
        tc::tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!tc::mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
          tc::tc_fence_after();
          const uint32_t sa = smem_addr + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          const uint64_t adesc = tc::make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t bdesc = BT ? tc::make_smem_desc_sw128(sb, 16, 1024) : tc::make_smem_desc_sw128(sb, BK * 128, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            tc::mma_f16_ss_pair(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(BT ? k * 2 : k * 128), idesc,
                                (kb | k) != 0 ? 1u : 0u);
          tc::mma_commit_pair_mc(empty_bar(stage), 3);  // frees the stage in both CTAs
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) tc::mma_commit_pair_mc(tfull_bar(acc), 3);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5 or 2..9, both CTAs)
    const int q = warp & 3;
    const int halves = ((blockDim.x >> 5) - 2) >> 2, half = (warp - 2) >> 2;
    StoreStager<OutT> st = make_stager<OutT>(staging, staging_addr, &tmC, warp, lane);
    int t = 0;
    for (int item = cluster_id; item < num_items; item += num_clusters, ++t) {
      const Item w = item_of(item);
      const int acc = t & 1;
      if (!tc::mbar_wait(tfull_bar(acc), (uint32_t)(t >> 1) & 1u, abort_flag)) break;
      tc::tc_fence_after();
      const int row0w = w.tm * 256 + (int)rank * BM + q * 32;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
      drain_accumulator<OutT, EPI, BN>(taddr, w.width, w.col0, row0w + lane, row0w, M, N, C, ldc, R, ldr, vec_ok, epi, halves,
                                       half, st, use_tma, r_vec);
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive_cluster(tc::map_to_rank(tempty_bar(acc), 0));
    }
    if (use_tma) st.drain();
  }

  // ------------------------------------------------------------ teardown
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc::tc_fence_before();
  tc::cluster_sync_all();  // nobody leaves while the peer may still signal or read this CTA
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&g_gemm_status, (int)HEXB_ERR_TIMEOUT);
}

// Tensor map of the output for the TMA-store epilogue (use == 0: the lanes store their rows directly).
struct StoreMap {
  CUtensorMap tm;
  int use;
  int r_vec;  // the residual rows can be read with 16-byte loads
};

template <typename OutT>
static StoreMap make_store_map(OutT *C, const __half *R, int64_t M, int64_t N, int64_t ldc, int64_t ldr,
                               const CUtensorMap &fallback) {
  StoreMap sm;
  sm.tm = fallback;
  sm.use = 0;
  sm.r_vec = R && aligned16(R) && ldr % 8 == 0;
  if (!option(OPT_gemm_tma_store, 1) || !aligned16(C) || (ldc * (int64_t)sizeof(OutT)) % 16) return sm;
  const uint64_t dims[2] = {(uint64_t)N, (uint64_t)M};
  int rc;
  if (sizeof(OutT) == 2) {
    const uint64_t strides[1] = {(uint64_t)ldc * 2};
    const uint32_t box[2] = {64, 32};
    rc = encode_tmap_f16_sw128(&sm.tm, C, 2, dims, strides, box);
  } else {
    const uint32_t box[2] = {32, 32};
    rc = encode_tmap_f32_sw128_2d(&sm.tm, C, dims, (uint64_t)ldc * 4, box);
  }
  if (rc == HEXB_OK) sm.use = 1;
  else sm.tm = fallback;
  return sm;
}

template <typename OutT, int EPI, bool BT = false>
static int launch_tc_pair(const EpiArgs &epi, const StoreMap &sm, const CUtensorMap &tmA, const CUtensorMap &tmB, OutT *C, const __half *R, int M, int N,
                          int K, int64_t ldc, int64_t ldr, int vec_ok, int sm_count, size_t l2_bytes, cudaStream_t st) {
  static PerDeviceOnce attr_done;
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = gemm_tc_pair_kernel<OutT, EPI, BT>;
  if (!attr_done.is_done(dev)) {
    HEXB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, pair::SMEM_BYTES));
    attr_done.mark(dev);
  }
  constexpr int OUT_COLS = EPI == 1 ? pair::BN / 2 : pair::BN;
  const int tiles_m = (M + 255) / 256, tiles_n = (N + OUT_COLS - 1) / OUT_COLS;
  const int tiles = tiles_m * tiles_n;
  const int max_clusters = sm_count / 2;
  // the tiles of the last partial wave are cut in two column slices when both halves still fit one wave
  int full_items = tiles, split = 1;
  if (EPI != 1 && tiles > max_clusters && option(OPT_gemm_tail_split, 1)) {
    const int rem = tiles % max_clusters;
    if (rem > 0 && 2 * rem <= max_clusters) {
      full_items = tiles - rem;
      split = 2;
    }
  }
  const int items = full_items + (tiles - full_items) * split;
  const int clusters = items < max_clusters ? items : max_clusters;
  const int group_m = choose_group_m(tiles_m, tiles_n, clusters, 256.0 * K * 2, (EPI == 1 ? 2.0 : 1.0) * OUT_COLS * K * 2, l2_bytes);
  launch_pdl(kern, dim3(2 * clusters), dim3(launch_threads(M, N, K, EPI == 1 ? 1 : epi.act, sm_count)),
             (size_t)pair::SMEM_BYTES, st, tmA, tmB, C, R, M, N, K, ldc, ldr, tiles_m, tiles_n, group_m, vec_ok, epi, sm.tm,
             sm.use, sm.r_vec, full_items, split);
  return check_launch("gemm_tc_pair");
}

template <int BN, int STAGES, typename OutT, int EPI = 0, bool BT = false>
static int launch_tc(const EpiArgs &epi, const StoreMap &sm, const CUtensorMap &tmA, const CUtensorMap &tmB, OutT *C, const __half *R, int M,
                     int N, int K, int64_t ldc, int64_t ldr, int vec_ok, int sm_count, size_t l2_bytes,
                     cudaStream_t st) {
  using cfg = Cfg<BN, STAGES>;
  static PerDeviceOnce attr_done;
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = gemm_tc_kernel<BN, STAGES, OutT, EPI, BT>;
  if (!attr_done.is_done(dev)) {
    HEXB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg::SMEM_BYTES));
    attr_done.mark(dev);
  }
  constexpr int OUT_COLS = EPI == 1 ? BN / 2 : BN;  // output columns per tile
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + OUT_COLS - 1) / OUT_COLS;
  const int tiles = tiles_m * tiles_n;
  // split the tiles of the last partial wave into column slices (>= 64 wide) while they still fit one wave
  int full_items = tiles / sm_count * sm_count, split = 1;
  const int rem = tiles - full_items;
  if (EPI == 0 && !BT && rem > 0 && option(OPT_gemm_tail_split, 1)) {
    while (split * 2 <= BN / 64 && rem * split * 2 <= sm_count) split *= 2;
  }
  if (split == 1) full_items = tiles;
  const int items = full_items + (tiles - full_items) * split;
  const int grid = items < sm_count ? items : sm_count;
  const uint32_t lbo = (uint32_t)HEXB_DEV_OPTION(OPT_gemm_b_lbo, BK * 128);
  const uint32_t sbo = (uint32_t)HEXB_DEV_OPTION(OPT_gemm_b_sbo, 1024);
  const int group_m = choose_group_m(tiles_m, tiles_n, grid, (double)BM * K * 2, (EPI == 1 ? 2.0 : 1.0) * OUT_COLS * K * 2, l2_bytes);
  launch_pdl(kern, dim3(grid), dim3(launch_threads(M, N, K, EPI == 1 ? 1 : epi.act, sm_count)), (size_t)cfg::SMEM_BYTES, st,
             tmA, tmB, C, R, M, N, K, ldc, ldr, tiles_m, tiles_n, group_m, vec_ok, lbo, sbo, full_items, split, epi, sm.tm,
             sm.use, sm.r_vec);
  return check_launch("gemm_tc");
}

// EPI 0: plain product (+ residual); EPI 2: bias / activation applied in the epilogue as well.
template <typename OutT, bool BT = false, int EPI = 0>
static int matmul_impl(const __half *A, const __half *B, OutT *C, const __half *R, int64_t M, int64_t N,
                       int64_t K, int64_t lda, int64_t ldb, int64_t ldc, cudaStream_t st,
                       const EpiArgs epi = EpiArgs{nullptr, 0}) {
  DeviceInfo di;
  if (int s = current_device(&di)) return s;
  const int64_t ldr = ldc;
  const bool tc_ok = K > 0 && lda % 8 == 0 && ldb % 8 == 0 && aligned16(A) && aligned16(B) &&
                     M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31) &&
                     !option(OPT_gemm_force_simt, 0);
  if (!tc_ok) {
    dim3 grid((unsigned)((N + 15) / 16), (unsigned)((M + 15) / 16));
    if (grid.y > 65535) return HEXB_ERR_UNSUPPORTED;
    gemm_simt_kernel<OutT><<<grid, 256, 0, st>>>(A, B, C, R, M, N, K, lda, ldb, ldc, ldr, BT ? 1 : 0, epi);
    return check_launch("gemm_simt");
  }
  CUtensorMap tmA, tmB;
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    const uint64_t strides[1] = {(uint64_t)lda * 2};
    const uint32_t box[2] = {BK, BM};
    if (int s = encode_tmap_f16_sw128(&tmA, A, 2, dims, strides, box)) return s;
  }
  if constexpr (BT) {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    const uint64_t strides[1] = {(uint64_t)ldb * 2};
    const uint32_t box[2] = {BK, 128};
    if (int s = encode_tmap_f16_sw128(&tmB, B, 2, dims, strides, box)) return s;
  } else {
    const uint64_t dims[2] = {(uint64_t)N, (uint64_t)K};
    const uint64_t strides[1] = {(uint64_t)ldb * 2};
    const uint32_t box[2] = {64, BK};
    if (int s = encode_tmap_f16_sw128(&tmB, B, 2, dims, strides, box)) return s;
  }
  constexpr int EV = 16 / (int)sizeof(OutT);
  const int vec_ok = (ldc % EV == 0) && aligned16(C) && (!R || (sizeof(OutT) == 2 && aligned16(R)));
  const StoreMap sm = make_store_map<OutT>(C, R, M, N, ldc, ldr, tmA);
  const int tiles_m = (int)((M + BM - 1) / BM);
  int bn = option(OPT_gemm_bn, 0);
  if (bn != 64 && bn != 128 && bn != 256) {
    bn = 256;
    if (N <= 64 || (int64_t)tiles_m * ((N + 127) / 128) < di.sm_count / 2) bn = 64;
    else if (N <= 128 || (int64_t)tiles_m * ((N + 255) / 256) < di.sm_count) bn = 128;
  }
  // CTA-pair kernel from 256 x 256 tiles for 27 % of the SMs on (40 tiles on 148 SMs).  Below a full wave
  // the alternative is 128 x 128 tiles on every SM, which fetch twice the operand bytes per FLOP through L2
  // and are bound by that: [1024 x 4096 x 4096] 39.7 us on 256 single-CTA tiles against 27.3 us on 64 pair
  // tiles, [768 x 4096 x 4096] 39.2 against 25.6; with 32 pair tiles ([512 x 4096 x 4096], [1024 x 2048 x
  // 2048]) the idle SMs weigh more and the single-CTA kernel stays 8-15 % ahead.
  const int64_t pair_tiles = ((M + 255) / 256) * ((N + 255) / 256);
  if (option(OPT_gemm_bn, 0) == 0 && option(OPT_gemm_pair, 1) &&
      pair_tiles >= option(OPT_gemm_pair_min_tiles, (di.sm_count * 27 + 99) / 100))
    return launch_tc_pair<OutT, EPI, BT>(epi, sm, tmA, tmB, C, R, (int)M, (int)N, (int)K, ldc, ldr, vec_ok, di.sm_count, di.l2_bytes, st);
  if (BT && bn == 64) bn = 128;  // the transposed form loads Bt in 128-row boxes
  switch (bn) {
    case 64:
      return launch_tc<64, 8, OutT, EPI, false>(epi, sm, tmA, tmB, C, R, (int)M, (int)N, (int)K, ldc, ldr, vec_ok, di.sm_count, di.l2_bytes, st);
    case 128:
      return launch_tc<128, 6, OutT, EPI, BT>(epi, sm, tmA, tmB, C, R, (int)M, (int)N, (int)K, ldc, ldr, vec_ok, di.sm_count, di.l2_bytes, st);
    default:
      return launch_tc<256, 4, OutT, EPI, BT>(epi, sm, tmA, tmB, C, R, (int)M, (int)N, (int)K, ldc, ldr, vec_ok, di.sm_count, di.l2_bytes, st);
  }
}

}  // namespace gemm

int gemm_device_status_fetch_and_clear(int *out) {
  int v = 0, zero = 0;
  HEXB_CUDA_OK(cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int)));
  if (v) HEXB_CUDA_OK(cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int)));
  *out = v;
  return HEXB_OK;
}

}  // namespace hexb

extern "C" int hexb_matmul_f16(const void *A, const void *B, void *C, const void *residual, int64_t M,
                               int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                               int out_dtype, void *stream) {
  using namespace hexb;
  if (M < 0 || N < 0 || K < 0) return HEXB_ERR_BAD_ARG;
  if (out_dtype != HEXB_DT_F16 && out_dtype != HEXB_DT_F32) return HEXB_ERR_UNSUPPORTED;
  if (M == 0 || N == 0) return HEXB_OK;
  if (!C || (K > 0 && (!A || !B))) return HEXB_ERR_BAD_ARG;
  if (lda < K || ldb < N || ldc < N) return HEXB_ERR_BAD_ARG;
  if (out_dtype == HEXB_DT_F16)
    return gemm::matmul_impl<__half>((const __half *)A, (const __half *)B, (__half *)C,
                                     (const __half *)residual, M, N, K, lda, ldb, ldc, (cudaStream_t)stream);
  return gemm::matmul_impl<float>((const __half *)A, (const __half *)B, (float *)C,
                                  (const __half *)residual, M, N, K, lda, ldb, ldc, (cudaStream_t)stream);
}

extern "C" int hexb_matmul_f16_nt(const void *A, const void *Bt, void *C, const void *residual, int64_t M,
                                  int64_t N, int64_t K, int64_t lda, int64_t ldbt, int64_t ldc, int out_dtype,
                                  void *stream) {
  using namespace hexb;
  if (M < 0 || N < 0 || K < 0) return HEXB_ERR_BAD_ARG;
  if (out_dtype != HEXB_DT_F16 && out_dtype != HEXB_DT_F32) return HEXB_ERR_UNSUPPORTED;
  if (M == 0 || N == 0) return HEXB_OK;
  if (!C || (K > 0 && (!A || !Bt))) return HEXB_ERR_BAD_ARG;
  if (lda < K || ldbt < K || ldc < N) return HEXB_ERR_BAD_ARG;
  if (out_dtype == HEXB_DT_F16)
    return gemm::matmul_impl<__half, true>((const __half *)A, (const __half *)Bt, (__half *)C,
                                           (const __half *)residual, M, N, K, lda, ldbt, ldc, (cudaStream_t)stream);
  return gemm::matmul_impl<float, true>((const __half *)A, (const __half *)Bt, (float *)C, (const __half *)residual,
                                        M, N, K, lda, ldbt, ldc, (cudaStream_t)stream);
}

extern "C" int hexb_linear_f16(const void *A, const void *W, const void *bias, const void *residual, void *C,
                               int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldw, int64_t ldc,
                               int w_transposed, int act, int out_dtype, void *stream) {
  using namespace hexb;
  if (M < 0 || N < 0 || K < 0) return HEXB_ERR_BAD_ARG;
  if (out_dtype != HEXB_DT_F16 && out_dtype != HEXB_DT_F32) return HEXB_ERR_UNSUPPORTED;
  if (act != 0 && act != 1) return HEXB_ERR_UNSUPPORTED;
  if (M == 0 || N == 0) return HEXB_OK;
  if (!C || (K > 0 && (!A || !W))) return HEXB_ERR_BAD_ARG;
  if (lda < K || ldc < N || ldw < (w_transposed ? K : N)) return HEXB_ERR_BAD_ARG;
  const gemm::EpiArgs epi{(const __half *)bias, act};
  const __half *a = (const __half *)A, *w = (const __half *)W, *r = (const __half *)residual;
  cudaStream_t st = (cudaStream_t)stream;
  if (!bias && !act) {  // nothing for the epilogue to add: the plain kernels
    if (out_dtype == HEXB_DT_F16) {
      if (w_transposed) return gemm::matmul_impl<__half, true>(a, w, (__half *)C, r, M, N, K, lda, ldw, ldc, st);
      return gemm::matmul_impl<__half, false>(a, w, (__half *)C, r, M, N, K, lda, ldw, ldc, st);
    }
    if (w_transposed) return gemm::matmul_impl<float, true>(a, w, (float *)C, r, M, N, K, lda, ldw, ldc, st);
    return gemm::matmul_impl<float, false>(a, w, (float *)C, r, M, N, K, lda, ldw, ldc, st);
  }
  if (out_dtype == HEXB_DT_F16) {
    if (w_transposed) return gemm::matmul_impl<__half, true, 2>(a, w, (__half *)C, r, M, N, K, lda, ldw, ldc, st, epi);
    return gemm::matmul_impl<__half, false, 2>(a, w, (__half *)C, r, M, N, K, lda, ldw, ldc, st, epi);
  }
  if (w_transposed) return gemm::matmul_impl<float, true, 2>(a, w, (float *)C, r, M, N, K, lda, ldw, ldc, st, epi);
  return gemm::matmul_impl<float, false, 2>(a, w, (float *)C, r, M, N, K, lda, ldw, ldc, st, epi);
}

extern "C" int hexb_matmul_swiglu_f16(const void *A, const void *B_gate_up, void *out, int64_t M, int64_t F,
                                      int64_t K, int64_t lda, int64_t ldb, int64_t ldo, void *stream) {
  using namespace hexb;
  using namespace hexb::gemm;
  if (M < 0 || F < 0 || K < 0) return HEXB_ERR_BAD_ARG;
  if (M == 0 || F == 0) return HEXB_OK;
  if (!A || !B_gate_up || !out || K == 0) return HEXB_ERR_BAD_ARG;
  if (lda < K || ldb < 2 * F || ldo < F) return HEXB_ERR_BAD_ARG;
  if (lda % 8 || ldb % 8 || F % 8 || !aligned16(A) || !aligned16(B_gate_up)) return HEXB_ERR_MISALIGNED;
  if (M >= (1ll << 31) || F >= (1ll << 30) || K >= (1ll << 31)) return HEXB_ERR_UNSUPPORTED;
  DeviceInfo di;
  if (int s = current_device(&di)) return s;
  CUtensorMap tmA, tmB;
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    const uint64_t strides[1] = {(uint64_t)lda * 2};
    const uint32_t box[2] = {BK, BM};
    if (int s = encode_tmap_f16_sw128(&tmA, A, 2, dims, strides, box)) return s;
  }
  {
    const uint64_t dims[2] = {(uint64_t)(2 * F), (uint64_t)K};
    const uint64_t strides[1] = {(uint64_t)ldb * 2};
    const uint32_t box[2] = {64, BK};
    if (int s = encode_tmap_f16_sw128(&tmB, B_gate_up, 2, dims, strides, box)) return s;
  }
  const int vec_ok = (ldo % 8 == 0) && aligned16(out);
  const gemm::StoreMap sm = gemm::make_store_map<__half>((__half *)out, nullptr, M, F, ldo, ldo, tmA);
  if (option(OPT_gemm_pair, 1) && ((M + 255) / 256) * ((F + 127) / 128) >= di.sm_count / 2)
    return launch_tc_pair<__half, 1>(gemm::EpiArgs{nullptr, 0}, sm, tmA, tmB, (__half *)out, nullptr, (int)M, (int)F, (int)K, ldo, ldo, vec_ok,
                                     di.sm_count, di.l2_bytes, (cudaStream_t)stream);
  return launch_tc<256, 4, __half, 1>(gemm::EpiArgs{nullptr, 0}, sm, tmA, tmB, (__half *)out, nullptr, (int)M, (int)F, (int)K, ldo, ldo, vec_ok,
                                      di.sm_count, di.l2_bytes, (cudaStream_t)stream);
}

extern "C" int hexkl_matmul_f16f16_f32(int64_t n_row, int64_t n_col, int64_t n_inner, float *outM,
                                       const void *inAct, const void *inW) {
  return hexb_matmul_f16(inAct, inW, outM, nullptr, n_row, n_col, n_inner, n_inner, n_col, n_col,
                         HEXB_DT_F32, nullptr);
}
