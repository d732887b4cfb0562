// Warp-private bulk-copy rings for the bandwidth-bound row kernels.
//
// The reference tiles operands into a 2 MB scratchpad and ping-pongs DMA transfers against compute
// (qcom_hexagon_backend/lib/Conversion/LinalgToLLVM/VTCMTiling.cpp:231-266,
// lib/Transforms/DoubleBufferGenericS1.cpp:102, bin/runtime/UserDMA/UserDMA.cc:27-172).  The B200
// form: a persistent CTA per SM; every warp owns a ring of SLOTS row buffers in shared memory and
// keeps SLOTS bulk copies (cp.async.bulk global -> shared, completion on an mbarrier) in flight for
// the rows it will process next.  A warp waits for its row, pulls it into registers with 16-byte
// shared loads, immediately re-arms the slot with the copy of a later row, and only then does the
// arithmetic and the global stores -- so the amount of data in flight per SM is set by the ring
// depth (8 KiB per warp, 64 KiB per SM by default), not by how many registers a thread can hold.  No warp ever waits for
// another warp: there is no CTA-wide barrier after set-up.
#pragma once
#include "tc_sm100.cuh"

namespace hexb {
namespace ring {

constexpr int WARPS = 8;                    // consumer warps per CTA (each runs its own ring)
constexpr int THREADS = WARPS * 32;
constexpr int RING_BYTES_PER_WARP = 8 * 1024;   // measured best on B200: deeper rings lose DRAM locality
constexpr int MAX_SLOTS = 8;
constexpr int MAX_ROW_BYTES = 8192;

__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// One row shared -> global as a single bulk store (bulk async-group completion).
__device__ __forceinline__ void bulk_store(void *dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void bulk_load_hint(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar,
                                               uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}
// Output store of one 16-byte vector; `mode` picks the cache policy (measurement knob).
__device__ __forceinline__ void store_out16(void *p, uint4 v, int mode, uint64_t policy) {
  if (mode == 0) {
    st_stream16(p, v);
  } else if (mode == 1) {
    asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  } else if (mode == 2) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  } else {
    asm volatile("st.global.L2::cache_hint.v4.u32 [%0], {%1,%2,%3,%4}, %5;" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w), "l"(policy)
                 : "memory");
  }
}

__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

struct Layout {
  int slots;          // ring depth per warp
  int slot_bytes;     // row bytes rounded up to 128
  int smem_bytes;     // dynamic shared memory of the CTA
};

inline Layout make_layout(int row_bytes, int extra_bytes = 0, int out_slots = 0) {
  Layout l;
  l.slot_bytes = (row_bytes + 127) / 128 * 128;
  l.slots = option(OPT_ring_bytes_per_warp, RING_BYTES_PER_WARP) / l.slot_bytes;
  if (l.slots < 1) l.slots = 1;
  if (l.slots > MAX_SLOTS) l.slots = MAX_SLOTS;
  // [ring buffers][barriers][abort flag, pad to 128][extra][slack for the 128-byte alignment]
  // [ring buffers][output slots][barriers][abort flag, pad to 128][extra][slack for the 128-byte alignment]
  l.smem_bytes = WARPS * (l.slots + out_slots) * l.slot_bytes + WARPS * MAX_SLOTS * 8 + 128 + extra_bytes + 128;
  return l;
}

// Per-warp view of the ring.  Row r of the matrix is handled by warp (r % WARPS) of CTA
// ((r / WARPS) % gridDim.x): the WARPS rows a CTA works on at one time are adjacent in memory.
struct WarpRing {
  uint32_t buf0;       // shared address of this warp's slot 0
  uint32_t bar0;       // shared address of this warp's barrier 0
  int slots, slot_bytes;
  volatile int *abort_flag;
  uint32_t extra;      // shared address of the CTA-wide extra region (after barriers and flag)
  uint32_t out0;       // shared address of this warp's first output slot (rows leave through bulk stores)
  uint64_t policy;     // L2 evict-first policy descriptor
  int load_hint;       // 1: bulk loads carry the evict-first hint

  __device__ __forceinline__ uint32_t slot_addr(int s) const { return buf0 + (uint32_t)(s * slot_bytes); }
  __device__ __forceinline__ uint32_t bar(int s) const { return bar0 + 8u * (uint32_t)s; }
  // lane 0 only
  __device__ __forceinline__ void arm(int s, const void *src, uint32_t bytes) const {
    tc::mbar_arrive_expect_tx(bar(s), bytes);
    if (load_hint) bulk_load_hint(slot_addr(s), src, bytes, bar(s), policy);
    else bulk_load(slot_addr(s), src, bytes, bar(s));
  }
};

// Carves the CTA's dynamic shared memory, initialises the barriers and returns this warp's ring.
__device__ __forceinline__ WarpRing setup(uint8_t *smem_raw, int slots, int slot_bytes, int load_hint = 0,
                                          int out_slots = 0) {
  const uint32_t raw = tc::smem_u32(smem_raw);
  const uint32_t base = (raw + 127u) & ~127u;
  const int warp = threadIdx.x >> 5;
  const uint32_t outs = base + (uint32_t)(WARPS * slots * slot_bytes);
  const uint32_t bars = outs + (uint32_t)(WARPS * out_slots * slot_bytes);
  WarpRing r;
  r.slots = slots;
  r.slot_bytes = slot_bytes;
  r.buf0 = base + (uint32_t)(warp * slots * slot_bytes);
  r.out0 = outs + (uint32_t)(warp * out_slots * slot_bytes);
  r.bar0 = bars + (uint32_t)(warp * MAX_SLOTS * 8);
  r.abort_flag = reinterpret_cast<volatile int *>(smem_raw + (bars + WARPS * MAX_SLOTS * 8 - raw));
  r.extra = bars + WARPS * MAX_SLOTS * 8 + 128;
  r.policy = policy_evict_first();
  r.load_hint = load_hint;
  if (threadIdx.x == 0) {
    for (int i = 0; i < WARPS * MAX_SLOTS; ++i) tc::mbar_init(bars + 8u * i, 1);
    *r.abort_flag = 0;
    tc::fence_barrier_init();
  }
  __syncthreads();
  return r;
}

// Which rows a warp walks.  map == 0: row r belongs to warp (r % WARPS) of CTA ((r / WARPS) % grid)
// (the rows in flight across the GPU form one sliding window); map == 1: every CTA owns one
// contiguous block of rows and its warps interleave inside it (one sequential stream per CTA).
struct RowWalk {
  int64_t first, step, end;
};
__device__ __forceinline__ RowWalk row_walk(int64_t rows, int map) {
  const int warp = threadIdx.x >> 5;
  RowWalk w;
  if (map == 0) {
    w.first = (int64_t)blockIdx.x * WARPS + warp;
    w.step = (int64_t)gridDim.x * WARPS;
    w.end = rows;
  } else {
    int64_t per = (rows + gridDim.x - 1) / gridDim.x;
    per = (per + WARPS - 1) / WARPS * WARPS;
    const int64_t start = (int64_t)blockIdx.x * per;
    w.first = start + warp;
    w.step = WARPS;
    w.end = start + per < rows ? start + per : rows;
  }
  return w;
}

}  // namespace ring
}  // namespace hexb
