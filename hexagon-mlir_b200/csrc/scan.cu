// Cumulative sum along one axis of a tensor viewed as [outer, len, inner].
//
// Reference semantics (qualcomm/hexagon-mlir): ttx.cumsum ins(x) outs(y) {axis}
// (qcom_hexagon_backend/include/hexagon/Dialect/TTX/IR/TTXOps.td:61-75) lowers to a sequential loop
// `p = x[..., 0]; for i in 1..len: p = p + x[..., i]; y[..., i] = p` over slices of the scanned axis
// (lib/Transforms/LowerTTX.cpp:179-300; lit tests test/Conversion/TtxToLinalg/cumsum_{1D_static,
// 1D_dynamic,2D}.mlir), and ttx.scan {axis, reverse} with an addition body is the same walk from the
// far end (LowerTTX.cpp:75-176, reverse_associative_scan_1D.mlir).  Integer results are exact; floating
// sums are accumulated in fp32 in a different association than the sequential loop.
//
// B200 form.  inner == 1 (the scanned axis is contiguous): a CTA owns a segment of a row and walks it
// in chunks; inside a chunk every warp owns a contiguous span, loads it as 16-byte vectors (lane-
// interleaved, so each load instruction covers 512 contiguous bytes), scans each vector in registers,
// scans the vector totals across the lanes with shuffles, and carries the running total from vector
// row to vector row -- no CTA barrier inside a span.  One barrier per chunk publishes the warp totals.
// A row longer than a CTA can stream well is cut into segments: a first launch reduces every segment,
// a one-warp-per-row launch turns the segment totals into offsets, and the scan launch starts each
// segment from its offset (reads the row twice: 1.5x the algorithmic traffic, only for rows that
// need it).  inner > 1: one thread per (outer, inner) column walks the axis with coalesced accesses.
#include "common.cuh"

namespace hexb {
namespace scan {

constexpr int THREADS = 256;
constexpr int WARPS = THREADS / 32;

template <typename T> struct AccOf { using type = float; };
template <> struct AccOf<int32_t> { using type = int32_t; };

template <typename T, typename A> __device__ __forceinline__ A load_acc(T v);
template <> __device__ __forceinline__ float load_acc<float, float>(float v) { return v; }
template <> __device__ __forceinline__ float load_acc<__half, float>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ int32_t load_acc<int32_t, int32_t>(int32_t v) { return v; }
template <typename T, typename A> __device__ __forceinline__ T store_acc(A v);
template <> __device__ __forceinline__ float store_acc<float, float>(float v) { return v; }
template <> __device__ __forceinline__ __half store_acc<__half, float>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ int32_t store_acc<int32_t, int32_t>(int32_t v) { return v; }

template <typename A>
__device__ __forceinline__ A warp_inclusive(A v, int lane) {
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const A o = __shfl_up_sync(0xffffffffu, v, d);
    if (lane >= d) v += o;
  }
  return v;
}

// One CTA per (row, segment).  MODE 0: scan and write, starting from offsets[row * segs + seg] (or 0);
// MODE 1: write only the segment's total to totals[row * segs + seg].
// VEC: 16-byte vector accesses (forward direction, aligned rows); otherwise element accesses, which
// also serve the reverse direction (logical position p is element len - 1 - p).
// KV: vectors per lane per chunk (the chunk is sized to the row so that short rows keep every warp busy).
template <typename T, int MODE, bool VEC, int KV>
__global__ void __launch_bounds__(THREADS)
cumsum_rows_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t len, int64_t seg_len, int segs, int reverse,
                   const typename AccOf<T>::type *__restrict__ offsets, typename AccOf<T>::type *__restrict__ totals) {
  using A = typename AccOf<T>::type;
  constexpr int E = VEC ? 16 / (int)sizeof(T) : 1;
  constexpr int SPAN = 32 * KV * E;       // elements one warp covers per chunk
  constexpr int CHUNK = WARPS * SPAN;
  __shared__ A warp_tot[2][WARPS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = blockIdx.x / segs;
  const int seg = (int)(blockIdx.x - row * segs);
  const int64_t p0 = (int64_t)seg * seg_len;
  const int64_t p1 = p0 + seg_len < len ? p0 + seg_len : len;
  const T *xr = x + row * len;
  T *yr = y + row * len;
  A carry = (MODE == 0 && offsets) ? offsets[blockIdx.x] : A(0);
  int par = 0;
  for (int64_t c0 = p0; c0 < p1; c0 += CHUNK, par ^= 1) {
    const int64_t w0 = c0 + (int64_t)warp * SPAN;
    A v[KV][E];
    A run = A(0);  // total of the vector rows of this span handled so far
#pragma unroll
    for (int k = 0; k < KV; ++k) {
      const int64_t p = w0 + ((int64_t)k * 32 + lane) * E;
      if constexpr (VEC) {
        if (p + E <= p1) {
          const uint4 raw = ld_stream16(xr + p);
          const T *t = reinterpret_cast<const T *>(&raw);
#pragma unroll
          for (int e = 0; e < E; ++e) v[k][e] = load_acc<T, A>(t[e]);
        } else {
#pragma unroll
          for (int e = 0; e < E; ++e) v[k][e] = (p + e < p1) ? load_acc<T, A>(xr[p + e]) : A(0);
        }
      } else {
        v[k][0] = (p < p1) ? load_acc<T, A>(xr[reverse ? len - 1 - p : p]) : A(0);
      }
#pragma unroll
      for (int e = 1; e < E; ++e) v[k][e] += v[k][e - 1];
      const A incl = warp_inclusive(v[k][E - 1], lane);
      const A excl = incl - v[k][E - 1] + run;
#pragma unroll
      for (int e = 0; e < E; ++e) v[k][e] += excl;
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) warp_tot[par][warp] = run;
    __syncthreads();  // one barrier per chunk: the other parity's slots are rewritten only after the next one
    A before = carry, all = A(0);
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const A t = warp_tot[par][w];
      if (w < warp) before += t;
      all += t;
    }
    carry += all;
    if constexpr (MODE == 0) {
#pragma unroll
      for (int k = 0; k < KV; ++k) {
        const int64_t p = w0 + ((int64_t)k * 32 + lane) * E;
        if constexpr (VEC) {
          if (p + E <= p1) {
            uint4 raw;
            T *t = reinterpret_cast<T *>(&raw);
#pragma unroll
            for (int e = 0; e < E; ++e) t[e] = store_acc<T, A>(v[k][e] + before);
            st_stream16(yr + p, raw);
          } else {
#pragma unroll
            for (int e = 0; e < E; ++e)
              if (p + e < p1) yr[p + e] = store_acc<T, A>(v[k][e] + before);
          }
        } else {
          if (p < p1) yr[reverse ? len - 1 - p : p] = store_acc<T, A>(v[k][0] + before);
        }
      }
    }
  }
  if (MODE == 1 && threadIdx.x == 0) totals[blockIdx.x] = carry;
}

// Segment totals -> exclusive offsets, one warp per row (segs is small: a few hundred at most).
template <typename A>
__global__ void __launch_bounds__(32) segment_offsets_kernel(const A *__restrict__ totals, A *__restrict__ offsets,
                                                             int segs) {
  const int lane = threadIdx.x;
  const int64_t base = (int64_t)blockIdx.x * segs;
  A carry = A(0);
  for (int s0 = 0; s0 < segs; s0 += 32) {
    const int s = s0 + lane;
    const A t = s < segs ? totals[base + s] : A(0);
    const A incl = warp_inclusive(t, lane);
    if (s < segs) offsets[base + s] = carry + incl - t;
    carry += __shfl_sync(0xffffffffu, incl, 31);
  }
}

// inner > 1: one thread per (outer, inner) column and segment of the axis (blockIdx.y), coalesced over
// inner; eight loads are issued before the dependent additions.  MODE as above; totals and offsets are
// laid out [segment][column].
// VEC: adjacent columns one thread carries (1, or a 16-byte vector of them when inner allows it).
template <typename T, int MODE, int VEC>
__global__ void __launch_bounds__(THREADS)
cumsum_strided_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t outer, int64_t len, int64_t inner,
                      int reverse, int64_t seg_len, const typename AccOf<T>::type *__restrict__ offsets,
                      typename AccOf<T>::type *__restrict__ totals) {
  using A = typename AccOf<T>::type;
  constexpr int U = VEC == 1 ? 8 : (sizeof(T) == 2 ? 4 : 8);
  const int64_t cols = outer * inner;
  const int64_t groups_per_row = inner / VEC;
  const int64_t grp = (int64_t)blockIdx.x * THREADS + threadIdx.x;
  if (grp >= outer * groups_per_row) return;
  const int64_t o = grp / groups_per_row, i = (grp - o * groups_per_row) * VEC;
  const int64_t col = o * inner + i;
  const T *xp = x + o * len * inner + i;
  T *yp = y + o * len * inner + i;
  const int64_t p0 = (int64_t)blockIdx.y * seg_len;
  const int64_t p1 = p0 + seg_len < len ? p0 + seg_len : len;
  A acc[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) acc[e] = (MODE == 0 && offsets) ? offsets[(int64_t)blockIdx.y * cols + col + e] : A(0);
  for (int64_t q0 = p0; q0 < p1; q0 += U) {
    A v[U][VEC];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t p = q0 + u;
      const int64_t l = reverse ? len - 1 - p : p;
      if constexpr (VEC == 1) {
        v[u][0] = p < p1 ? load_acc<T, A>(xp[l * inner]) : A(0);
      } else {
        if (p < p1) {
          const uint4 raw = ld_stream16(xp + l * inner);
          const T *t = reinterpret_cast<const T *>(&raw);
#pragma unroll
          for (int e = 0; e < VEC; ++e) v[u][e] = load_acc<T, A>(t[e]);
        } else {
#pragma unroll
          for (int e = 0; e < VEC; ++e) v[u][e] = A(0);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t p = q0 + u;
      const int64_t l = reverse ? len - 1 - p : p;
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] += v[u][e];
      if (MODE == 0 && p < p1) {
        if constexpr (VEC == 1) {
          yp[l * inner] = store_acc<T, A>(acc[0]);
        } else {
          uint4 raw;
          T *t = reinterpret_cast<T *>(&raw);
#pragma unroll
          for (int e = 0; e < VEC; ++e) t[e] = store_acc<T, A>(acc[e]);
          st_stream16(yp + l * inner, raw);
        }
      }
    }
  }
  if (MODE == 1) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) totals[(int64_t)blockIdx.y * cols + col + e] = acc[e];
  }
}

template <typename A>
__global__ void __launch_bounds__(THREADS)
strided_offsets_kernel(const A *__restrict__ totals, A *__restrict__ offsets, int64_t cols, int segs) {
  const int64_t col = (int64_t)blockIdx.x * THREADS + threadIdx.x;
  if (col >= cols) return;
  A carry = A(0);
  for (int s = 0; s < segs; ++s) {
    const A t = totals[(int64_t)s * cols + col];
    offsets[(int64_t)s * cols + col] = carry;
    carry += t;
  }
}

template <typename T, bool VEC, int KV>
static int launch_rows(const T *x, T *y, int64_t outer, int64_t len, int reverse, int sm_count, cudaStream_t st) {
  using A = typename AccOf<T>::type;
  constexpr int E = VEC ? 16 / (int)sizeof(T) : 1;
  const int64_t chunk = (int64_t)WARPS * 32 * KV * E;
  // cut rows into segments until the grid has about four CTAs per SM, segments of at least 8 chunks
  int64_t segs = 1;
  const int64_t want = 4ll * sm_count;
  if (outer < want) {
    segs = (want + outer - 1) / outer;
    const int64_t max_segs = (len + 8 * chunk - 1) / (8 * chunk);
    if (segs > max_segs) segs = max_segs;
    if (segs < 1) segs = 1;
  }
  if (int64_t forced = option(OPT_scan_segments, 0)) segs = forced;
  int64_t seg_len = (len + segs - 1) / segs;
  seg_len = (seg_len + chunk - 1) / chunk * chunk;  // whole chunks: vector accesses stay aligned
  segs = (len + seg_len - 1) / seg_len;
  const int64_t ctas = outer * segs;
  if (ctas > 0x7fffffffll || segs > 0x7fffffffll) return HEXB_ERR_UNSUPPORTED;
  A *scratch = nullptr;
  if (segs > 1) {
    // stream-ordered scratch for the segment totals and offsets (a few KiB)
    if (int e = scratch_alloc(reinterpret_cast<void **>(&scratch), (size_t)ctas * 2 * sizeof(A), st)) return e;
    cumsum_rows_kernel<T, 1, VEC, KV><<<(unsigned)ctas, THREADS, 0, st>>>(x, y, len, seg_len, (int)segs, reverse,
                                                                          nullptr, scratch);
    segment_offsets_kernel<A><<<(unsigned)outer, 32, 0, st>>>(scratch, scratch + ctas, (int)segs);
  }
  cumsum_rows_kernel<T, 0, VEC, KV><<<(unsigned)ctas, THREADS, 0, st>>>(x, y, len, seg_len, (int)segs, reverse,
                                                                        segs > 1 ? scratch + ctas : nullptr, nullptr);
  const int rc = check_launch("cumsum_rows");
  if (int e = scratch_free(scratch, st)) return e;
  return rc;
}

template <typename T>
static int run(const T *x, T *y, int64_t outer, int64_t len, int64_t inner, int reverse, cudaStream_t st) {
  using A = typename AccOf<T>::type;
  DeviceInfo di;
  if (int e = current_device(&di)) return e;
  if (inner > 1) {
    const int64_t cols = outer * inner;
    constexpr int EV = 16 / (int)sizeof(T);
    const bool vecs = inner % EV == 0 && aligned16(x) && aligned16(y) && !option(OPT_scan_force_scalar, 0);
    const int64_t groups = vecs ? cols / EV : cols;            // threads along the columns
    const int64_t grp_ctas = (groups + THREADS - 1) / THREADS;
    const int64_t col_ctas = (cols + THREADS - 1) / THREADS;
    if (col_ctas > 0x7fffffffll) return HEXB_ERR_UNSUPPORTED;
    // enough threads to keep the memory system busy: about 2048 per SM, segments of at least 64 steps
    int64_t segs = (2048ll * di.sm_count + groups - 1) / groups;
    if (segs > (len + 63) / 64) segs = (len + 63) / 64;
    // the offsets pass walks the segments serially per column and the scratch is [segments][columns]:
    // keep both small (at most 64 segments, at most 16 MiB of totals + offsets)
    if (segs > 64) segs = 64;
    const int64_t by_scratch = ((int64_t)16 << 20) / (cols * 2 * (int64_t)sizeof(A));
    if (segs > by_scratch) segs = by_scratch;
    if (segs < 1) segs = 1;
    if (int64_t forced = option(OPT_scan_segments, 0)) segs = forced < 65535 ? forced : 65535;
    const int64_t seg_len = (len + segs - 1) / segs;
    segs = (len + seg_len - 1) / seg_len;
    const dim3 grid((unsigned)grp_ctas, (unsigned)segs);
    A *scratch = nullptr;
    if (segs > 1) {
      if (int e = scratch_alloc(reinterpret_cast<void **>(&scratch), (size_t)(cols * segs) * 2 * sizeof(A), st)) return e;
      if (vecs) cumsum_strided_kernel<T, 1, EV><<<grid, THREADS, 0, st>>>(x, y, outer, len, inner, reverse, seg_len, nullptr, scratch);
      else cumsum_strided_kernel<T, 1, 1><<<grid, THREADS, 0, st>>>(x, y, outer, len, inner, reverse, seg_len, nullptr, scratch);
      strided_offsets_kernel<A><<<(unsigned)col_ctas, THREADS, 0, st>>>(scratch, scratch + cols * segs, cols, (int)segs);
    }
    const A *offs = segs > 1 ? scratch + cols * segs : nullptr;
    if (vecs) cumsum_strided_kernel<T, 0, EV><<<grid, THREADS, 0, st>>>(x, y, outer, len, inner, reverse, seg_len, offs, nullptr);
    else cumsum_strided_kernel<T, 0, 1><<<grid, THREADS, 0, st>>>(x, y, outer, len, inner, reverse, seg_len, offs, nullptr);
    const int rc = check_launch("cumsum_strided");
    if (int e = scratch_free(scratch, st)) return e;
    return rc;
  }
  constexpr int E = 16 / (int)sizeof(T);
  const bool vec = !reverse && aligned16(x) && aligned16(y) && (outer == 1 || len % E == 0) &&
                   !option(OPT_scan_force_scalar, 0);
  const int64_t per_kv = (int64_t)WARPS * 32 * (vec ? E : 1);   // elements of a chunk per unit of KV
  const int64_t kv_cap = option(OPT_scan_kv, 2);
  if (vec) {
    if (len >= 4 * per_kv && kv_cap >= 4) return launch_rows<T, true, 4>(x, y, outer, len, reverse, di.sm_count, st);
    if (len >= 2 * per_kv && kv_cap >= 2) return launch_rows<T, true, 2>(x, y, outer, len, reverse, di.sm_count, st);
    return launch_rows<T, true, 1>(x, y, outer, len, reverse, di.sm_count, st);
  }
  if (len >= 4 * per_kv) return launch_rows<T, false, 4>(x, y, outer, len, reverse, di.sm_count, st);
  return launch_rows<T, false, 1>(x, y, outer, len, reverse, di.sm_count, st);
}

}  // namespace scan
}  // namespace hexb

extern "C" int hexb_cumsum(int dtype, const void *x, void *y, int64_t outer, int64_t len, int64_t inner, int reverse,
                           void *stream) {
  using namespace hexb;
  if (outer < 0 || len < 0 || inner < 0) return HEXB_ERR_BAD_ARG;
  if (outer == 0 || len == 0 || inner == 0) return HEXB_OK;
  if (!x || !y) return HEXB_ERR_BAD_ARG;
  if (outer >= (1ll << 31)) return HEXB_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case HEXB_DT_F32: return scan::run<float>((const float *)x, (float *)y, outer, len, inner, reverse ? 1 : 0, st);
    case HEXB_DT_F16: return scan::run<__half>((const __half *)x, (__half *)y, outer, len, inner, reverse ? 1 : 0, st);
    case HEXB_DT_I32: return scan::run<int32_t>((const int32_t *)x, (int32_t *)y, outer, len, inner, reverse ? 1 : 0, st);
    default: return HEXB_ERR_UNSUPPORTED;
  }
}
