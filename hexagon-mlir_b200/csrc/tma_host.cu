// Host side of the TMA path: tensor-map encoding through the driver entry point, and the
// aggregated device status word.
#include <cstring>
#include <mutex>

#include "tc_sm100.cuh"

namespace hexb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      cudaGetLastError();
  });
  return fn;
}

int encode_tmap_f16_sw128_uncached(CUtensorMap *out, const void *base, int rank, const uint64_t *dims,
                                   const uint64_t *strides_bytes, const uint32_t *box);
int encode_tmap_f32_sw128_2d_uncached(CUtensorMap *out, const void *base, const uint64_t *dims, uint64_t row_stride_bytes,
                                      const uint32_t *box);

// ---- per-thread cache of encoded tensor maps.  A tensor map depends only on (base address, element type,
// extents, strides, box), and a model replays the same few dozen combinations launch after launch; the
// driver call that encodes one costs about a microsecond, more than the rest of a launch's host work.
// Direct-mapped, 256 entries per host thread (no lock, no sharing), keyed by an FNV-1a hash of the
// arguments and verified field by field on a hit.  Option "tmap_cache" = 0 bypasses it.
struct TmapKey {
  const void *base;
  uint32_t dtype, rank;
  uint64_t dims[5], strides[4];
  uint32_t box[5];
  uint32_t pad;
};
struct TmapEntry {
  TmapKey key;
  CUtensorMap map;
  bool valid;
};
static inline uint64_t fnv1a(const void *p, size_t n) {
  const unsigned char *b = static_cast<const unsigned char *>(p);
  uint64_t h = 1469598103934665603ull;
  for (size_t i = 0; i < n; ++i) h = (h ^ b[i]) * 1099511628211ull;
  return h;
}
static TmapEntry *tmap_cache_slot(const TmapKey &k, bool *hit) {
  static thread_local TmapEntry cache[256] = {};
  TmapEntry *e = &cache[fnv1a(&k, sizeof(k)) & 255u];
  *hit = e->valid && memcmp(&e->key, &k, sizeof(k)) == 0;
  return e;
}
static TmapKey make_key(const void *base, uint32_t dtype, int rank, const uint64_t *dims, const uint64_t *strides,
                        const uint32_t *box) {
  TmapKey k;
  memset(&k, 0, sizeof(k));
  k.base = base;
  k.dtype = dtype;
  k.rank = (uint32_t)rank;
  for (int i = 0; i < rank; ++i) { k.dims[i] = dims[i]; k.box[i] = box[i]; }
  for (int i = 0; i + 1 < rank; ++i) k.strides[i] = strides[i];
  return k;
}

int encode_tmap_f16_sw128(CUtensorMap *out, const void *base, int rank, const uint64_t *dims,
                          const uint64_t *strides_bytes, const uint32_t *box) {
  if (rank < 2 || rank > 5) return HEXB_ERR_BAD_ARG;
  TmapEntry *slot = nullptr;
  TmapKey key;
  if (option(OPT_tmap_cache, 1)) {
    key = make_key(base, 16, rank, dims, strides_bytes, box);
    bool hit = false;
    slot = tmap_cache_slot(key, &hit);
    if (hit) {
      *out = slot->map;
      return HEXB_OK;
    }
  }
  const int status = encode_tmap_f16_sw128_uncached(out, base, rank, dims, strides_bytes, box);
  if (status == HEXB_OK && slot) {
    slot->key = key;
    slot->map = *out;
    slot->valid = true;
  }
  return status;
}

static int encode_tmap_sw128_uncached(CUtensorMap *out, CUtensorMapDataType dtype, const void *base, int rank,
                                      const uint64_t *dims, const uint64_t *strides_bytes, const uint32_t *box);

int encode_tmap_f16_sw128_uncached(CUtensorMap *out, const void *base, int rank, const uint64_t *dims,
                                   const uint64_t *strides_bytes, const uint32_t *box) {
  return encode_tmap_sw128_uncached(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, base, rank, dims, strides_bytes, box);
}

// fp32 tensors of rank 2..5 (box inner extent 32 floats = 128 bytes), cached like the fp16 maps.
int encode_tmap_f32_sw128(CUtensorMap *out, const void *base, int rank, const uint64_t *dims,
                          const uint64_t *strides_bytes, const uint32_t *box) {
  if (rank < 2 || rank > 5) return HEXB_ERR_BAD_ARG;
  TmapEntry *slot = nullptr;
  TmapKey key;
  if (option(OPT_tmap_cache, 1)) {
    key = make_key(base, 33, rank, dims, strides_bytes, box);
    bool hit = false;
    slot = tmap_cache_slot(key, &hit);
    if (hit) {
      *out = slot->map;
      return HEXB_OK;
    }
  }
  const int status = encode_tmap_sw128_uncached(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, base, rank, dims, strides_bytes, box);
  if (status == HEXB_OK && slot) {
    slot->key = key;
    slot->map = *out;
    slot->valid = true;
  }
  return status;
}

static int encode_tmap_sw128_uncached(CUtensorMap *out, CUtensorMapDataType dtype, const void *base, int rank,
                                      const uint64_t *dims, const uint64_t *strides_bytes, const uint32_t *box) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_cuda_error(cudaErrorNotSupported, "cuTensorMapEncodeTiled entry point");
    return HEXB_ERR_CUDA;
  }
  if (rank < 2 || rank > 5) return HEXB_ERR_BAD_ARG;
  if (!aligned16(base)) return HEXB_ERR_MISALIGNED;
  cuuint64_t gd[5], gs[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    gd[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (dims[i] == 0) return HEXB_ERR_BAD_ARG;
  }
  for (int i = 0; i + 1 < rank; ++i) {
    gs[i] = strides_bytes[i];
    if (gs[i] % 16) return HEXB_ERR_MISALIGNED;
  }
  CUresult r = fn(out, dtype, (cuuint32_t)rank, const_cast<void *>(base), gd,
                  gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
    return HEXB_ERR_CUDA;
  }
  return HEXB_OK;
}

// Same for a 2-D fp32 tensor (dims and box in elements; the box's inner extent is 32 floats = 128 bytes).
int encode_tmap_f32_sw128_2d(CUtensorMap *out, const void *base, const uint64_t *dims, uint64_t row_stride_bytes,
                             const uint32_t *box) {
  TmapEntry *slot = nullptr;
  TmapKey key;
  if (option(OPT_tmap_cache, 1)) {
    key = make_key(base, 32, 2, dims, &row_stride_bytes, box);
    bool hit = false;
    slot = tmap_cache_slot(key, &hit);
    if (hit) {
      *out = slot->map;
      return HEXB_OK;
    }
  }
  const int status = encode_tmap_f32_sw128_2d_uncached(out, base, dims, row_stride_bytes, box);
  if (status == HEXB_OK && slot) {
    slot->key = key;
    slot->map = *out;
    slot->valid = true;
  }
  return status;
}

int encode_tmap_f32_sw128_2d_uncached(CUtensorMap *out, const void *base, const uint64_t *dims, uint64_t row_stride_bytes,
                                      const uint32_t *box) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_cuda_error(cudaErrorNotSupported, "cuTensorMapEncodeTiled entry point");
    return HEXB_ERR_CUDA;
  }
  if (!aligned16(base) || row_stride_bytes % 16) return HEXB_ERR_MISALIGNED;
  if (dims[0] == 0 || dims[1] == 0) return HEXB_ERR_BAD_ARG;
  cuuint64_t gd[2] = {dims[0], dims[1]}, gs[1] = {row_stride_bytes};
  cuuint32_t bx[2] = {box[0], box[1]}, es[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(base), gd, gs, bx, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
    return HEXB_ERR_CUDA;
  }
  return HEXB_OK;
}

// ------------------------------------------------------------------ bounded-wait self-test
// One CTA with the role layout of the tensor-core kernels (warp 0 producer, warp 1 owner of the TMEM
// allocation, warps 2-5 consumers).  It initialises one mbarrier that nothing ever arrives on; the
// producer waits on it with the given limit, gives up, raises the CTA's abort flag; the consumers,
// waiting on the same barrier with the default limit, see the flag at their next look and leave too;
// everyone meets at the common teardown, the TMEM columns are released and the status word is set.
static __device__ int g_selftest_status = 0;

__global__ void __launch_bounds__(192, 1) bounded_wait_selftest_kernel(unsigned long long limit_ns) {
  __shared__ __align__(8) unsigned long long bar_storage;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_word;
  volatile int *abort_flag = &abort_word;
  const uint32_t bar = tc::smem_u32(&bar_storage);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    tc::mbar_init(bar, 1);
    abort_word = 0;
    tc::fence_barrier_init();
  }
  if (warp == 1) {
    tc::tmem_alloc(tc::smem_u32(&tmem_slot), 32);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  bool ok = true;
  if (warp == 0) {
    if (lane == 0) ok = tc::mbar_wait(bar, 0, abort_flag, limit_ns);   // runs out: nobody arrives
  } else if (warp >= 2) {
    ok = tc::mbar_wait(bar, 0, abort_flag);                            // leaves through the abort flag
  }
  (void)ok;
  // common teardown, as in the tensor-core kernels
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, 32);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&g_selftest_status, (int)HEXB_ERR_TIMEOUT);
}

static int selftest_device_status_fetch_and_clear(int *out) {
  int v = 0, zero = 0;
  HEXB_CUDA_OK(cudaMemcpyFromSymbol(&v, g_selftest_status, sizeof(int)));
  if (v) HEXB_CUDA_OK(cudaMemcpyToSymbol(g_selftest_status, &zero, sizeof(int)));
  *out = v;
  return HEXB_OK;
}

int gemm_device_status_fetch_and_clear(int *out);
int attn_device_status_fetch_and_clear(int *out);
int norm_device_status_fetch_and_clear(int *out);
int softmax_device_status_fetch_and_clear(int *out);
int embed_device_status_fetch_and_clear(int *out);

}  // namespace hexb

extern "C" int hexb_device_status(int *out) {
  using namespace hexb;
  if (!out) return HEXB_ERR_BAD_ARG;
  HEXB_CUDA_OK(cudaDeviceSynchronize());
  int v[6] = {0, 0, 0, 0, 0, 0};
  if (int s = gemm_device_status_fetch_and_clear(&v[0])) return s;
  if (int s = attn_device_status_fetch_and_clear(&v[1])) return s;
  if (int s = norm_device_status_fetch_and_clear(&v[2])) return s;
  if (int s = softmax_device_status_fetch_and_clear(&v[3])) return s;
  if (int s = embed_device_status_fetch_and_clear(&v[4])) return s;
  if (int s = selftest_device_status_fetch_and_clear(&v[5])) return s;
  *out = v[0] ? v[0] : v[1] ? v[1] : v[2] ? v[2] : v[3] ? v[3] : v[4] ? v[4] : v[5];
  return HEXB_OK;
}

extern "C" int hexb_selftest_bounded_wait(int limit_us, void *stream) {
  using namespace hexb;
  if (limit_us < 1 || limit_us > 1000000) return HEXB_ERR_BAD_ARG;   // 1 us .. 1 s
  DeviceInfo di;
  if (int e = current_device(&di)) return e;
  bounded_wait_selftest_kernel<<<1, 192, 0, (cudaStream_t)stream>>>((unsigned long long)limit_us * 1000ull);
  return check_launch("bounded_wait_selftest");
}
