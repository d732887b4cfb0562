// Host-side runtime of libhexb200: status strings, error text, option store, device cache, and the
// `_host` launcher entry points that stage tensors across the host/device boundary.
//
// The `_host` entry points take the place of the wrapper main() the reference generates per kernel
// (qcom_hexagon_backend/backend/triton_hexagon_launcher.py:111-123): that program loads the input
// tensors from files pushed over adb, runs the kernel and dumps the outputs for the host to pull
// back; here the crossing is a pair of PCIe copies around an in-process launch.
#include <cstdio>
#include <cstring>
#include <atomic>
#include <mutex>

#include "common.cuh"

namespace hexb {

static thread_local char g_err_text[256] = "";

void set_cuda_error(cudaError_t e, const char *where) {
  snprintf(g_err_text, sizeof(g_err_text), "%s: %s (%s)", where, cudaGetErrorName(e),
           cudaGetErrorString(e));
}

int check_launch(const char *where) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_cuda_error(e, where);
    return HEXB_ERR_CUDA;
  }
  return HEXB_OK;
}

static std::mutex g_mu;

// ---- option store: one atomic word per option (bit 32 = "has been set", low 32 bits = value)
static std::atomic<int64_t> g_opt[OPT_COUNT];
static const char *const kOptName[OPT_COUNT] = {
#define HEXB_X(n) #n,
    HEXB_OPTIONS(HEXB_X) HEXB_DEV_OPTIONS(HEXB_X)
#undef HEXB_X
};
#define HEXB_X(n) +1
static constexpr int kShippedOptions = 0 HEXB_OPTIONS(HEXB_X);  // the dev-only names follow these
#undef HEXB_X

int option(Opt key, int dflt) {
  const int64_t v = g_opt[key].load(std::memory_order_relaxed);
  return (v >> 32) & 1 ? (int)(uint32_t)v : dflt;
}

static int find_option(const char *key) {
#ifdef HEXB_DEV
  const int n = OPT_COUNT;
#else
  const int n = kShippedOptions;
#endif
  for (int i = 0; i < n; ++i)
    if (!strcmp(kOptName[i], key)) return i;
  return -1;
}

int current_device(DeviceInfo *out) {
  static DeviceInfo cache[64];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return HEXB_ERR_NO_DEVICE;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceInfo &d = cache[dev];
  if (d.device != dev) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
      cudaGetLastError();
      return HEXB_ERR_NO_DEVICE;
    }
    d.sm_count = v;
    cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    d.smem_optin = (size_t)v;
    cudaDeviceGetAttribute(&v, cudaDevAttrL2CacheSize, dev);
    d.l2_bytes = (size_t)v;
    d.device = dev;
  }
  *out = d;
  if (d.cc_major != 10) return HEXB_ERR_NO_DEVICE;  // the binary holds sm_100a code only
  return HEXB_OK;
}

// ---- library-owned memory pool for stream-ordered scratch
int scratch_alloc(void **ptr, size_t bytes, cudaStream_t st) {
  static cudaMemPool_t pools[64] = {};
  int dev = 0;
  HEXB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return HEXB_ERR_NO_DEVICE;
  cudaMemPool_t mine = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!pools[dev]) {
      cudaMemPoolProps props = {};
      props.allocType = cudaMemAllocationTypePinned;
      props.handleTypes = cudaMemHandleTypeNone;
      props.location.type = cudaMemLocationTypeDevice;
      props.location.id = dev;
      cudaMemPool_t pool = nullptr;
      HEXB_CUDA_OK(cudaMemPoolCreate(&pool, &props));
      unsigned long long keep = ~0ull;  // freed blocks stay in the pool
      HEXB_CUDA_OK(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
      pools[dev] = pool;
    }
    mine = pools[dev];
  }
  HEXB_CUDA_OK(cudaMallocFromPoolAsync(ptr, bytes, mine, st));
  return HEXB_OK;
}

int scratch_free(void *ptr, cudaStream_t st) {
  if (ptr) HEXB_CUDA_OK(cudaFreeAsync(ptr, st));
  return HEXB_OK;
}

// ---- per-device staging memory for the `_host` entry points (grow-only, released on request).
struct Staging {
  void *ptr = nullptr;
  size_t bytes = 0;
  static constexpr int kMaxChunks = 64;
  cudaStream_t streams[3] = {nullptr, nullptr, nullptr};  // upload, compute, download
  cudaEvent_t ev_in[kMaxChunks] = {}, ev_k[kMaxChunks] = {};
  bool ready = false;
};
static Staging g_staging[64];
static std::mutex g_staging_mu;

static int staging_get(size_t bytes, Staging **out) {
  int dev = -1;
  HEXB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return HEXB_ERR_NO_DEVICE;
  Staging &s = g_staging[dev];
  if (!s.ready) {
    for (auto &st : s.streams) HEXB_CUDA_OK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    for (auto &ev : s.ev_in) HEXB_CUDA_OK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    for (auto &ev : s.ev_k) HEXB_CUDA_OK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    s.ready = true;
  }
  if (s.bytes < bytes) {
    if (s.ptr) HEXB_CUDA_OK(cudaFree(s.ptr));
    s.ptr = nullptr;
    s.bytes = 0;
    HEXB_CUDA_OK(cudaMalloc(&s.ptr, bytes));
    s.bytes = bytes;
  }
  *out = &s;
  return HEXB_OK;
}

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
static inline size_t dt_size(int dt) { return dt == HEXB_DT_F16 ? 2 : dt == HEXB_DT_F32 ? 4 : 0; }

// Row-wise operators: the rows are cut into chunks that flow through three streams -- upload,
// compute, download -- chained by events, so that the upload of chunk i+1, the kernel of chunk i
// and the download of chunk i-1 overlap (PCIe is full duplex and each direction has its own copy
// engine).  `launch(x_dev, y_dev, extra_dev, row0, nrows, stream)`; a call with x_dev == nullptr
// uploads the operator's small operands (gains, biases), one with nrows == -1 downloads its small
// results (statistics) after the last chunk.  The overlap needs page-locked host buffers
// (cudaHostAlloc / cudaHostRegister, torch's pin_memory()): with pageable memory the runtime stages
// every copy through its own bounce buffer and the device-to-host copies block the calling thread,
// so the chunks run one after the other (the results are the same).
// Waits for everything queued on the staging streams.  Every `_host` entry point calls this before it
// returns an error: copies against the caller's host buffers must not still be in flight when the
// caller gets control back (it may free them), nor when the next call reuses the staging block.
static void staging_drain(Staging *s) {
  if (!s) return;
  for (auto &st : s->streams)
    if (st) cudaStreamSynchronize(st);
  cudaGetLastError();
}

// Cuts `units` into at most `chunks` consecutive pieces whose sizes are multiples of `granule`; writes
// the piece boundaries to bounds[0..n] and returns n.  Equal pieces by default: with the download of a
// piece starting when its upload and kernel are done, the whole call takes (all uploads) + (the
// downloads from the largest piece on), so the largest piece should be as small as the per-copy
// overhead allows.  Tapered pieces (weights 1, 2, 4, 8, ..., 8, 4, 2, 1) measured 3 % faster for the
// matmul, whose first upload carries all of B, and 5 % slower for the row operators; host_taper = 0 / 1
// forces one or the other (negative: back to the per-operator default).
static int chunk_plan(int64_t units, int chunks, int64_t granule, int64_t *bounds, int taper_default = 0) {
  if (chunks < 1) chunks = 1;
  if (chunks > Staging::kMaxChunks) chunks = Staging::kMaxChunks;
  if (granule < 1) granule = 1;
  const int tv = option(OPT_host_taper, -1);   // negative: the caller's default
  const bool taper = chunks >= 4 && (tv < 0 ? taper_default : tv) != 0;
  int64_t w[Staging::kMaxChunks], total = 0;
  for (int i = 0; i < chunks; ++i) {
    const int edge = i < chunks - 1 - i ? i : chunks - 1 - i;
    w[i] = taper ? (edge >= 3 ? 8 : (int64_t)1 << edge) : 1;
    total += w[i];
  }
  int n = 0;
  int64_t acc = 0, at = 0;
  bounds[0] = 0;
  for (int i = 0; i < chunks && at < units; ++i) {
    acc += w[i];
    int64_t end = i == chunks - 1 ? units : (units * acc / total + granule - 1) / granule * granule;
    if (end > units) end = units;
    if (end <= at) continue;
    bounds[++n] = end;
    at = end;
  }
  if (at < units) bounds[n > 0 ? n : ++n] = units;
  return n;
}

// The three-stage pipeline every `_host` entry point runs: for each piece c, up(c, stream) queues its
// uploads, run(c, stream) its kernels, down(c, stream) its downloads; events chain the stages, so the
// upload of piece c+1, the kernels of piece c and the download of piece c-1 overlap.  One stream per
// direction: two uploads (or two downloads) in flight at once share the link and measured 10-20 %
// slower.  Returns with everything queued; the caller synchronises *last_out (the download stream) or
// drains on error.
template <typename Up, typename Run, typename Down>
static int staged_pipeline(Staging *s, int pieces, Up &&up, Run &&run, Down &&down, cudaStream_t *last_out) {
  cudaStream_t s_in = s->streams[0], s_k = s->streams[1], s_out = s->streams[2];
  *last_out = s_out;
  for (int c = 0; c < pieces; ++c) {
    if (int e = up(c, s_in)) return e;
    HEXB_CUDA_OK(cudaEventRecord(s->ev_in[c], s_in));
    HEXB_CUDA_OK(cudaStreamWaitEvent(s_k, s->ev_in[c], 0));
    if (int e = run(c, s_k)) return e;
    HEXB_CUDA_OK(cudaEventRecord(s->ev_k[c], s_k));
    HEXB_CUDA_OK(cudaStreamWaitEvent(s_out, s->ev_k[c], 0));
    if (int e = down(c, s_out)) return e;
  }
  return HEXB_OK;
}

template <typename F>
static int rows_pipeline(const void *x, void *y, int64_t rows, int64_t cols, size_t esz,
                         size_t extra_bytes, F &&launch_with_extra) {
  if (rows < 0 || cols < 0) return HEXB_ERR_BAD_ARG;
  if (rows == 0 || cols == 0) return HEXB_OK;
  if (!x || !y) return HEXB_ERR_BAD_ARG;
  const size_t row_bytes = (size_t)cols * esz;
  const size_t mat = align_up((size_t)rows * row_bytes, 256);
  const size_t extra = align_up(extra_bytes, 256);
  Staging *s = nullptr;
  if (int st = staging_get(2 * mat + extra, &s)) return st;
  char *dx = (char *)s->ptr, *dy = dx + mat, *de = dy + mat;
  int chunks = option(OPT_host_chunks, 8);
  if ((int64_t)chunks > rows) chunks = (int)rows;
  if ((size_t)rows * row_bytes < ((size_t)4 << 20)) chunks = 1;
  int64_t bounds[Staging::kMaxChunks + 1];
  chunks = chunk_plan(rows, chunks, 1, bounds);
  auto body = [&]() -> int {
    if (int st = launch_with_extra(nullptr, nullptr, de, 0, 0, s->streams[0])) return st;  // small operands
    auto span = [&](int c, size_t *off, int64_t *nr) {
      *off = (size_t)bounds[c] * row_bytes;
      *nr = bounds[c + 1] - bounds[c];
    };
    cudaStream_t last = nullptr;
    const int e = staged_pipeline(
        s, chunks,
        [&](int c, cudaStream_t st) -> int {
          size_t off; int64_t nr; span(c, &off, &nr);
          HEXB_CUDA_OK(cudaMemcpyAsync(dx + off, (const char *)x + off, (size_t)nr * row_bytes, cudaMemcpyHostToDevice, st));
          return HEXB_OK;
        },
        [&](int c, cudaStream_t st) -> int {
          size_t off; int64_t nr; span(c, &off, &nr);
          return launch_with_extra(dx + off, dy + off, de, bounds[c], nr, st);
        },
        [&](int c, cudaStream_t st) -> int {
          size_t off; int64_t nr; span(c, &off, &nr);
          HEXB_CUDA_OK(cudaMemcpyAsync((char *)y + off, dy + off, (size_t)nr * row_bytes, cudaMemcpyDeviceToHost, st));
          return HEXB_OK;
        },
        &last);
    if (e) return e;
    if (int st = launch_with_extra(dx, dy, de, 0, -1, last)) return st;  // small results
    HEXB_CUDA_OK(cudaStreamSynchronize(last));
    return HEXB_OK;
  };
  const int status = body();
  if (status != HEXB_OK) staging_drain(s);
  return status;
}

}  // namespace hexb

using namespace hexb;

extern "C" int hexb_version(void) { return 100; }

extern "C" const char *hexb_status_string(int s) {
  switch (s) {
    case HEXB_OK: return "HEXB_OK";
    case HEXB_ERR_BAD_ARG: return "HEXB_ERR_BAD_ARG";
    case HEXB_ERR_UNSUPPORTED: return "HEXB_ERR_UNSUPPORTED";
    case HEXB_ERR_MISALIGNED: return "HEXB_ERR_MISALIGNED";
    case HEXB_ERR_CUDA: return "HEXB_ERR_CUDA";
    case HEXB_ERR_TIMEOUT: return "HEXB_ERR_TIMEOUT";
    case HEXB_ERR_WORKSPACE: return "HEXB_ERR_WORKSPACE";
    case HEXB_ERR_NO_DEVICE: return "HEXB_ERR_NO_DEVICE";
    default: return "HEXB_ERR_UNKNOWN";
  }
}

extern "C" const char *hexb_last_cuda_error(void) { return g_err_text; }

extern "C" int hexb_set_option(const char *key, int value) {
  if (!key) return HEXB_ERR_BAD_ARG;
  const int i = find_option(key);
  if (i < 0) return HEXB_ERR_BAD_ARG;
  g_opt[i].store(((int64_t)1 << 32) | (uint32_t)value, std::memory_order_relaxed);
  return HEXB_OK;
}

extern "C" int hexb_get_option(const char *key, int *value) {
  if (!key || !value) return HEXB_ERR_BAD_ARG;
  const int i = find_option(key);
  if (i < 0) return HEXB_ERR_BAD_ARG;
  const int64_t v = g_opt[i].load(std::memory_order_relaxed);
  if (!((v >> 32) & 1)) return HEXB_ERR_BAD_ARG;  // never set: the launchers use their own defaults
  *value = (int)(uint32_t)v;
  return HEXB_OK;
}

extern "C" int hexb_host_staging_release(void) {
  int dev = -1;
  HEXB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return HEXB_ERR_NO_DEVICE;
  std::lock_guard<std::mutex> lk(g_staging_mu);
  Staging &s = g_staging[dev];
  if (s.ptr) HEXB_CUDA_OK(cudaFree(s.ptr));
  s.ptr = nullptr;
  s.bytes = 0;
  return HEXB_OK;
}

extern "C" int hexb_softmax_host(int dtype, const void *x, void *y, int64_t rows, int64_t cols) {
  const size_t esz = dt_size(dtype);
  if (!esz) return HEXB_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lk(g_staging_mu);
  return rows_pipeline(x, y, rows, cols, esz, 0,
                       [&](void *dx, void *dy, void *, int64_t, int64_t nr, cudaStream_t st) -> int {
                         if (!dx || nr < 0) return HEXB_OK;
                         return dtype == HEXB_DT_F16
                                    ? hexb_softmax_f16(dx, dy, nr, cols, cols, cols, st)
                                    : hexb_softmax_f32((const float *)dx, (float *)dy, nr, cols, cols, cols, st);
                       });
}

extern "C" int hexb_layer_norm_host(int dtype, const void *x, void *y, const void *w, const void *b,
                                    float *mean, float *rstd, int64_t rows, int64_t cols, float eps) {
  const size_t esz = dt_size(dtype);
  if (!esz) return HEXB_ERR_UNSUPPORTED;
  if (rows > 0 && cols > 0 && (!w || !b)) return HEXB_ERR_BAD_ARG;
  std::lock_guard<std::mutex> lk(g_staging_mu);
  const size_t vb = align_up((size_t)cols * esz, 256);
  const size_t sb = align_up((size_t)rows * 4, 256);
  int st = rows_pipeline(
      x, y, rows, cols, esz, 2 * vb + 2 * sb,
      [&](void *dx, void *dy, void *de, int64_t r0, int64_t nr, cudaStream_t s) -> int {
        char *dw = (char *)de, *db = dw + vb;
        float *dm = (float *)(db + vb), *dr = (float *)((char *)dm + sb);
        if (!dx) {
          HEXB_CUDA_OK(cudaMemcpyAsync(dw, w, (size_t)cols * esz, cudaMemcpyHostToDevice, s));
          HEXB_CUDA_OK(cudaMemcpyAsync(db, b, (size_t)cols * esz, cudaMemcpyHostToDevice, s));
          return HEXB_OK;
        }
        if (nr < 0) {  // statistics of all rows, after the last chunk
          if (mean) HEXB_CUDA_OK(cudaMemcpyAsync(mean, dm, (size_t)rows * 4, cudaMemcpyDeviceToHost, s));
          if (rstd) HEXB_CUDA_OK(cudaMemcpyAsync(rstd, dr, (size_t)rows * 4, cudaMemcpyDeviceToHost, s));
          return HEXB_OK;
        }
        return dtype == HEXB_DT_F16
                   ? hexb_layer_norm_f16(dx, dy, dw, db, dm + r0, dr + r0, nr, cols, cols, cols, eps, s)
                   : hexb_layer_norm_f32((const float *)dx, (float *)dy, (const float *)dw,
                                         (const float *)db, dm + r0, dr + r0, nr, cols, cols, cols, eps, s);
      });
  return st;
}

extern "C" int hexb_rms_norm_host(int dtype, const void *x, void *y, const void *w, int64_t rows,
                                  int64_t cols, float eps) {
  const size_t esz = dt_size(dtype);
  if (!esz) return HEXB_ERR_UNSUPPORTED;
  if (rows > 0 && cols > 0 && !w) return HEXB_ERR_BAD_ARG;
  std::lock_guard<std::mutex> lk(g_staging_mu);
  const size_t vb = align_up((size_t)cols * esz, 256);
  return rows_pipeline(
      x, y, rows, cols, esz, vb,
      [&](void *dx, void *dy, void *de, int64_t, int64_t nr, cudaStream_t s) -> int {
        if (!dx) {
          HEXB_CUDA_OK(cudaMemcpyAsync(de, w, (size_t)cols * esz, cudaMemcpyHostToDevice, s));
          return HEXB_OK;
        }
        if (nr < 0) return HEXB_OK;
        return dtype == HEXB_DT_F16
                   ? hexb_rms_norm_f16(dx, dy, de, nr, cols, cols, cols, eps, s)
                   : hexb_rms_norm_f32((const float *)dx, (float *)dy, (const float *)de, nr, cols, cols, cols, eps, s);
      });
}

extern "C" int hexb_matmul_f16_host(const void *A, const void *B, void *C, int64_t M, int64_t N,
                                    int64_t K, int out_dtype) {
  if (M < 0 || N < 0 || K < 0) return HEXB_ERR_BAD_ARG;
  const size_t osz = dt_size(out_dtype);
  if (!osz) return HEXB_ERR_UNSUPPORTED;
  if (M == 0 || N == 0) return HEXB_OK;
  if (!A || !B || !C) return HEXB_ERR_BAD_ARG;
  std::lock_guard<std::mutex> lk(g_staging_mu);
  const size_t ab = align_up((size_t)M * K * 2, 256), bb = align_up((size_t)K * N * 2, 256);
  const size_t cb = align_up((size_t)M * N * osz, 256);
  Staging *s = nullptr;
  if (int st = staging_get(ab + bb + cb, &s)) return st;
  char *dA = (char *)s->ptr, *dB = dA + ab, *dC = dB + bb;
  // B is needed whole by every row block; A goes up and C comes back in blocks of rows (multiples of
  // 256, the tile height of the CTA-pair kernel) so that the upload of block i+1, the product of
  // block i and the download of block i-1 overlap.
  int chunks = option(OPT_host_chunks, 8);
  if ((size_t)M * K * 2 < ((size_t)4 << 20)) chunks = 1;
  int64_t bounds[Staging::kMaxChunks + 1];
  chunks = chunk_plan(M, chunks, 256, bounds, 1);
  auto body = [&]() -> int {
    cudaStream_t last = nullptr;
    const int e = staged_pipeline(
        s, chunks,
        [&](int c, cudaStream_t st) -> int {
          const int64_t r0 = bounds[c], nr = bounds[c + 1] - r0;
          if (c == 0 && K > 0) HEXB_CUDA_OK(cudaMemcpyAsync(dB, B, (size_t)K * N * 2, cudaMemcpyHostToDevice, st));
          if (K > 0)
            HEXB_CUDA_OK(cudaMemcpyAsync(dA + (size_t)r0 * K * 2, (const char *)A + (size_t)r0 * K * 2, (size_t)nr * K * 2,
                                         cudaMemcpyHostToDevice, st));
          return HEXB_OK;
        },
        [&](int c, cudaStream_t st) -> int {
          const int64_t r0 = bounds[c], nr = bounds[c + 1] - r0;
          return hexb_matmul_f16(dA + (size_t)r0 * K * 2, dB, dC + (size_t)r0 * N * osz, nullptr, nr, N, K, K, N, N, out_dtype, st);
        },
        [&](int c, cudaStream_t st) -> int {
          const int64_t r0 = bounds[c], nr = bounds[c + 1] - r0;
          HEXB_CUDA_OK(cudaMemcpyAsync((char *)C + (size_t)r0 * N * osz, dC + (size_t)r0 * N * osz, (size_t)nr * N * osz,
                                       cudaMemcpyDeviceToHost, st));
          return HEXB_OK;
        },
        &last);
    if (e) return e;
    HEXB_CUDA_OK(cudaStreamSynchronize(last));
    return HEXB_OK;
  };
  const int status = body();
  if (status != HEXB_OK) staging_drain(s);
  return status;
}

extern "C" int hexb_attention_fwd_host(int dtype, const void *Q, const void *K, const void *V,
                                       void *Out, int64_t Z, int64_t H, int64_t N_CTX, int64_t D,
                                       float sm_scale, int causal) {
  const size_t esz = dt_size(dtype);
  if (!esz) return HEXB_ERR_UNSUPPORTED;
  if (Z < 0 || H < 0 || N_CTX < 0 || D < 0) return HEXB_ERR_BAD_ARG;
  if (Z == 0 || H == 0 || N_CTX == 0 || D == 0) return HEXB_OK;
  if (!Q || !K || !V || !Out) return HEXB_ERR_BAD_ARG;
  std::lock_guard<std::mutex> lk(g_staging_mu);
  // (batch, head) pairs are independent and contiguous in the [Z, H, N, D] layout: pieces of
  // consecutive pairs flow through the upload / compute / download pipeline, each computed as one
  // call with Z = 1 and H = the pairs of the piece.
  const size_t per_u = (size_t)N_CTX * D * esz;
  const int64_t units = Z * H;
  const size_t tb = align_up((size_t)units * per_u, 256);
  Staging *s = nullptr;
  if (int st = staging_get(4 * tb, &s)) return st;
  char *dq = (char *)s->ptr, *dk = dq + tb, *dv = dk + tb, *dout = dv + tb;
  int chunks = option(OPT_host_chunks, 8);
  if ((size_t)units * per_u < ((size_t)4 << 20)) chunks = 1;
  int64_t bounds[Staging::kMaxChunks + 1];
  chunks = chunk_plan(units, chunks, 1, bounds);
  auto body = [&]() -> int {
    cudaStream_t last = nullptr;
    const int e = staged_pipeline(
        s, chunks,
        [&](int c, cudaStream_t st) -> int {
          const size_t off = (size_t)bounds[c] * per_u, len = (size_t)(bounds[c + 1] - bounds[c]) * per_u;
          HEXB_CUDA_OK(cudaMemcpyAsync(dq + off, (const char *)Q + off, len, cudaMemcpyHostToDevice, st));
          HEXB_CUDA_OK(cudaMemcpyAsync(dk + off, (const char *)K + off, len, cudaMemcpyHostToDevice, st));
          HEXB_CUDA_OK(cudaMemcpyAsync(dv + off, (const char *)V + off, len, cudaMemcpyHostToDevice, st));
          return HEXB_OK;
        },
        [&](int c, cudaStream_t st) -> int {
          const size_t off = (size_t)bounds[c] * per_u;
          const int64_t nu = bounds[c + 1] - bounds[c];
          const int64_t sz = nu * N_CTX * D, sh = N_CTX * D, sn = D;
          const int64_t strides[12] = {sz, sh, sn, sz, sh, sn, sz, sh, sn, sz, sh, sn};
          return dtype == HEXB_DT_F16
                     ? hexb_attention_fwd_f16(dq + off, dk + off, dv + off, dout + off, 1, nu, N_CTX, D, strides, sm_scale,
                                              causal, st)
                     : hexb_attention_fwd_f32((const float *)(dq + off), (const float *)(dk + off), (const float *)(dv + off),
                                              (float *)(dout + off), 1, nu, N_CTX, D, strides, sm_scale, causal, st);
        },
        [&](int c, cudaStream_t st) -> int {
          const size_t off = (size_t)bounds[c] * per_u, len = (size_t)(bounds[c + 1] - bounds[c]) * per_u;
          HEXB_CUDA_OK(cudaMemcpyAsync((char *)Out + off, dout + off, len, cudaMemcpyDeviceToHost, st));
          return HEXB_OK;
        },
        &last);
    if (e) return e;
    HEXB_CUDA_OK(cudaStreamSynchronize(last));
    return HEXB_OK;
  };
  const int status = body();
  if (status != HEXB_OK) staging_drain(s);
  return status;
}
