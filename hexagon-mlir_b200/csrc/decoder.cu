// Decoder-only block stack, forward pass, composed on one stream from the library's own kernels.
//
// There is no single reference function for this: the reference runs whole models by compiling
// the graph (test/python/torch-mlir/gpt2lmheadmodel.py:143-169 of qualcomm/hexagon-mlir); the
// blocks here are built from the operators of its Triton tests: rms_norm_fwd_kernel
// (test_rms_norm.py:37-63), matmul (test_matmul.py:35-70), attention_fwd_kernel
// (test_flash_attention.py:37-168, causal) and silu_kernel (test_silu.py:38-52).
//
//   h  = x + Attn(RMSNorm(x, g1) . Wqkv) . Wo
//   x' = h + (SiLU(n . Wg) * (n . Wu)) . Wd,   n = RMSNorm(h, g2)
//
// Heads are split and merged by strides inside the attention call (q|k|v column blocks of the
// QKV product, head-major inside each block); no transposes.  The residual adds ride in the
// epilogue of the Wo and Wd products, the SwiGLU gating in the epilogue of the gate/up product.
#include <mutex>

#include "common.cuh"

namespace hexb {

struct DecoderPlan {
  size_t n_off, qkv_off, attn_off, h_off, gu_off, act_off, x_off, total;
};

static inline size_t up256(size_t v) { return (v + 255) / 256 * 256; }

static int decoder_plan(const hexb_decoder_config *c, DecoderPlan *p) {
  if (!c) return HEXB_ERR_BAD_ARG;
  if (c->n_layers < 0 || c->d_model <= 0 || c->n_heads <= 0 || c->head_dim <= 0 || c->d_ff <= 0 ||
      c->batch < 0 || c->seq < 0)
    return HEXB_ERR_BAD_ARG;
  if ((int64_t)c->n_heads * c->head_dim != c->d_model) return HEXB_ERR_BAD_ARG;
  if (c->d_model % 8 || c->d_ff % 8) return HEXB_ERR_UNSUPPORTED;
  const size_t T = (size_t)c->batch * c->seq, d = c->d_model, f = c->d_ff;
  size_t off = 0;
  p->n_off = off;    off += up256(T * d * 2);
  p->qkv_off = off;  off += up256(T * 3 * d * 2);
  p->attn_off = off; off += up256(T * d * 2);
  p->h_off = off;    off += up256(T * d * 2);
  p->gu_off = off;   off += up256(T * 2 * f * 2);
  p->act_off = off;  off += up256(T * f * 2);
  p->x_off = off;    off += up256(T * d * 2);
  p->total = off;
  return HEXB_OK;
}

}  // namespace hexb

extern "C" size_t hexb_decoder_workspace_bytes(const hexb_decoder_config *cfg) {
  hexb::DecoderPlan p;
  if (hexb::decoder_plan(cfg, &p)) return 0;
  return p.total;
}

extern "C" int hexb_decoder_forward_f16(const hexb_decoder_config *cfg, const hexb_decoder_weights *w,
                                        const void *x, void *out, void *workspace,
                                        size_t workspace_bytes, void *stream) {
  using namespace hexb;
  DecoderPlan p;
  if (int s = decoder_plan(cfg, &p)) return s;
  const int64_t T = (int64_t)cfg->batch * cfg->seq;
  if (T == 0) return HEXB_OK;
  if (!x || !out) return HEXB_ERR_BAD_ARG;
  const int64_t d = cfg->d_model, f = cfg->d_ff, hd = cfg->head_dim, S = cfg->seq;
  if (cfg->n_layers == 0) {
    HEXB_CUDA_OK(cudaMemcpyAsync(out, x, (size_t)T * d * 2, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    return HEXB_OK;
  }
  if (!w || !w->wqkv || !w->wo || !w->wgu || !w->wd || !w->g1 || !w->g2) return HEXB_ERR_BAD_ARG;
  if (!workspace || workspace_bytes < p.total) return HEXB_ERR_WORKSPACE;
  if (!aligned16(workspace)) return HEXB_ERR_MISALIGNED;
  char *ws = (char *)workspace;
  void *n = ws + p.n_off, *qkv = ws + p.qkv_off, *attn = ws + p.attn_off, *h = ws + p.h_off,
       *gu = ws + p.gu_off, *act = ws + p.act_off, *xbuf = ws + p.x_off;
  const char *qkv_c = (const char *)qkv;
  const int64_t strides[12] = {S * 3 * d, hd, 3 * d, S * 3 * d, hd, 3 * d, S * 3 * d, hd, 3 * d,
                               S * d,     hd, d};
  const float scale = 1.0f / sqrtf((float)hd);
  const void *xin = x;
  for (int l = 0; l < cfg->n_layers; ++l) {
    void *xout = (l == cfg->n_layers - 1) ? out : xbuf;
    int s;
    if ((s = hexb_rms_norm_f16(xin, n, w->g1[l], T, d, d, d, cfg->rms_eps, stream))) return s;
    if ((s = hexb_matmul_f16(n, w->wqkv[l], qkv, nullptr, T, 3 * d, d, d, 3 * d, 3 * d, HEXB_DT_F16, stream))) return s;
    if ((s = hexb_attention_fwd_f16(qkv_c, qkv_c + d * 2, qkv_c + 2 * d * 2, attn, cfg->batch,
                                    cfg->n_heads, S, hd, strides, scale, 1, stream)))
      return s;
    if ((s = hexb_matmul_f16(attn, w->wo[l], h, xin, T, d, d, d, d, d, HEXB_DT_F16, stream))) return s;
    if ((s = hexb_rms_norm_f16(h, n, w->g2[l], T, d, d, d, cfg->rms_eps, stream))) return s;
    if (option(OPT_decoder_fused_swiglu, 1)) {
      if ((s = hexb_matmul_swiglu_f16(n, w->wgu[l], act, T, f, d, d, 2 * f, f, stream))) return s;
    } else {
      if ((s = hexb_matmul_f16(n, w->wgu[l], gu, nullptr, T, 2 * f, d, d, 2 * f, 2 * f, HEXB_DT_F16, stream))) return s;
      if ((s = hexb_swiglu_f16(gu, act, T, f, stream))) return s;
    }
    if ((s = hexb_matmul_f16(act, w->wd[l], xout, h, T, d, f, f, d, d, HEXB_DT_F16, stream))) return s;
    xin = xout;
  }
  return HEXB_OK;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant.  The workspace of hexb_decoder_forward_f16 is replaced by a fixed array
// in the library image, for hosts that cannot call cudaMalloc at this point (all device memory
// already handed to their own pool, or a latency bound that rules out an allocation).
//
// In host code `g_decoder_scratch` is only a handle for the symbol, not a device address: its
// address is fetched once per device with cudaGetSymbolAddress while that device is current, and
// that pointer is what the kernels receive.  The array is shared by every call on the device and
// keeps the previous call's contents; the block stack writes each intermediate before reading it,
// so no clearing is needed, but overlapping calls on one device would race on it.
static __device__ __align__(256) unsigned char g_decoder_scratch[HEXB_DECODER_STATIC_SCRATCH_BYTES];

extern "C" int hexb_decoder_forward_f16_noalloc(const hexb_decoder_config *cfg,
                                                const hexb_decoder_weights *w, const void *x,
                                                void *out, void *stream) {
  using namespace hexb;
  static void *scratch_ptr[64] = {};
  static std::mutex mu;
  DecoderPlan p;
  if (int s = decoder_plan(cfg, &p)) return s;
  if (p.total > (size_t)HEXB_DECODER_STATIC_SCRATCH_BYTES) return HEXB_ERR_WORKSPACE;  // beyond the fixed array
  int dev = -1;
  HEXB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return HEXB_ERR_NO_DEVICE;
  void *ptr = nullptr;
  {
    std::lock_guard<std::mutex> lk(mu);
    if (!scratch_ptr[dev]) {
      void *sym = nullptr;
      HEXB_CUDA_OK(cudaGetSymbolAddress((void **)&sym, g_decoder_scratch));  // device `dev` is current
      scratch_ptr[dev] = sym;
    }
    ptr = scratch_ptr[dev];
  }
  return hexb_decoder_forward_f16(cfg, w, x, out, ptr, (size_t)HEXB_DECODER_STATIC_SCRATCH_BYTES, stream);
}
