// liboxb, paged attention entry points.
#include "common.cuh"
#include "attention.cuh"
using namespace oxb;

// ----------------------------------------------------------------------------- attention
// Sizes of the split-KV scratch for a launch shape (floats).
OXB_API int oxb_attn_ws_floats(int B, int nkv, int max_mtiles, int n_cta_splits, int hd, size_t* o_floats,
                               size_t* ml_floats) {
  const size_t tasks = (size_t)B * nkv * max_mtiles * n_cta_splits;
  *o_floats = n_cta_splits > 1 ? tasks * 16 * hd : 0;
  *ml_floats = n_cta_splits > 1 ? tasks * 16 * 2 : 0;
  return 0;
}

template <int HD>
static int attn_launch(const AttnArgs& a, int B, int G, cudaStream_t stream) {
  constexpr int STAGE = 32 * (HD * 2 + 16);
  constexpr int SMEM_MAX = ATT_WARPS * (ATT_STAGES + 1) * STAGE;
  // quantized KV needs one extra decode buffer per warp
  const int smem = ATT_WARPS * (ATT_STAGES + (a.kv_mode >= 2 ? 1 : 0)) * STAGE;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(paged_attention_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_MAX);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(a.max_mtiles * a.n_cta_splits, a.nkv, B);
  // (The KV splits of a row tile stay independent CTAs and the last one to finish merges: inside a thread-block
  // cluster every CTA would wait for the slowest split.)
  if (a.n_cta_splits > 1 && (a.ws_o == nullptr || a.ws_ml == nullptr || a.counters == nullptr)) return (int)cudaErrorInvalidValue;
  oxb_launch(paged_attention_kernel<HD>, grid, dim3(ATT_WARPS * 32), (size_t)smem, stream, a, G);
  OXB_CHECK_LAUNCH();
  return 0;
}

OXB_API int oxb_paged_attention(const void* q, void* out, const void* kv_data, const float* kv_scales,
                                const int* block_tables, const int* seq_lens, const int* query_start, int B,
                                int max_blocks, int nq, int nkv, int hd, int kv_mode, int max_query_len,
                                int n_cta_splits, int window, float scale, float softcap, float* ws_o, float* ws_ml,
                                int* counters, int num_blocks, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (nq % nkv != 0) return (int)cudaErrorInvalidValue;
  const int G = nq / nkv;
  AttnArgs a;
  a.q = reinterpret_cast<const __nv_bfloat16*>(q);
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.kv_data = kv_data;
  a.kv_scales = kv_scales;
  a.block_tables = block_tables;
  a.seq_lens = seq_lens;
  a.query_start = query_start;
  a.max_blocks = max_blocks;
  a.nq = nq;
  a.nkv = nkv;
  a.kv_mode = kv_mode;
  a.n_cta_splits = n_cta_splits < 1 ? 1 : n_cta_splits;
  a.max_mtiles = (max_query_len * G + 15) / 16;
  a.window = window;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.cap_log2 = softcap > 0.f ? softcap * 1.4426950408889634f : 0.f;
  a.cap_arg = softcap > 0.f ? scale / softcap : 0.f;
  a.ws_o = ws_o;
  a.ws_ml = ws_ml;
  a.counters = counters;
  a.num_blocks = num_blocks;
  a.trace = g_oxb_attn_trace;
  if (hd == 128) return attn_launch<128>(a, B, G, stream);
  if (hd == 64) return attn_launch<64>(a, B, G, stream);
  return (int)cudaErrorInvalidValue;
}

