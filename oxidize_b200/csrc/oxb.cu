// liboxb: the sm_100a kernel library of oxidize_b200, exported with a plain C ABI
// (loaded from Python with ctypes; every launcher takes raw device pointers and a stream and
// returns a cudaError_t code, 0 on success).  The library is several independently compiled translation units
// linked into one shared object (oxb.cu: globals, host utilities and the
// small kernels; oxb_gemm.cu: the tcgen05 GEMM entry points; oxb_mmq_*.cu: one packed-weight format each;
// oxb_gemv.cu; oxb_attn.cu), so that a rebuild takes the time of the slowest unit.
#include "common.cuh"
#include "quant_blocks.cuh"
#include "elementwise.cuh"
#include "gemm_tcgen05.cuh"
#include "gemv_quant.cuh"
#include "sampling.cuh"
#include "comm_fused.cuh"
#include <string.h>
using namespace oxb;

// readers of every translation unit's copy of the device status word (see common.cuh)
static OxbStatusUnit*& status_units() {
  static OxbStatusUnit* head = nullptr;
  return head;
}
void oxb_register_status_unit(OxbStatusUnit* u) {
  u->next = status_units();
  status_units() = u;
}

int g_oxb_pdl = 1;
int oxb::g_oxb_cluster_splitk = 1;
int oxb::g_oxb_gemm_l2_prefetch_kb = 0;
// Token tile of prefill-sized GEMM calls: 256-token tiles halve the weight re-reads of 128-token ones and are the
// faster choice on every projection shape of the 8B / 70B models; 128 and 0 (= by wave count) remain selectable.
int oxb::g_oxb_gemm_prefill_tn = 256;

OXB_API int oxb_set_gemm_prefill_tn(int tn) {
  const int old = oxb::g_oxb_gemm_prefill_tn;
  oxb::g_oxb_gemm_prefill_tn = (tn == 128 || tn == 256) ? tn : 0;  // 0 = choose by wave count
  return old;
}

// Weight k-blocks (16 KB each) per CTA that GEMMs launched from now on request into the L2 before their grid
// dependency resolves; the caller sets it around a GEMM that follows a collective and resets it to 0.
OXB_API int oxb_set_gemm_l2_prefetch(int kb) {
  const int old = oxb::g_oxb_gemm_l2_prefetch_kb;
  oxb::g_oxb_gemm_l2_prefetch_kb = kb < 0 ? 0 : kb;
  return old;
}

OXB_API int oxb_set_cluster_splitk(int on) {
  const int old = g_oxb_cluster_splitk;
  g_oxb_cluster_splitk = on ? 1 : 0;
  return old;
}
// Packed-weight calls of at most this many tokens take the dp4a GEMV (0 = never).  With one or two tokens it is up to
// twice as fast as the tensor-core kernel on the tall matrices (qkv, gate_up, lm_head); from three tokens on it processes
// four at a time and the tensor-core kernel wins (by 2x on the wide ffn_down shape).
int g_oxb_gemv_max_t = 2;
int g_oxb_gemv_wide = 0;
OXB_API int oxb_set_gemv_wide(int on) {
  const int old = g_oxb_gemv_wide;
  g_oxb_gemv_wide = on ? 1 : 0;
  return old;
}
OXB_API int oxb_set_gemv_max_tokens(int t) {
  const int old = g_oxb_gemv_max_t;
  g_oxb_gemv_max_t = t < 0 ? 0 : (t > GV_MAX_T ? GV_MAX_T : t);
  return old;
}
int g_oxb_ar_ll_min_world = 2;  // rank counts from which the fused all-reduce uses the LL two-shot exchange

unsigned long long* g_oxb_ar_trace = nullptr;

unsigned long long* g_oxb_attn_trace = nullptr;
OXB_API void oxb_set_attn_trace(unsigned long long* p) { g_oxb_attn_trace = p; }

// Device buffer of 16 u64 that receives phase timestamps of piece 0 of each fused all-reduce (null = off).
OXB_API void oxb_set_ar_trace(unsigned long long* p) { g_oxb_ar_trace = p; }

// w < 0 only reads the current value
OXB_API int oxb_set_ar_ll_min_world(int w) {
  const int old = g_oxb_ar_ll_min_world;
  if (w >= 0) g_oxb_ar_ll_min_world = w;
  return old;
}

// Switch programmatic dependent launch on or off (also: environment OXB_PDL=0 at load time).
OXB_API int oxb_set_pdl(int on) {
  const int old = g_oxb_pdl;
  g_oxb_pdl = on ? 1 : 0;
  return old;
}

// ----------------------------------------------------------------------------- host utilities
PFN_encodeTiled oxb_get_encode_tiled() {
  static PFN_encodeTiled fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_encodeTiled>(p);
  }
  return fn;
}

int oxb_make_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride_bytes,
                     uint32_t box_rows, uint32_t box_cols, int elem_bytes) {
  PFN_encodeTiled enc = oxb_get_encode_tiled();
  if (enc == nullptr) return (int)cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (row_stride_bytes & 15) != 0) return (int)cudaErrorInvalidValue;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = enc(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// Byte view of packed weight rows for the staged MMQ path: [rows, row_bytes] uint8, no swizzle.
int oxb_make_tmap_bytes(CUtensorMap* out, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows,
                        uint32_t box_bytes) {
  // 32-bit elements: a box may then be up to 1 KB wide (256 elements); coordinates are in words
  PFN_encodeTiled enc = oxb_get_encode_tiled();
  if (enc == nullptr) return (int)cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (row_bytes & 15) != 0 || (box_bytes & 15) != 0 || box_bytes > 1024)
    return (int)cudaErrorInvalidValue;
  cuuint64_t dims[2] = {row_bytes / 4, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {box_bytes / 4, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// SM count of the current device (cached per device ordinal)
int oxb_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}
static int sm_count() { return oxb_sm_count(); }

OXB_API int oxb_version() { return 100; }

// Copy the device status word {code, detail, count, _} to the host (synchronises the device).
OXB_API int oxb_status(int* out4, int reset) {
  out4[0] = out4[1] = out4[2] = out4[3] = 0;
  for (OxbStatusUnit* u = status_units(); u != nullptr; u = u->next) {
    int s[4] = {0, 0, 0, 0};
    const int e = u->read(s, reset);
    if (e != 0) return e;
    if (out4[0] == 0 && s[0] != 0) {
      out4[0] = s[0];
      out4[1] = s[1];
    }
    out4[2] += s[2];
  }
  return 0;
}

// One-shot all-reduce (sum) of X[T, N] bf16 (row stride ld) into Y through the same symmetric buffers.
OXB_API int oxb_allreduce_oneshot(const void* X, void* Y, int T, int N, int ld, int world, int rank,
                                  const uint64_t* data_ptrs, const uint64_t* flag_ptrs, int* ctrl, int t_max, int n_max,
                                  int max_tiles, unsigned long long timeout_ns, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  const int tiles = (N + 127) / 128;
  // LL exchange: pieces of 16 tokens (more CTAs, shorter polls); one-shot: one piece per column tile (one flag each)
  const int ll = world >= g_oxb_ar_ll_min_world;
  const int tg = ll ? 16 : T;
  const int groups = (T + tg - 1) / tg;
  if (N % 8 != 0 || T > t_max || N > n_max || (!ll && tiles > max_tiles) || tiles * groups > sm_count() * 8 ||
      tg * 256 > 200 * 1024)
    return (int)cudaErrorInvalidValue;
  ArArgs ar;
  int e = fill_ar(ar, world, rank, data_ptrs, flag_ptrs, ctrl, t_max, n_max, max_tiles, timeout_ns, nullptr);
  if (e) return e;
  const size_t smem = (size_t)tg * 256;
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    cudaError_t ce = cudaFuncSetAttribute(allreduce_oneshot_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return (int)ce;
    configured = smem;
  }
  oxb_launch(allreduce_oneshot_kernel, dim3(tiles, groups), dim3(128), smem, stream, ar,
             reinterpret_cast<const __nv_bfloat16*>(X), reinterpret_cast<__nv_bfloat16*>(Y), T, N, ld, tg);
  OXB_CHECK_LAUNCH();
  return 0;
}

// ----------------------------------------------------------------------------- dequant / embed / norms
__global__ void dequant_rows_kernel(const uint8_t* __restrict__ src, int qtype, size_t row_bytes, int cols,
                                    __nv_bfloat16* __restrict__ dst) {
  const uint8_t* row = src + (size_t)blockIdx.x * row_bytes;
  __nv_bfloat16* o = dst + (size_t)blockIdx.x * cols;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) o[i] = __float2bfloat16(dequant_elem(qtype, row, i));
}

// Fast form for the block formats the GEMM's producers decode: one thread per (row, 64-value k-block) runs the same
// mantissa-trick decoder and writes its 128 bytes with eight 16-byte stores; a warp covers 32 consecutive k-blocks
// of a row, so the stores of a warp are one contiguous 4 KB run.
template <int QT>
static __global__ void dequant_rows_fast_kernel(const uint8_t* __restrict__ src, size_t row_bytes, int rows, int cols,
                                                __nv_bfloat16* __restrict__ dst) {
  const int kbs = cols >> 6;
  const long long total = (long long)rows * kbs;
  const QwArgs qw{nullptr, row_bytes, nullptr, 0, 0};
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(t / kbs), kb = (int)(t % kbs);
    uint4* out = reinterpret_cast<uint4*>(dst + (size_t)r * cols + (size_t)kb * 64);
    dequant64_chunks<QT>(src + (size_t)r * row_bytes, kb * 64, qw, 0,
                         [&](int c, uint32_t a, uint32_t b, uint32_t cc, uint32_t d) { out[c] = make_uint4(a, b, cc, d); });
  }
}

// fast != 0: the vectorised decoder where it applies.  Its scales and offsets enter the arithmetic as bf16, exactly as
// in the fused GEMM (about 2^-9 of the sub-block's range per value); fast == 0 always takes the exact per-element form.
OXB_API int oxb_dequant_rows(const void* src, int qtype, size_t row_bytes, int rows, int cols, void* dst_bf16, int fast,
                             cudaStream_t stream) {
  if (rows <= 0) return 0;
  const uint8_t* s8 = reinterpret_cast<const uint8_t*>(src);
  __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(dst_bf16);
  // Q4_K blocks are read with 16-byte loads, Q6_K / Q8_0 blocks through aligned words from any even address
  const size_t src_align = qtype == QT_Q4_K ? 16 : 2;
  const bool aligned = cols % 64 == 0 && (reinterpret_cast<uintptr_t>(dst_bf16) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(src) % src_align) == 0 && row_bytes % src_align == 0 &&
                       (qtype != QT_Q8_0 || (reinterpret_cast<uintptr_t>(src) & 3) == 0);
  if (fast && aligned && (qtype == QT_Q4_K || qtype == QT_Q6_K || qtype == QT_Q8_0)) {
    const long long total = (long long)rows * (cols >> 6);
    const int blocks = (int)((total + 255) / 256 < (long long)sm_count() * 16 ? (total + 255) / 256 : (long long)sm_count() * 16);
    if (qtype == QT_Q4_K) dequant_rows_fast_kernel<QT_Q4_K><<<blocks, 256, 0, stream>>>(s8, row_bytes, rows, cols, d);
    else if (qtype == QT_Q6_K) dequant_rows_fast_kernel<QT_Q6_K><<<blocks, 256, 0, stream>>>(s8, row_bytes, rows, cols, d);
    else dequant_rows_fast_kernel<QT_Q8_0><<<blocks, 256, 0, stream>>>(s8, row_bytes, rows, cols, d);
    OXB_CHECK_LAUNCH();
    return 0;
  }
  dequant_rows_kernel<<<rows, 256, 0, stream>>>(s8, qtype, row_bytes, cols, d);
  OXB_CHECK_LAUNCH();
  return 0;
}

OXB_API int oxb_embed(const int* tokens, const void* table, int qtype, size_t row_bytes, int H, int vocab, float scale,
                      void* out_bf16, int T, cudaStream_t stream) {
  if (T <= 0) return 0;
  oxb_launch(embed_kernel, dim3(T), dim3(256), 0, stream, tokens, reinterpret_cast<const uint8_t*>(table), qtype, row_bytes,
             H, vocab, scale, reinterpret_cast<__nv_bfloat16*>(out_bf16));
  OXB_CHECK_LAUNCH();
  return 0;
}

OXB_API int oxb_add_rmsnorm(const void* x, const void* res_in, void* res_out, const float* w, void* y, int T, int H,
                            float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* rb = reinterpret_cast<const __nv_bfloat16*>(res_in);
  __nv_bfloat16* ro = reinterpret_cast<__nv_bfloat16*>(res_out);
  __nv_bfloat16* yb = reinterpret_cast<__nv_bfloat16*>(y);
  if (H % 8 == 0 && H / 8 <= 4096) {
    const int H8 = H / 8;
    const int ch = H8 <= 1024 ? 1 : (H8 <= 2048 ? 2 : 4);
    const int threads = ((H8 + ch - 1) / ch + 31) / 32 * 32;
    if (ch == 1) oxb_launch(add_rmsnorm_reg_kernel<1>, dim3(T), dim3(threads), 0, stream, xb, rb, ro, w, yb, H, eps);
    else if (ch == 2) oxb_launch(add_rmsnorm_reg_kernel<2>, dim3(T), dim3(threads), 0, stream, xb, rb, ro, w, yb, H, eps);
    else oxb_launch(add_rmsnorm_reg_kernel<4>, dim3(T), dim3(threads), 0, stream, xb, rb, ro, w, yb, H, eps);
    OXB_CHECK_LAUNCH();
    return 0;
  }
  const size_t smem = (size_t)H * sizeof(float);
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  const int threads = H >= 4096 ? 512 : 256;
  add_rmsnorm_kernel<<<T, threads, smem, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(res_in),
      reinterpret_cast<__nv_bfloat16*>(res_out), w, reinterpret_cast<__nv_bfloat16*>(y), H, eps);
  OXB_CHECK_LAUNCH();
  return 0;
}

// out[t] = fixed-point sum of squares of row t of x[T, H] (bf16); `clear` (optional, [T]) is reset to zero.
OXB_API int oxb_row_sumsq(const void* x, int ldx, int T, int H, void* out, void* clear, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0 || ldx % 8 != 0) return (int)cudaErrorInvalidValue;
  oxb_launch(row_sumsq_kernel, dim3((T + 7) / 8), dim3(256), 0, stream, reinterpret_cast<const __nv_bfloat16*>(x), ldx, T, H,
             reinterpret_cast<unsigned long long*>(out), reinterpret_cast<unsigned long long*>(clear));
  OXB_CHECK_LAUNCH();
  return 0;
}

template <bool GELU>
static int gated_act_mul(const void* gu, void* out, int T, int I, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (I % 8 != 0) return (int)cudaErrorInvalidValue;
  const size_t total = (size_t)T * (I / 8);
  int blocks = (int)((total + 255) / 256);
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  oxb_launch(silu_mul_kernel<GELU>, dim3(blocks), dim3(256), 0, stream, reinterpret_cast<const __nv_bfloat16*>(gu),
             reinterpret_cast<__nv_bfloat16*>(out), T, I);
  OXB_CHECK_LAUNCH();
  return 0;
}

OXB_API int oxb_silu_mul(const void* gu, void* out, int T, int I, cudaStream_t stream) {
  return gated_act_mul<false>(gu, out, T, I, stream);
}

// tanh-GELU(gate) * up (GeGLU)
OXB_API int oxb_gelu_mul(const void* gu, void* out, int T, int I, cudaStream_t stream) {
  return gated_act_mul<true>(gu, out, T, I, stream);
}

OXB_API int oxb_qk_rope_kvwrite(const void* qkv, const int* positions, const int* slots, const float* cos_sin,
                                int max_pos, int rot, int pairing, const float* q_norm, const float* k_norm, float eps,
                                int T, int nq, int nkv, int hd, void* q_out, void* kv_data, float* kv_scales,
                                int kv_mode, int page, int num_blocks, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hd % 32 != 0 || hd > 1024) return (int)cudaErrorInvalidValue;
  KvWriteArgs kv{kv_data, kv_scales, kv_mode, page, nkv, num_blocks};
  dim3 grid(T, nq + 2 * nkv);
  oxb_launch(qk_rope_kvwrite_kernel, grid, dim3(hd), hd * sizeof(float), stream,
             reinterpret_cast<const __nv_bfloat16*>(qkv), positions, slots, cos_sin, max_pos, rot, pairing, q_norm, k_norm,
             eps, nq, nkv, hd, reinterpret_cast<__nv_bfloat16*>(q_out), kv);
  OXB_CHECK_LAUNCH();
  return 0;
}

OXB_API int oxb_argmax(const float* logits, int R, int V, int ld, int tie_highest, int* out, float* out_val,
                       int index_offset, cudaStream_t stream) {
  if (R <= 0) return 0;
  oxb_launch(argmax_kernel, dim3(R), dim3(1024), 0, stream, logits, V, ld, tie_highest, out, out_val, index_offset);
  OXB_CHECK_LAUNCH();
  return 0;
}

// Greedy token per row of this rank's logits shard [R, V] (dtype: 0 = fp32, 2 = bf16), exchanged with the other
// tensor-parallel ranks inside the kernel when world > 1 (peer_bufs: every rank's exchange buffer
// [2][world][rmax][2] u64, zeroed once; ctrl: 2 local ints, zeroed once).  out2 (optional) receives the tokens too.
OXB_API int oxb_argmax_tp(const void* logits, int dtype, int R, int V, int ld, int tie_highest, int* out, int* out2,
                          int index_offset, int world, int rank, const uint64_t* peer_bufs, int* ctrl, int rmax,
                          unsigned long long timeout_ns, cudaStream_t stream) {
  if (R <= 0) return 0;
  ArgmaxXchg xa;
  memset(&xa, 0, sizeof(xa));
  if (world > 1) {
    if (world > 8 || rank < 0 || rank >= world || peer_bufs == nullptr || ctrl == nullptr || R > rmax) return (int)cudaErrorInvalidValue;
    xa.world = world;
    xa.rank = rank;
    xa.ctrl = ctrl;
    xa.rmax = rmax;
    xa.timeout_ns = timeout_ns;
    for (int i = 0; i < world; ++i) xa.bufs[i] = reinterpret_cast<unsigned long long*>(peer_bufs[i]);
  }
  if (dtype == 0) {
    oxb_launch(argmax_tp_kernel<float>, dim3(R), dim3(1024), 0, stream, reinterpret_cast<const float*>(logits), V, ld, tie_highest,
               out, out2, index_offset, xa);
  } else if (dtype == 2) {
    oxb_launch(argmax_tp_kernel<__nv_bfloat16>, dim3(R), dim3(1024), 0, stream, reinterpret_cast<const __nv_bfloat16*>(logits), V,
               ld, tie_highest, out, out2, index_offset, xa);
  } else {
    return (int)cudaErrorInvalidValue;
  }
  OXB_CHECK_LAUNCH();
  return 0;
}

// Per-row sampling of fp32 logits [R, V] (row stride ld) with per-row knobs and uniforms.
OXB_API int oxb_sample(const float* logits, int R, int V, int ld, const float* temperature, const int* top_k,
                       const float* top_p, const float* min_p, const float* random, int tie_highest, int* out,
                       cudaStream_t stream) {
  if (R <= 0) return 0;
  oxb_launch(sample_kernel, dim3(R), dim3(SMP_THREADS), 0, stream, logits, V, ld, temperature, top_k, top_p, min_p, random,
             tie_highest, out);
  OXB_CHECK_LAUNCH();
  return 0;
}

// Speculative verification of S sequences in one launch (see SpecVerifyArgs in sampling.cuh).
OXB_API int oxb_spec_verify(const float* target, int ld_t, const float* draft, int ld_d, const int* draft_tokens, const int* row0,
                            const int* n_draft, const float* temperature, const float* uniforms, int* out_tokens, int* out_count,
                            int S, int K, int V, int tie_highest, cudaStream_t stream) {
  if (S <= 0) return 0;
  if (K < 1 || K > 64 || V <= 0) return (int)cudaErrorInvalidValue;
  SpecVerifyArgs a{target, draft, draft_tokens, row0, n_draft, temperature, uniforms, out_tokens, out_count, V, K, ld_t, ld_d,
                   tie_highest};
  oxb_launch(spec_verify_kernel, dim3(S), dim3(SMP_THREADS), 0, stream, a);
  OXB_CHECK_LAUNCH();
  return 0;
}

// ----------------------------------------------------------------------------- mixture of experts
#include "moe.cuh"

OXB_API int oxb_moe_route(const float* logits, int T, int E, int ld, int k, int sigmoid, const float* sel_bias, int renorm,
                          float weight_scale, int* ids, float* wts, float* scale, int scale_ld, int first_local,
                          int n_local, int n_groups, int groups_used, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E > MOE_MAX_EXPERTS || k > MOE_MAX_TOPK || k < 1 || k > E) return (int)cudaErrorInvalidValue;
  if (n_groups > 1 && (n_groups > 32 || E % n_groups != 0 || groups_used > n_groups)) return (int)cudaErrorInvalidValue;
  const int warps = 4;
  cudaError_t e = oxb_launch(moe_route_kernel, dim3((T + warps - 1) / warps), dim3(warps * 32), 0, stream, logits, T, E, ld,
                             k, sigmoid, sel_bias, renorm, weight_scale, ids, wts, scale, scale_ld, first_local, n_local,
                             n_groups, groups_used);
  if (e != cudaSuccess) return (int)e;
  OXB_CHECK_LAUNCH();
  return 0;
}

OXB_API int oxb_moe_combine(const void* y, const float* scale, int scale_ld, const void* shared, void* out, int E, int T,
                            int H, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0) return (int)cudaErrorInvalidValue;
  cudaError_t e = oxb_launch(moe_combine_kernel, dim3(T), dim3(256), 0, stream, reinterpret_cast<const __nv_bfloat16*>(y),
                             scale, scale_ld, reinterpret_cast<const __nv_bfloat16*>(shared),
                             reinterpret_cast<__nv_bfloat16*>(out), E, T, H);
  if (e != cudaSuccess) return (int)e;
  OXB_CHECK_LAUNCH();
  return 0;
}


// ----------------------------------------------------------------------------- mixture of experts: token dispatch / combine
OXB_API int oxb_moe_permute(const int* ids, int T, int k, int first_local, int n_local, int* offsets, int* perm, int* inv,
                            cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n_local < 1 || n_local > MOE_MAX_EXPERTS || k < 1) return (int)cudaErrorInvalidValue;
  oxb_launch(moe_permute_kernel, dim3(1), dim3(1024), 0, stream, ids, T, k, first_local, n_local, offsets, perm, inv);
  OXB_CHECK_LAUNCH();
  return 0;
}

OXB_API int oxb_moe_gather(const void* X, int H, const int* perm, const int* n_rows_dev, int rows_cap, void* Xg,
                           cudaStream_t stream) {
  if (rows_cap <= 0) return 0;
  if (H % 8 != 0) return (int)cudaErrorInvalidValue;
  int grid = rows_cap < oxb_sm_count() * 8 ? rows_cap : oxb_sm_count() * 8;
  oxb_launch(moe_gather_kernel, dim3(grid), dim3(H / 8 < 256 ? ((H / 8 + 31) / 32 * 32) : 256), 0, stream,
             reinterpret_cast<const __nv_bfloat16*>(X), H, perm, n_rows_dev, reinterpret_cast<__nv_bfloat16*>(Xg));
  OXB_CHECK_LAUNCH();
  return 0;
}

OXB_API int oxb_silu_mul_rows(const void* gu, void* out, const int* n_rows_dev, int rows_cap, int I, cudaStream_t stream) {
  if (rows_cap <= 0) return 0;
  if (I % 8 != 0) return (int)cudaErrorInvalidValue;
  const size_t total = (size_t)rows_cap * (I / 8);
  int blocks = (int)((total + 255) / 256);
  if (blocks > oxb_sm_count() * 16) blocks = oxb_sm_count() * 16;
  oxb_launch(silu_mul_rows_kernel, dim3(blocks), dim3(256), 0, stream, reinterpret_cast<const __nv_bfloat16*>(gu),
             reinterpret_cast<__nv_bfloat16*>(out), n_rows_dev, I);
  OXB_CHECK_LAUNCH();
  return 0;
}

// out[t] = sum_k wts[t, k] * Y[inv[t, k]] (+ shared).  With world > 1 the partial sums of the expert-parallel ranks are
// all-reduced inside the same kernel through the symmetric buffers of the fused collectives (arguments as oxb_gemm_ar).
OXB_API int oxb_moe_combine_gathered(const void* Y, const int* inv, const float* wts, int k, const void* shared, void* out,
                                     int T, int H, int world, int rank, const uint64_t* data_ptrs, const uint64_t* flag_ptrs,
                                     int* ctrl, int t_max, int n_max, int max_tiles, unsigned long long timeout_ns,
                                     cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0) return (int)cudaErrorInvalidValue;
  const __nv_bfloat16* y = reinterpret_cast<const __nv_bfloat16*>(Y);
  const __nv_bfloat16* sh = reinterpret_cast<const __nv_bfloat16*>(shared);
  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out);
  if (world <= 1) {
    oxb_launch(moe_combine_gathered_kernel, dim3(T), dim3(256), 0, stream, y, inv, wts, k, sh, o, T, H);
    OXB_CHECK_LAUNCH();
    return 0;
  }
  const int tiles = (H + 127) / 128;
  const int tg = 16;
  const int groups = (T + tg - 1) / tg;
  if (world < g_oxb_ar_ll_min_world || T > t_max || H > n_max || tiles * groups > sm_count() * 8) return (int)cudaErrorInvalidValue;
  ArArgs ar;
  int e = fill_ar(ar, world, rank, data_ptrs, flag_ptrs, ctrl, t_max, n_max, max_tiles, timeout_ns, nullptr);
  if (e) return e;
  oxb_launch(moe_combine_exchange_kernel, dim3(tiles, groups), dim3(128), (size_t)tg * 256, stream, ar, y, inv, wts, k, sh, o, T,
             H, tg);
  OXB_CHECK_LAUNCH();
  return 0;
}
