// liboxb: the sm_100a kernel library of oxidize_b200, exported with a plain C ABI
// (loaded from Python with ctypes; every launcher takes raw device pointers and a stream and
// returns a cudaError_t code, 0 on success).  Built as ONE translation unit.
#include "common.cuh"
#include "quant_blocks.cuh"
#include "elementwise.cuh"
#include "gemm_tcgen05.cuh"
#include "attention.cuh"
#include "sampling.cuh"
#include "comm_fused.cuh"
using namespace oxb;

int g_oxb_pdl = 1;
int oxb::g_oxb_cluster_splitk = 1;
int oxb::g_oxb_gemm_l2_prefetch_kb = 0;
int oxb::g_oxb_gemm_prefill_tn = 256;  // until the 128-token choice is measured: keep 256

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
int g_oxb_ar_ll_min_world = 2;  // rank counts from which the fused all-reduce uses the LL two-shot exchange

static unsigned long long* g_oxb_ar_trace = nullptr;

static unsigned long long* g_oxb_attn_trace = nullptr;
OXB_API void oxb_set_attn_trace(unsigned long long* p) { g_oxb_attn_trace = p; }

// Device buffer of 16 u64 that receives phase timestamps of piece 0 of each fused all-reduce (null = off).
OXB_API void oxb_set_ar_trace(unsigned long long* p) { g_oxb_ar_trace = p; }

OXB_API int oxb_set_ar_ll_min_world(int w) {
  const int old = g_oxb_ar_ll_min_world;
  g_oxb_ar_ll_min_world = w;
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
  PFN_encodeTiled enc = oxb_get_encode_tiled();
  if (enc == nullptr) return (int)cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (row_bytes & 15) != 0 || (box_bytes & 15) != 0 || box_bytes > 256)
    return (int)cudaErrorInvalidValue;
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {box_bytes, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

OXB_API int oxb_version() { return 100; }

// Copy the device status word {code, detail, count, _} to the host (synchronises the device).
OXB_API int oxb_status(int* out4, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(out4, g_oxb_status, 4 * sizeof(int));
  if (e != cudaSuccess) return (int)e;
  if (reset) {
    int z[4] = {0, 0, 0, 0};
    e = cudaMemcpyToSymbol(g_oxb_status, z, sizeof(z));
  }
  return (int)e;
}

// ----------------------------------------------------------------------------- GEMM
OXB_API int oxb_gemm_plan(int T, int N, int K, int splits_hint, int* out4, size_t* ws_bytes, int* n_counters) {
  GemmPlan p = gemm_plan(T, N, K, splits_hint, sm_count());
  out4[0] = p.tn;
  out4[1] = p.n_tiles;
  out4[2] = p.t_tiles;
  out4[3] = p.splits;
  *ws_bytes = p.ws_bytes;
  *n_counters = p.n_counters;
  return 0;
}

// Y[T, ldY>=N] (bf16) = X[T, K] (bf16, contiguous) · W[N, K]^T (bf16, contiguous) (+bias f32[N]).
// `ws` (fp32 scratch) and `counters` (zero-initialised ints, left zeroed) are only touched when
// the plan splits K; if they are too small the split count is reduced to fit.
OXB_API int oxb_gemm_bf16(const void* X, const void* W, void* Y, const float* bias, int T, int N, int K, int ldY,
                          int epi_mode, int splits_hint, void* ws, size_t ws_bytes, int* counters, int n_counters,
                          cudaStream_t stream) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 8 != 0) return (int)cudaErrorInvalidValue;  // TMA rows must be 16-byte multiples
  const bool swiglu = epi_mode == EPI_SWIGLU;
  // the SwiGLU epilogue exists on the staged (vector-store) paths only: whole 128-row tiles, 16-byte output rows
  if (swiglu && (N % GEMM_BM != 0 || ldY % 8 != 0 || (reinterpret_cast<uintptr_t>(Y) & 15) != 0 || bias != nullptr))
    return (int)cudaErrorInvalidValue;
  GemmPlan p = gemm_plan(T, N, K, splits_hint, sm_count(), swiglu ? 1 : -1);
  // split-K CTAs of a tile wait for one another, so the whole grid has to fit in one wave
  while (p.splits > 1 && !p.cluster && (p.ws_bytes > ws_bytes || p.n_counters > n_counters || ws == nullptr || counters == nullptr ||
                          p.n_tiles * p.t_tiles * p.splits > sm_count()))
    p = gemm_plan(T, N, K, p.splits - 1, sm_count());
  CUtensorMap tmW, tmX;
  int e = oxb_make_tmap_2d(&tmW, W, N, K, (uint64_t)K * 2, GEMM_BM, GEMM_BK, 2);
  if (e) return e;
  e = oxb_make_tmap_2d(&tmX, X, T, K, (uint64_t)K * 2, p.tn, GEMM_BK, 2);
  if (e) return e;
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(Y);
  float* wsf = reinterpret_cast<float*>(ws);
  ArArgs ar;
  memset(&ar, 0, sizeof(ar));
  switch (p.tn) {
    case 16: return gemm_launch<16>(tmW, tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream);
    case 32: return gemm_launch<32>(tmW, tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream);
    case 64: return gemm_launch<64>(tmW, tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream);
    case 128: return gemm_launch<128>(tmW, tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream);
    default: return gemm_launch<256>(tmW, tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream);
  }
}

// Y[T, N] = X[T, K] (bf16) · dequant(Wq)[N, K]^T for packed weights (qtype as in quant_blocks.cuh, or
// 9 = block-scaled fp8 with `scales` [N, scale_ld]).  The blocks are decoded inside the GEMM by its
// producer warps; nothing is dequantized to global memory.  K must be a multiple of 64.
OXB_API int oxb_gemm_quant(const void* X, const void* Wq, int qtype, size_t row_bytes, const float* scales, int scale_ld,
                           void* Y, const float* bias, int T, int N, int K, int ldY, int epi_mode, int splits_hint,
                           void* ws, size_t ws_bytes, int* counters, int n_counters, cudaStream_t stream) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 64 != 0) return (int)cudaErrorInvalidValue;
  GemmPlan p = gemm_plan(T, N, K, splits_hint, sm_count());
  while (p.splits > 1 && !p.cluster && (p.ws_bytes > ws_bytes || p.n_counters > n_counters || ws == nullptr || counters == nullptr ||
                          p.n_tiles * p.t_tiles * p.splits > sm_count()))
    p = gemm_plan(T, N, K, p.splits - 1, sm_count());
  CUtensorMap tmX;
  int e = oxb_make_tmap_2d(&tmX, X, T, K, (uint64_t)K * 2, p.tn, GEMM_BK, 2);
  if (e) return e;
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(Y);
  float* wsf = reinterpret_cast<float*>(ws);
  ArArgs ar;
  memset(&ar, 0, sizeof(ar));
  QwArgs qw{reinterpret_cast<const uint8_t*>(Wq), row_bytes, scales, scale_ld, 0};
  switch (qtype) {
    case QT_Q4_K:
    case QT_Q6_K: {
      // staged path (packed super-blocks by TMA) when the byte map can be built: 16-byte rows and base
      CUtensorMap tmWq;
      const int box = qtype == QT_Q4_K ? MmqStage<QT_Q4_K>::BOX : MmqStage<QT_Q6_K>::BOX;
      if (p.tn <= 64 && oxb_make_tmap_bytes(&tmWq, Wq, (uint64_t)N, row_bytes, GEMM_BM, box) == 0) qw.staged = 1;
      const GroupArgs g0{0, 0, 0, 0, nullptr, 0, 0};
      if (qtype == QT_Q4_K)
        return gemm_launch_mmq<QT_Q4_K>(tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream, qw, g0, 1,
                                        qw.staged ? &tmWq : nullptr);
      return gemm_launch_mmq<QT_Q6_K>(tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream, qw, g0, 1,
                                      qw.staged ? &tmWq : nullptr);
    }
    case QT_Q8_0: return gemm_launch_mmq<QT_Q8_0>(tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream, qw);
    case QT_Q4_0: return gemm_launch_mmq<QT_Q4_0>(tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream, qw);
    case QT_NVFP4: return gemm_launch_mmq<QT_NVFP4>(tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream, qw);
    case QT_FP8B:
      if (scales == nullptr) return (int)cudaErrorInvalidValue;
      return gemm_launch_mmq<QT_FP8B>(tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream, qw);
    default: return (int)cudaErrorInvalidValue;
  }
}

static int fill_ar(ArArgs& ar, int world, int rank, const uint64_t* data_ptrs, const uint64_t* flag_ptrs, int* ctrl,
                   int t_max, int n_max, int max_tiles, unsigned long long timeout_ns, const void* residual) {
  memset(&ar, 0, sizeof(ar));
  ar.mode = world >= g_oxb_ar_ll_min_world ? 1 : 0;
  ar.trace = g_oxb_ar_trace;
  if (world < 1 || world > AR_MAX_WORLD || rank < 0 || rank >= world || ctrl == nullptr) return (int)cudaErrorInvalidValue;
  ar.world = world;
  ar.rank = rank;
  ar.t_max = t_max;
  ar.n_max = n_max;
  ar.max_tiles = max_tiles;
  ar.timeout_ns = timeout_ns;
  ar.ctrl = ctrl;
  ar.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  for (int i = 0; i < world; ++i) {
    ar.data[i] = reinterpret_cast<__nv_bfloat16*>(data_ptrs[i]);
    ar.flags[i] = reinterpret_cast<uint32_t*>(flag_ptrs[i]);
  }
  return 0;
}

// Row-parallel GEMM fused with a one-shot all-reduce over peer memory:
//   Y[T, N] = sum over ranks of X_r[T, K_r] · W_r[N, K_r]^T  (+ residual), identical on every rank.
// data_ptrs / flag_ptrs: every rank's symmetric receive buffer [2][world+1][t_max][n_max] bf16 and flag
// array [2][world+1][max_tiles] u32 (zeroed once); ctrl: 2 local ints, zeroed once.
// Limits: T <= min(t_max, 256), N <= n_max, N % 8 == 0, N/128 <= max_tiles, and the whole grid must be
// co-resident (<= SM count) because CTAs wait on their peers' copies of the same tile.
OXB_API int oxb_gemm_ar(const void* X, const void* W, void* Y, const void* residual, int T, int N, int K, int ldY,
                        int world, int rank, const uint64_t* data_ptrs, const uint64_t* flag_ptrs, int* ctrl, int t_max,
                        int n_max, int max_tiles, unsigned long long timeout_ns, void* ws, size_t ws_bytes, int* counters,
                        int n_counters, cudaStream_t stream) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  const int ll = world >= g_oxb_ar_ll_min_world;
  if (K % 8 != 0 || N % 8 != 0 || (T > 256 && !ll) || T > t_max || N > n_max) return (int)cudaErrorInvalidValue;
  GemmPlan p;
  if (T <= 256) {
    // CTAs wait for the CTAs with the same piece index on the other GPUs, so the whole grid is kept
    // resident at once on every rank: bound tiles*splits by what the SMs can hold.
    int resident = sm_count() * (T <= 64 ? GemmTile<64>::CTAS_PER_SM : 1);
    if (!ll && resident > max_tiles) resident = max_tiles;  // the one-shot exchange has one flag per piece
    p = gemm_plan(T, N, K, 0, sm_count(), -1, resident);
    while (p.splits > 1 && !p.cluster && (p.ws_bytes > ws_bytes || p.n_counters > n_counters || ws == nullptr ||
                                          counters == nullptr || p.n_tiles * p.splits > sm_count()))
      p = gemm_plan(T, N, K, p.splits - 1, sm_count(), -1, resident);
    if (p.n_tiles * p.splits > resident || p.t_tiles != 1) return (int)cudaErrorInvalidConfiguration;
  } else {
    // Prefill-sized calls (LL exchange only): several waves of 256-token tiles, no split-K.  A tile's
    // exchange overlaps the MMAs of the tiles behind it.  Progress relies on both ranks dispatching
    // CTAs in block-index order, so that the lowest unfinished piece is resident everywhere; the
    // bounded polls turn a violation into an error status, not a hang.
    p = gemm_plan(T, N, K, 1, sm_count(), 0);
  }
  ArArgs ar;
  int e = fill_ar(ar, world, rank, data_ptrs, flag_ptrs, ctrl, t_max, n_max, max_tiles, timeout_ns, residual);
  if (e) return e;
  CUtensorMap tmW, tmX;
  e = oxb_make_tmap_2d(&tmW, W, N, K, (uint64_t)K * 2, GEMM_BM, GEMM_BK, 2);
  if (e) return e;
  e = oxb_make_tmap_2d(&tmX, X, T, K, (uint64_t)K * 2, p.tn, GEMM_BK, 2);
  if (e) return e;
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(Y);
  float* wsf = reinterpret_cast<float*>(ws);
  switch (p.tn) {
    case 16: return gemm_launch<16>(tmW, tmX, y, nullptr, N, T, K, ldY, p, wsf, counters, 0, ar, stream);
    case 32: return gemm_launch<32>(tmW, tmX, y, nullptr, N, T, K, ldY, p, wsf, counters, 0, ar, stream);
    case 64: return gemm_launch<64>(tmW, tmX, y, nullptr, N, T, K, ldY, p, wsf, counters, 0, ar, stream);
    case 128: return gemm_launch<128>(tmW, tmX, y, nullptr, N, T, K, ldY, p, wsf, counters, 0, ar, stream);
    default: return gemm_launch<256>(tmW, tmX, y, nullptr, N, T, K, ldY, p, wsf, counters, 0, ar, stream);
  }
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

OXB_API int oxb_dequant_rows(const void* src, int qtype, size_t row_bytes, int rows, int cols, void* dst_bf16,
                             cudaStream_t stream) {
  if (rows <= 0) return 0;
  dequant_rows_kernel<<<rows, 256, 0, stream>>>(reinterpret_cast<const uint8_t*>(src), qtype, row_bytes, cols,
                                                reinterpret_cast<__nv_bfloat16*>(dst_bf16));
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

OXB_API int oxb_silu_mul(const void* gu, void* out, int T, int I, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (I % 8 != 0) return (int)cudaErrorInvalidValue;
  const size_t total = (size_t)T * (I / 8);
  int blocks = (int)((total + 255) / 256);
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  oxb_launch(silu_mul_kernel, dim3(blocks), dim3(256), 0, stream, reinterpret_cast<const __nv_bfloat16*>(gu),
             reinterpret_cast<__nv_bfloat16*>(out), T, I);
  OXB_CHECK_LAUNCH();
  return 0;
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

// Fused qkv projection: qkv = X · Wqkv^T with RoPE + KV write as the GEMM's epilogue (EPI_ROPE).  Wqkv rows
// are [nq heads | nkv key heads | nkv value heads] of head_dim 128; bf16 KV pages only; full rotary (rot == 128).
OXB_API int oxb_gemm_qkv_rope(const void* X, const void* W, int T, int K, const int* positions, const int* slots,
                              const float* cos_sin, int max_pos, int rot, int pairing, int nq, int nkv, void* q_out,
                              void* kv_data, int page, int num_blocks, cudaStream_t stream) {
  if (T <= 0) return 0;
  const int N = (nq + 2 * nkv) * 128;
  if (K % 8 != 0 || rot != 128 || page <= 0 || (reinterpret_cast<uintptr_t>(q_out) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(kv_data) & 15) != 0)
    return (int)cudaErrorInvalidValue;
  GemmPlan p = gemm_plan(T, N, K, 0, sm_count(), 1);
  CUtensorMap tmW, tmX;
  int e = oxb_make_tmap_2d(&tmW, W, N, K, (uint64_t)K * 2, GEMM_BM, GEMM_BK, 2);
  if (e) return e;
  e = oxb_make_tmap_2d(&tmX, X, T, K, (uint64_t)K * 2, p.tn, GEMM_BK, 2);
  if (e) return e;
  ArArgs ar;
  memset(&ar, 0, sizeof(ar));
  RopeArgs ro{positions, slots, cos_sin, max_pos, rot, pairing, nq, nkv, page, num_blocks, reinterpret_cast<__nv_bfloat16*>(q_out),
              reinterpret_cast<__nv_bfloat16*>(kv_data)};
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(q_out);  // only its alignment is looked at
  const QwArgs qw{nullptr, 0, nullptr, 0, 0};
  const GroupArgs gr{0, 0, 0, 0, nullptr, 0, 0};
  switch (p.tn) {
    case 16: return gemm_launch<16>(tmW, tmX, y, nullptr, N, T, K, N, p, nullptr, nullptr, EPI_ROPE, ar, stream, qw, gr, 1, ro);
    case 32: return gemm_launch<32>(tmW, tmX, y, nullptr, N, T, K, N, p, nullptr, nullptr, EPI_ROPE, ar, stream, qw, gr, 1, ro);
    case 64: return gemm_launch<64>(tmW, tmX, y, nullptr, N, T, K, N, p, nullptr, nullptr, EPI_ROPE, ar, stream, qw, gr, 1, ro);
    case 128: return gemm_launch<128>(tmW, tmX, y, nullptr, N, T, K, N, p, nullptr, nullptr, EPI_ROPE, ar, stream, qw, gr, 1, ro);
    default: return gemm_launch<256>(tmW, tmX, y, nullptr, N, T, K, N, p, nullptr, nullptr, EPI_ROPE, ar, stream, qw, gr, 1, ro);
  }
}

OXB_API int oxb_argmax(const float* logits, int R, int V, int ld, int tie_highest, int* out, float* out_val,
                       int index_offset, cudaStream_t stream) {
  if (R <= 0) return 0;
  oxb_launch(argmax_kernel, dim3(R), dim3(1024), 0, stream, logits, V, ld, tie_highest, out, out_val, index_offset);
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
  // (Merging the KV splits of a row tile inside a thread-block cluster was measured and is slower here:
  // every CTA then waits for the slowest split, 21.7 vs 19.0 us on 64 x 1400-token decode.  The splits
  // stay independent CTAs; the last one to finish merges.)
  if (a.n_cta_splits > 1 && (a.ws_o == nullptr || a.ws_ml == nullptr || a.counters == nullptr)) return (int)cudaErrorInvalidValue;
  oxb_launch(paged_attention_kernel<HD>, grid, dim3(ATT_WARPS * 32), (size_t)smem, stream, a, G);
  OXB_CHECK_LAUNCH();
  return 0;
}

OXB_API int oxb_paged_attention(const void* q, void* out, const void* kv_data, const float* kv_scales,
                                const int* block_tables, const int* seq_lens, const int* query_start, int B,
                                int max_blocks, int nq, int nkv, int hd, int kv_mode, int max_query_len,
                                int n_cta_splits, int window, float scale, float* ws_o, float* ws_ml, int* counters,
                                int num_blocks, cudaStream_t stream) {
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
  a.ws_o = ws_o;
  a.ws_ml = ws_ml;
  a.counters = counters;
  a.num_blocks = num_blocks;
  a.trace = g_oxb_attn_trace;
  if (hd == 128) return attn_launch<128>(a, B, G, stream);
  if (hd == 64) return attn_launch<64>(a, B, G, stream);
  return (int)cudaErrorInvalidValue;
}

// ----------------------------------------------------------------------------- allocation-free GEMM
// See oxb_noalloc.h for the contract.  The split-K scratch of the GEMM lives in this fixed device
// array: [0, 16 KiB) rendezvous counters, the rest fp32 partials.
#include "oxb_noalloc.h"
#include <stdio.h>

static __device__ __align__(256) unsigned char g_noalloc_scratch[OXB_NOALLOC_SCRATCH_BYTES];

// In host code `g_noalloc_scratch` is only a handle for the runtime, not a device address, so the
// address is looked up once per device and cached here.
static void* g_noalloc_dev_ptr[64] = {nullptr};

extern "C" __attribute__((visibility("default"))) int oxb_gemm_bf16_noalloc(
    const void* X, const void* W, void* Y, const float* bias, int T, int N, int K, int ldY, void* cuda_stream) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
  if (X == nullptr || W == nullptr || Y == nullptr || T <= 0 || N <= 0 || K <= 0 || K % 8 != 0 || ldY < N)
    return OXB_NOALLOC_E_BAD_ARGUMENT;
  if (T > OXB_NOALLOC_MAX_TOKENS) {
    fprintf(stderr, "oxb_gemm_bf16_noalloc: T=%d exceeds the limit of %d tokens per call (static scratch of %d bytes)\n",
            T, OXB_NOALLOC_MAX_TOKENS, (int)OXB_NOALLOC_SCRATCH_BYTES);
    return OXB_NOALLOC_E_TOO_LARGE;
  }
  int dev = 0;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess) return (int)ce;
  if (dev < 0 || dev >= 64) return OXB_NOALLOC_E_BAD_ARGUMENT;
  if (g_noalloc_dev_ptr[dev] == nullptr) {
    void* p = nullptr;
    ce = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (ce != cudaSuccess) return (int)ce;
    g_noalloc_dev_ptr[dev] = p;
  }
  unsigned char* base = reinterpret_cast<unsigned char*>(g_noalloc_dev_ptr[dev]);
  int* counters = reinterpret_cast<int*>(base);
  float* ws = reinterpret_cast<float*>(base + OXB_NOALLOC_COUNTER_BYTES);
  const size_t ws_bytes = OXB_NOALLOC_SCRATCH_BYTES - OXB_NOALLOC_COUNTER_BYTES;
  const int n_counters = OXB_NOALLOC_COUNTER_BYTES / (int)sizeof(int);
  GemmPlan p = gemm_plan(T, N, K, 0, sm_count(), 0);  // always the global-scratch split-K: that is what this entry is for
  while (p.splits > 1 && (p.ws_bytes > ws_bytes || p.n_counters > n_counters || p.n_tiles * p.t_tiles * p.splits > sm_count()))
    p = gemm_plan(T, N, K, p.splits - 1, sm_count(), 0);
  if (p.splits > 1) {
    // the counters must start at zero; an earlier call that gave up could have left them set
    ce = cudaMemsetAsync(counters, 0, (size_t)p.n_counters * sizeof(int), stream);
    if (ce != cudaSuccess) return (int)ce;
  }
  CUtensorMap tmW, tmX;
  int e = oxb_make_tmap_2d(&tmW, W, N, K, (uint64_t)K * 2, GEMM_BM, GEMM_BK, 2);
  if (e) return e;
  e = oxb_make_tmap_2d(&tmX, X, T, K, (uint64_t)K * 2, p.tn, GEMM_BK, 2);
  if (e) return e;
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(Y);
  ArArgs ar;
  memset(&ar, 0, sizeof(ar));
  switch (p.tn) {
    case 16: return gemm_launch<16>(tmW, tmX, y, bias, N, T, K, ldY, p, ws, counters, 0, ar, stream);
    case 32: return gemm_launch<32>(tmW, tmX, y, bias, N, T, K, ldY, p, ws, counters, 0, ar, stream);
    case 64: return gemm_launch<64>(tmW, tmX, y, bias, N, T, K, ldY, p, ws, counters, 0, ar, stream);
    case 128: return gemm_launch<128>(tmW, tmX, y, bias, N, T, K, ldY, p, ws, counters, 0, ar, stream);
    default: return gemm_launch<256>(tmW, tmX, y, bias, N, T, K, ldY, p, ws, counters, 0, ar, stream);
  }
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

// Grouped GEMM over `groups` experts in ONE launch: for group g,
//   Y[g] [T, N] = X_g [T, K] · W_g [N, K]^T,   W stacked as [(groups*N), K] (bf16 or packed rows),
//   X_g = X + g*x_rows rows (x_rows = 0: every group reads the same X),  Y[g] = Y + g*y_stride elements.
// Groups whose `scale` row (per-token routing weights, [groups, scale_ld]) is all zero are skipped on the
// device.  T <= 256.
OXB_API int oxb_gemm_grouped(const void* X, int x_rows, const void* W, int qtype, size_t row_bytes, void* Y,
                             long long y_stride, const float* scale, int scale_ld, int groups, int T, int N, int K,
                             int ldY, void* ws, size_t ws_bytes, int* counters, int n_counters, cudaStream_t stream) {
  if (T <= 0 || N <= 0 || K <= 0 || groups <= 0) return 0;
  if (T > 256 || K % 64 != 0) return (int)cudaErrorInvalidValue;
  GemmPlan p = gemm_plan(T, N, K, 0, sm_count());
  while (p.splits > 1 && !p.cluster && (p.ws_bytes * groups > ws_bytes || p.n_counters * groups > n_counters || ws == nullptr ||
                          counters == nullptr || p.n_tiles * p.splits * groups > sm_count()))
    p = gemm_plan(T, N, K, p.splits - 1, sm_count());
  CUtensorMap tmW, tmX;
  const uint64_t xr = x_rows > 0 ? (uint64_t)groups * x_rows : (uint64_t)T;
  int e = oxb_make_tmap_2d(&tmX, X, xr, K, (uint64_t)K * 2, p.tn, GEMM_BK, 2);
  if (e) return e;
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(Y);
  float* wsf = reinterpret_cast<float*>(ws);
  ArArgs ar;
  memset(&ar, 0, sizeof(ar));
  GroupArgs gr{1, N, x_rows, y_stride, scale, scale_ld, 0};
  QwArgs qw{reinterpret_cast<const uint8_t*>(W), row_bytes, nullptr, 0, 0};
  if (qtype == QT_BF16) {
    e = oxb_make_tmap_2d(&tmW, W, (uint64_t)groups * N, K, (uint64_t)K * 2, GEMM_BM, GEMM_BK, 2);
    if (e) return e;
    switch (p.tn) {
      case 16: return gemm_launch<16>(tmW, tmX, y, nullptr, N, T, K, ldY, p, wsf, counters, 0, ar, stream, qw, gr, groups);
      case 32: return gemm_launch<32>(tmW, tmX, y, nullptr, N, T, K, ldY, p, wsf, counters, 0, ar, stream, qw, gr, groups);
      case 64: return gemm_launch<64>(tmW, tmX, y, nullptr, N, T, K, ldY, p, wsf, counters, 0, ar, stream, qw, gr, groups);
      case 128: return gemm_launch<128>(tmW, tmX, y, nullptr, N, T, K, ldY, p, wsf, counters, 0, ar, stream, qw, gr, groups);
      default: return gemm_launch<256>(tmW, tmX, y, nullptr, N, T, K, ldY, p, wsf, counters, 0, ar, stream, qw, gr, groups);
    }
  }
  switch (qtype) {
    case QT_Q4_K:
    case QT_Q6_K: {
      CUtensorMap tmWq;
      const int box = qtype == QT_Q4_K ? MmqStage<QT_Q4_K>::BOX : MmqStage<QT_Q6_K>::BOX;
      if (p.tn <= 64 && oxb_make_tmap_bytes(&tmWq, W, (uint64_t)groups * N, row_bytes, GEMM_BM, box) == 0) qw.staged = 1;
      if (qtype == QT_Q4_K)
        return gemm_launch_mmq<QT_Q4_K>(tmX, y, nullptr, N, T, K, ldY, p, wsf, counters, 0, ar, stream, qw, gr, groups,
                                        qw.staged ? &tmWq : nullptr);
      return gemm_launch_mmq<QT_Q6_K>(tmX, y, nullptr, N, T, K, ldY, p, wsf, counters, 0, ar, stream, qw, gr, groups,
                                      qw.staged ? &tmWq : nullptr);
    }
    case QT_Q8_0: return gemm_launch_mmq<QT_Q8_0>(tmX, y, nullptr, N, T, K, ldY, p, wsf, counters, 0, ar, stream, qw, gr, groups);
    case QT_Q4_0: return gemm_launch_mmq<QT_Q4_0>(tmX, y, nullptr, N, T, K, ldY, p, wsf, counters, 0, ar, stream, qw, gr, groups);
    case QT_NVFP4: return gemm_launch_mmq<QT_NVFP4>(tmX, y, nullptr, N, T, K, ldY, p, wsf, counters, 0, ar, stream, qw, gr, groups);
    default: return (int)cudaErrorInvalidValue;
  }
}
