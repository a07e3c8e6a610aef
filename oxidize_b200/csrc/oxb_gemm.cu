// liboxb, GEMM entry points: bf16 tcgen05 GEMM, packed-weight dispatch, fused GEMM + all-reduce, fused qkv + RoPE,
// grouped (per-expert) GEMM and the allocation-free variant.
#include "common.cuh"
#include "quant_blocks.cuh"
#include "gemm_tcgen05.cuh"
#include "gemv_quant.cuh"
#include "mmq_dispatch.h"
using namespace oxb;
static int sm_count() { return oxb_sm_count(); }

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
static int gemm_bf16_impl(const void* X, const void* W, void* Y, const float* bias, int T, int N, int K, int ldY,
                          int epi_mode, int splits_hint, void* ws, size_t ws_bytes, int* counters, int n_counters,
                          cudaStream_t stream, const NormArgs& nm) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  // the per-row sums of squares come out of the vector-store epilogues only
  const bool swiglu = epi_mode == EPI_SWIGLU || epi_mode == EPI_GEGLU;  // gated-activation epilogues: SiLU or tanh-GELU on the gate
  if (nm.sumsq_out != nullptr && (N % 8 != 0 || ldY % 8 != 0 || (reinterpret_cast<uintptr_t>(Y) & 15) != 0 || swiglu))
    return (int)cudaErrorInvalidValue;
  if (K % 8 != 0) return (int)cudaErrorInvalidValue;  // TMA rows must be 16-byte multiples
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
  const QwArgs qw{nullptr, 0, nullptr, 0, 0};
  const GroupArgs gr{0, 0, 0, 0, nullptr, 0, 0, nullptr, 1};
  const RopeArgs ro{nullptr, nullptr, nullptr, 0, 0, 0, 0, 0, 0, 0, nullptr, nullptr};
  switch (p.tn) {
    case 16: return gemm_launch<16>(tmW, tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream, qw, gr, 1, ro, nm);
    case 32: return gemm_launch<32>(tmW, tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream, qw, gr, 1, ro, nm);
    case 64: return gemm_launch<64>(tmW, tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream, qw, gr, 1, ro, nm);
    case 128: return gemm_launch<128>(tmW, tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream, qw, gr, 1, ro, nm);
    default: return gemm_launch<256>(tmW, tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream, qw, gr, 1, ro, nm);
  }
}

static NormArgs make_norm(const void* sumsq_in, int norm_dim, float eps, void* clear, void* sumsq_out) {
  NormArgs nm{reinterpret_cast<const unsigned long long*>(sumsq_in), norm_dim > 0 ? 1.f / (float)norm_dim : 0.f, eps,
              reinterpret_cast<unsigned long long*>(clear), reinterpret_cast<unsigned long long*>(sumsq_out)};
  return nm;
}
static NormArgs no_norm() { return make_norm(nullptr, 0, 0.f, nullptr, nullptr); }

OXB_API int oxb_gemm_bf16(const void* X, const void* W, void* Y, const float* bias, int T, int N, int K, int ldY,
                          int epi_mode, int splits_hint, void* ws, size_t ws_bytes, int* counters, int n_counters,
                          cudaStream_t stream) {
  return gemm_bf16_impl(X, W, Y, bias, T, N, K, ldY, epi_mode, splits_hint, ws, ws_bytes, counters, n_counters, stream,
                        no_norm());
}

// The same GEMM as one half of a folded RMSNorm (see NormArgs in gemm_tcgen05.cuh); the accumulators are [>= T] u64:
//  * sumsq_in  != null: X holds un-normalised rows; the accumulator of token t is multiplied by
//    rsqrt(sumsq_in[t] * 2^-28 / norm_dim + eps) (the norm weight is already inside W's columns);
//    `clear` (optional) is reset to zero for the producer that follows;
//  * sumsq_out != null: the epilogue (store or accumulate-into) adds the sum of squares of the values written for
//    token t to sumsq_out[t] (which its previous consumer left at zero).
OXB_API int oxb_gemm_bf16_norm(const void* X, const void* W, void* Y, const float* bias, int T, int N, int K, int ldY,
                               int epi_mode, int splits_hint, void* ws, size_t ws_bytes, int* counters, int n_counters,
                               const void* sumsq_in, int norm_dim, float eps, void* clear, void* sumsq_out,
                               cudaStream_t stream) {
  if (sumsq_in != nullptr && norm_dim <= 0) return (int)cudaErrorInvalidValue;
  return gemm_bf16_impl(X, W, Y, bias, T, N, K, ldY, epi_mode, splits_hint, ws, ws_bytes, counters, n_counters, stream,
                        make_norm(sumsq_in, norm_dim, eps, clear, sumsq_out));
}

// Launch the packed-weight GEMM of the given format.  The packed rows are read through a TMA byte map (rows and base
// must be 16-byte multiples and K a multiple of 256; otherwise the producers read global memory themselves).
static int launch_mmq(int qtype, const void* W, uint64_t w_rows, const CUtensorMap& tmX, __nv_bfloat16* y, const float* bias,
                      int N, int T, int K, int ldY, const GemmPlan& p, float* wsf, int* counters, int epi_mode, const ArArgs& ar,
                      cudaStream_t stream, QwArgs qw, const GroupArgs& gr, int groups) {
  CUtensorMap tmWq;
  if (K % 256 == 0 &&
      oxb_make_tmap_bytes(&tmWq, W, w_rows, qw.row_bytes, GEMM_BM, (uint32_t)mmq_box_bytes(qtype)) == 0)
    qw.staged = 1;
  const CUtensorMap* tw = qw.staged ? &tmWq : nullptr;
  switch (qtype) {
    case QT_Q4_K: return gemm_mmq_q4_k(tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream, qw, gr, groups, tw);
    case QT_Q6_K: return gemm_mmq_q6_k(tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream, qw, gr, groups, tw);
    case QT_Q8_0: return gemm_mmq_q8_0(tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream, qw, gr, groups, tw);
    case QT_Q4_0: return gemm_mmq_q4_0(tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream, qw, gr, groups, tw);
    case QT_NVFP4: return gemm_mmq_nvfp4(tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream, qw, gr, groups, tw);
    case QT_FP8B:
      if (qw.scales == nullptr) return (int)cudaErrorInvalidValue;
      return gemm_mmq_fp8b(tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream, qw, gr, groups, tw);
    default: return (int)cudaErrorInvalidValue;
  }
}


// Y[T, N] = X[T, K] (bf16) · dequant(Wq)[N, K]^T for packed weights (qtype as in quant_blocks.cuh, or
// 9 = block-scaled fp8 with `scales` [N, scale_ld]).  The blocks are decoded inside the GEMM by its
// producer warps; nothing is dequantized to global memory.  K must be a multiple of 64.
OXB_API int oxb_gemm_quant(const void* X, const void* Wq, int qtype, size_t row_bytes, const float* scales, int scale_ld,
                           void* Y, const float* bias, int T, int N, int K, int ldY, int epi_mode, int splits_hint,
                           void* ws, size_t ws_bytes, int* counters, int n_counters, cudaStream_t stream) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  // One or two tokens (g_oxb_gemv_max_t): the packed bytes go straight into dp4a (gemv_quant.cuh), no tensor-core staging.
  // ... unless the matrix is wide and short (ffn_down: few rows, long K): the GEMV's warps then each walk a long row
  // with little parallelism across rows, and the split-K tensor-core kernel is ahead even at one token
  // (4096 x 14336: 23.6 against 25.6 us for Q4_K, 29.9 against 38.2 us for Q6_K).
  const bool wide = !g_oxb_gemv_wide && (long long)K >= 2LL * N && K % 256 == 0;
  if (g_oxb_gemv_max_t > 0 && T <= g_oxb_gemv_max_t && !wide && (epi_mode == EPI_STORE || epi_mode == EPI_ADD_INTO) &&
      gemv_quant_supported(qtype, T, K, row_bytes, Wq, X, K))
    return gemv_quant_run(qtype, reinterpret_cast<const uint8_t*>(Wq), row_bytes, reinterpret_cast<const __nv_bfloat16*>(X), K,
                      reinterpret_cast<__nv_bfloat16*>(Y), ldY, bias, T, N, K, epi_mode == EPI_ADD_INTO, sm_count(), stream);
  if (K % 64 != 0) return (int)cudaErrorInvalidValue;
  GemmPlan p = gemm_plan(T, N, K, splits_hint, sm_count(), -1, 0, true);
  while (p.splits > 1 && !p.cluster && (p.ws_bytes > ws_bytes || p.n_counters > n_counters || ws == nullptr || counters == nullptr ||
                          p.n_tiles * p.t_tiles * p.splits > sm_count()))
    p = gemm_plan(T, N, K, p.splits - 1, sm_count(), -1, 0, true);
  CUtensorMap tmX;
  int e = oxb_make_tmap_2d(&tmX, X, T, K, (uint64_t)K * 2, p.tn, GEMM_BK, 2);
  if (e) return e;
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(Y);
  float* wsf = reinterpret_cast<float*>(ws);
  ArArgs ar;
  memset(&ar, 0, sizeof(ar));
  QwArgs qw{reinterpret_cast<const uint8_t*>(Wq), row_bytes, scales, scale_ld, 0};
  const GroupArgs g0{0, 0, 0, 0, nullptr, 0, 0, nullptr, 1};
  return launch_mmq(qtype, Wq, (uint64_t)N, tmX, y, bias, N, T, K, ldY, p, wsf, counters, epi_mode, ar, stream, qw, g0, 1);
}

// Row-parallel GEMM fused with a one-shot all-reduce over peer memory:
//   Y[T, N] = sum over ranks of X_r[T, K_r] · W_r[N, K_r]^T  (+ residual), identical on every rank.
// data_ptrs / flag_ptrs: every rank's symmetric receive buffer [2][world+1][t_max][n_max] bf16 and flag
// array [2][world+1][max_tiles] u32 (zeroed once); ctrl: 2 local ints, zeroed once.
// Limits: T <= min(t_max, 256), N <= n_max, N % 8 == 0, N/128 <= max_tiles, and the whole grid must be
// co-resident (<= SM count) because CTAs wait on their peers' copies of the same tile.
static int gemm_ar_impl(const void* X, const void* W, void* Y, const void* residual, int T, int N, int K, int ldY,
                        int world, int rank, const uint64_t* data_ptrs, const uint64_t* flag_ptrs, int* ctrl, int t_max,
                        int n_max, int max_tiles, unsigned long long timeout_ns, void* ws, size_t ws_bytes, int* counters,
                        int n_counters, cudaStream_t stream, const NormArgs& nm) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  const int ll = world >= g_oxb_ar_ll_min_world;
  if (nm.sumsq_out != nullptr && (!ll || ldY % 8 != 0)) return (int)cudaErrorInvalidValue;
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
  const QwArgs qw0{nullptr, 0, nullptr, 0, 0};
  const GroupArgs gr0{0, 0, 0, 0, nullptr, 0, 0, nullptr, 1};
  const RopeArgs ro0{nullptr, nullptr, nullptr, 0, 0, 0, 0, 0, 0, 0, nullptr, nullptr};
  switch (p.tn) {
    case 16: return gemm_launch<16>(tmW, tmX, y, nullptr, N, T, K, ldY, p, wsf, counters, 0, ar, stream, qw0, gr0, 1, ro0, nm);
    case 32: return gemm_launch<32>(tmW, tmX, y, nullptr, N, T, K, ldY, p, wsf, counters, 0, ar, stream, qw0, gr0, 1, ro0, nm);
    case 64: return gemm_launch<64>(tmW, tmX, y, nullptr, N, T, K, ldY, p, wsf, counters, 0, ar, stream, qw0, gr0, 1, ro0, nm);
    case 128: return gemm_launch<128>(tmW, tmX, y, nullptr, N, T, K, ldY, p, wsf, counters, 0, ar, stream, qw0, gr0, 1, ro0, nm);
    default: return gemm_launch<256>(tmW, tmX, y, nullptr, N, T, K, ldY, p, wsf, counters, 0, ar, stream, qw0, gr0, 1, ro0, nm);
  }
}

OXB_API int oxb_gemm_ar(const void* X, const void* W, void* Y, const void* residual, int T, int N, int K, int ldY,
                        int world, int rank, const uint64_t* data_ptrs, const uint64_t* flag_ptrs, int* ctrl, int t_max,
                        int n_max, int max_tiles, unsigned long long timeout_ns, void* ws, size_t ws_bytes, int* counters,
                        int n_counters, cudaStream_t stream) {
  return gemm_ar_impl(X, W, Y, residual, T, N, K, ldY, world, rank, data_ptrs, flag_ptrs, ctrl, t_max, n_max, max_tiles,
                      timeout_ns, ws, ws_bytes, counters, n_counters, stream, no_norm());
}

// oxb_gemm_ar whose exchange also adds the sum of squares of the values written for token t (after the residual
// add) to sumsq_out[t]: the producer half of a folded RMSNorm.  Two-shot exchange only.
OXB_API int oxb_gemm_ar_norm(const void* X, const void* W, void* Y, const void* residual, int T, int N, int K, int ldY,
                             int world, int rank, const uint64_t* data_ptrs, const uint64_t* flag_ptrs, int* ctrl, int t_max,
                             int n_max, int max_tiles, unsigned long long timeout_ns, void* ws, size_t ws_bytes, int* counters,
                             int n_counters, void* sumsq_out, cudaStream_t stream) {
  if (sumsq_out == nullptr) return (int)cudaErrorInvalidValue;
  return gemm_ar_impl(X, W, Y, residual, T, N, K, ldY, world, rank, data_ptrs, flag_ptrs, ctrl, t_max, n_max, max_tiles,
                      timeout_ns, ws, ws_bytes, counters, n_counters, stream, make_norm(nullptr, 0, 0.f, nullptr, sumsq_out));
}

// Fused qkv projection: qkv = X · Wqkv^T with RoPE + KV write as the GEMM's epilogue (EPI_ROPE).  Wqkv rows
// are [nq heads | nkv key heads | nkv value heads] of head_dim 128; bf16 KV pages only; full rotary (rot == 128).
static int gemm_qkv_rope_impl(const void* X, const void* W, int T, int K, const int* positions, const int* slots,
                              const float* cos_sin, int max_pos, int rot, int pairing, int nq, int nkv, void* q_out,
                              void* kv_data, int page, int num_blocks, cudaStream_t stream, const NormArgs& nm) {
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
  const GroupArgs gr{0, 0, 0, 0, nullptr, 0, 0, nullptr, 1};
  switch (p.tn) {
    case 16: return gemm_launch<16>(tmW, tmX, y, nullptr, N, T, K, N, p, nullptr, nullptr, EPI_ROPE, ar, stream, qw, gr, 1, ro, nm);
    case 32: return gemm_launch<32>(tmW, tmX, y, nullptr, N, T, K, N, p, nullptr, nullptr, EPI_ROPE, ar, stream, qw, gr, 1, ro, nm);
    case 64: return gemm_launch<64>(tmW, tmX, y, nullptr, N, T, K, N, p, nullptr, nullptr, EPI_ROPE, ar, stream, qw, gr, 1, ro, nm);
    case 128: return gemm_launch<128>(tmW, tmX, y, nullptr, N, T, K, N, p, nullptr, nullptr, EPI_ROPE, ar, stream, qw, gr, 1, ro, nm);
    default: return gemm_launch<256>(tmW, tmX, y, nullptr, N, T, K, N, p, nullptr, nullptr, EPI_ROPE, ar, stream, qw, gr, 1, ro, nm);
  }
}

OXB_API int oxb_gemm_qkv_rope(const void* X, const void* W, int T, int K, const int* positions, const int* slots,
                              const float* cos_sin, int max_pos, int rot, int pairing, int nq, int nkv, void* q_out,
                              void* kv_data, int page, int num_blocks, cudaStream_t stream) {
  return gemm_qkv_rope_impl(X, W, T, K, positions, slots, cos_sin, max_pos, rot, pairing, nq, nkv, q_out, kv_data, page,
                            num_blocks, stream, no_norm());
}

// The fused qkv projection as the consumer half of a folded RMSNorm (X un-normalised, per-token scale from sumsq_in).
OXB_API int oxb_gemm_qkv_rope_norm(const void* X, const void* W, int T, int K, const int* positions, const int* slots,
                                   const float* cos_sin, int max_pos, int rot, int pairing, int nq, int nkv, void* q_out,
                                   void* kv_data, int page, int num_blocks, const void* sumsq_in, int norm_dim, float eps,
                                   void* clear, cudaStream_t stream) {
  if (sumsq_in == nullptr || norm_dim <= 0) return (int)cudaErrorInvalidValue;
  return gemm_qkv_rope_impl(X, W, T, K, positions, slots, cos_sin, max_pos, rot, pairing, nq, nkv, q_out, kv_data, page,
                            num_blocks, stream, make_norm(sumsq_in, norm_dim, eps, clear, nullptr));
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

// Grouped GEMM over `groups` experts in ONE launch: for group g,
//   Y[g] [T, N] = X_g [T, K] · W_g [N, K]^T,   W stacked as [(groups*N), K] (bf16 or packed rows),
//   X_g = X + g*x_rows rows (x_rows = 0: every group reads the same X),  Y[g] = Y + g*y_stride elements.
// Groups whose `scale` row (per-token routing weights, [groups, scale_ld]) is all zero are skipped on the
// device.  T <= 256 (bf16 weights) or 128 (packed weights).
OXB_API int oxb_gemm_grouped(const void* X, int x_rows, const void* W, int qtype, size_t row_bytes, void* Y,
                             long long y_stride, const float* scale, int scale_ld, int groups, int T, int N, int K,
                             int ldY, void* ws, size_t ws_bytes, int* counters, int n_counters, cudaStream_t stream) {
  if (T <= 0 || N <= 0 || K <= 0 || groups <= 0) return 0;
  const bool packed = qtype != QT_BF16;
  if (T > (packed ? 128 : 256) || K % 64 != 0) return (int)cudaErrorInvalidValue;  // one token tile per group
  GemmPlan p = gemm_plan(T, N, K, 0, sm_count(), -1, 0, packed, groups);
  while (p.splits > 1 && !p.cluster && (p.ws_bytes * groups > ws_bytes || p.n_counters * groups > n_counters || ws == nullptr ||
                          counters == nullptr || p.n_tiles * p.splits * groups > sm_count()))
    p = gemm_plan(T, N, K, p.splits - 1, sm_count(), -1, 0, packed, groups);
  CUtensorMap tmW, tmX;
  const uint64_t xr = x_rows > 0 ? (uint64_t)groups * x_rows : (uint64_t)T;
  int e = oxb_make_tmap_2d(&tmX, X, xr, K, (uint64_t)K * 2, p.tn, GEMM_BK, 2);
  if (e) return e;
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(Y);
  float* wsf = reinterpret_cast<float*>(ws);
  ArArgs ar;
  memset(&ar, 0, sizeof(ar));
  GroupArgs gr{1, N, x_rows, y_stride, scale, scale_ld, 0, nullptr, 1};
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
  if (qtype == QT_FP8B) return (int)cudaErrorInvalidValue;
  return launch_mmq(qtype, W, (uint64_t)groups * N, tmX, y, nullptr, N, T, K, ldY, p, wsf, counters, 0, ar, stream, qw, gr, groups);
}


// Grouped GEMM over token-gathered groups (mixture-of-experts dispatch): group g multiplies the activation rows
// [row_offsets[g], row_offsets[g+1]) of X ([rows_cap, K], gathered expert by expert) with its own weights
// W_g ([N, K] at rows g*N of the stacked matrix) and writes the same rows of Y ([rows_cap, ldY]).  row_offsets is a
// device array of groups + 1 ints written by the upstream kernel; max_rows bounds the rows of any one group (it sizes
// the token tile and the grid; CTAs past a group's rows leave at once).
OXB_API int oxb_gemm_grouped_rows(const void* X, int rows_cap, const void* W, int qtype, size_t row_bytes, void* Y,
                                  const int* row_offsets, int groups, int max_rows, int N, int K, int ldY,
                                  cudaStream_t stream) {
  if (rows_cap <= 0 || max_rows <= 0 || N <= 0 || K <= 0 || groups <= 0) return 0;
  if (K % 64 != 0 || row_offsets == nullptr) return (int)cudaErrorInvalidValue;
  const bool packed = qtype != QT_BF16;
  GemmPlan p = gemm_plan(max_rows, N, K, 0, sm_count(), 1, 0, packed, groups);
  if (p.splits > 1 && !p.cluster) p = gemm_plan(max_rows, N, K, 1, sm_count(), 1, 0, packed, groups);
  CUtensorMap tmW, tmX;
  int e = oxb_make_tmap_2d(&tmX, X, (uint64_t)rows_cap, K, (uint64_t)K * 2, p.tn, GEMM_BK, 2);
  if (e) return e;
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(Y);
  ArArgs ar;
  memset(&ar, 0, sizeof(ar));
  GroupArgs gr{1, N, 0, 0, nullptr, 0, 0, row_offsets, p.t_tiles};
  QwArgs qw{reinterpret_cast<const uint8_t*>(W), row_bytes, nullptr, 0, 0};
  if (qtype == QT_BF16) {
    e = oxb_make_tmap_2d(&tmW, W, (uint64_t)groups * N, K, (uint64_t)K * 2, GEMM_BM, GEMM_BK, 2);
    if (e) return e;
    switch (p.tn) {
      case 16: return gemm_launch<16>(tmW, tmX, y, nullptr, N, max_rows, K, ldY, p, nullptr, nullptr, 0, ar, stream, qw, gr, groups);
      case 32: return gemm_launch<32>(tmW, tmX, y, nullptr, N, max_rows, K, ldY, p, nullptr, nullptr, 0, ar, stream, qw, gr, groups);
      case 64: return gemm_launch<64>(tmW, tmX, y, nullptr, N, max_rows, K, ldY, p, nullptr, nullptr, 0, ar, stream, qw, gr, groups);
      case 128: return gemm_launch<128>(tmW, tmX, y, nullptr, N, max_rows, K, ldY, p, nullptr, nullptr, 0, ar, stream, qw, gr, groups);
      default: return gemm_launch<256>(tmW, tmX, y, nullptr, N, max_rows, K, ldY, p, nullptr, nullptr, 0, ar, stream, qw, gr, groups);
    }
  }
  if (qtype == QT_FP8B) return (int)cudaErrorInvalidValue;
  return launch_mmq(qtype, W, (uint64_t)groups * N, tmX, y, nullptr, N, max_rows, K, ldY, p, nullptr, nullptr, 0, ar, stream, qw, gr,
                    groups);
}
