// Packed-weight GEMM launchers, one per block format; each is defined in its own translation unit
// (oxb_mmq_<format>.cu) so that the formats compile in parallel.
#pragma once
#include "gemm_tcgen05.cuh"

namespace oxb {

#define OXB_MMQ_ARGS                                                                                                          \
  const CUtensorMap &tmX, __nv_bfloat16 *Y, const float *bias, int N, int T, int K, int ldY, const GemmPlan &p, float *ws,       \
      int *counters, int epi_mode, const ArArgs &ar, cudaStream_t stream, const QwArgs &qw, const GroupArgs &gr, int groups,    \
      const CUtensorMap *tmWq

#define OXB_MMQ_ARGS_DEFAULTED                                                                                                \
  const CUtensorMap &tmX, __nv_bfloat16 *Y, const float *bias, int N, int T, int K, int ldY, const GemmPlan &p, float *ws,       \
      int *counters, int epi_mode, const ArArgs &ar, cudaStream_t stream, const QwArgs &qw,                                     \
      const GroupArgs &gr = GroupArgs{0, 0, 0, 0, nullptr, 0, 0, nullptr, 1}, int groups = 1, const CUtensorMap *tmWq = nullptr

int gemm_mmq_q4_k(OXB_MMQ_ARGS_DEFAULTED);
int gemm_mmq_q6_k(OXB_MMQ_ARGS_DEFAULTED);
int gemm_mmq_q8_0(OXB_MMQ_ARGS_DEFAULTED);
int gemm_mmq_q4_0(OXB_MMQ_ARGS_DEFAULTED);
int gemm_mmq_nvfp4(OXB_MMQ_ARGS_DEFAULTED);
int gemm_mmq_fp8b(OXB_MMQ_ARGS_DEFAULTED);

// dp4a GEMV for decode batches of up to 8 tokens (gemv_quant.cuh; defined in oxb_gemv.cu)
int gemv_quant_run(int qtype, const uint8_t* W, size_t row_bytes, const __nv_bfloat16* X, int ldX, __nv_bfloat16* Y, int ldY,
                   const float* bias, int T, int N, int K, int add_into, int sm_count, cudaStream_t stream);

#define OXB_DEFINE_MMQ(name, QT)                                                                                              \
  int name(OXB_MMQ_ARGS) {                                                                                                    \
    return gemm_launch_mmq<QT>(tmX, Y, bias, N, T, K, ldY, p, ws, counters, epi_mode, ar, stream, qw, gr, groups, tmWq);       \
  }

}  // namespace oxb
