// liboxb: the packed-weight dp4a GEMV (all formats and token counts it covers).
#include "gemv_quant.cuh"
#include "mmq_dispatch.h"
namespace oxb {
int gemv_quant_run(int qtype, const uint8_t* W, size_t row_bytes, const __nv_bfloat16* X, int ldX, __nv_bfloat16* Y, int ldY,
                   const float* bias, int T, int N, int K, int add_into, int sm_count, cudaStream_t stream) {
  return gemv_quant(qtype, W, row_bytes, X, ldX, Y, ldY, bias, T, N, K, add_into, sm_count, stream);
}
}  // namespace oxb
