// liboxb: the packed-weight tcgen05 GEMM for one block format (QT_Q4_K), all token tiles.
#include "mmq_dispatch.h"
namespace oxb {
OXB_DEFINE_MMQ(gemm_mmq_q4_k, QT_Q4_K)
}
#ifdef OXB_MMQ_TRACE
// debugging aid: the phase trace of the last traced CTA of this unit's kernels
extern "C" __attribute__((visibility("default"))) int oxb_mmq_trace(long long* out32) {
  return (int)cudaMemcpyFromSymbol(out32, oxb::g_oxb_mmq_trace, 32 * sizeof(long long));
}
#endif
