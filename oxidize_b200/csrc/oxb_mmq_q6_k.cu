// liboxb: the packed-weight tcgen05 GEMM for one block format (QT_Q6_K), all token tiles.
#include "mmq_dispatch.h"
namespace oxb {
OXB_DEFINE_MMQ(gemm_mmq_q6_k, QT_Q6_K)
}
