// liboxb: the packed-weight tcgen05 GEMM for one block format (QT_Q4_0), all token tiles.
#include "mmq_dispatch.h"
namespace oxb {
OXB_DEFINE_MMQ(gemm_mmq_q4_0, QT_Q4_0)
}
