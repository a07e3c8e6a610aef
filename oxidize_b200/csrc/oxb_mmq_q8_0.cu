// liboxb: the packed-weight tcgen05 GEMM for one block format (QT_Q8_0), all token tiles.
#include "mmq_dispatch.h"
namespace oxb {
OXB_DEFINE_MMQ(gemm_mmq_q8_0, QT_Q8_0)
}
