// liboxb: the packed-weight tcgen05 GEMM for one block format (QT_FP8B), all token tiles.
#include "mmq_dispatch.h"
namespace oxb {
OXB_DEFINE_MMQ(gemm_mmq_fp8b, QT_FP8B)
}
