// liboxb: the packed-weight tcgen05 GEMM for one block format (QT_NVFP4), all token tiles.
#include "mmq_dispatch.h"
namespace oxb {
OXB_DEFINE_MMQ(gemm_mmq_nvfp4, QT_NVFP4)
}
