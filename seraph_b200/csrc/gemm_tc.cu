// placeholder until the tcgen05 path lands
#include "sb_internal.h"
extern "C" int sb_gemm_tc(sb_ctx_t*, const float*, const float*, float*, int, int, int, int, int, int, int) { return 1; }
