// placeholder until the tcgen05 GEMM lands
#include "nrs_internal.h"
int nrs_tc_gemm(nrs_ctx*, int, int, int, int, int, int, const float*, const float*, float*, const float*, int, float) {
  return NRS_ERR_UNSUPPORTED;
}
extern "C" int nrs_has_tensor_core_path(void) { return 0; }
