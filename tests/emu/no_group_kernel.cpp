// Stands in for the shuffle-based group kernel (quant_groups.cu) when quant_rows.cu is emulated on its own: it
// declines every shape, so group-wise requests run through the general row kernels.  TEST INFRASTRUCTURE ONLY.
#include <cuda_runtime.h>
#include <stdint.h>

namespace amct {
int quant_groups_try(const void*, int, int64_t, int64_t, int64_t, const void*, int, int, int, int, int, float*, int*, int,
                     void*, int64_t, int*, cudaStream_t) {
  return 1;
}
}  // namespace amct
