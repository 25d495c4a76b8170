// Prefill dequant-GEMM on tcgen05 (placeholder until the kernel lands: reports
// "not eligible", so the operator uses the GEMV path in row chunks).
#include "gaf_internal.h"

namespace tgaf {

bool gemm_tc_eligible(const WeightView &, uint32_t) { return false; }

cudaError_t gemm_tc(const WeightView &, const void *, void *, uint32_t, cudaStream_t, int, unsigned int *) {
    return cudaErrorNotSupported;
}

}  // namespace tgaf
