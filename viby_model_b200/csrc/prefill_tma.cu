// Placeholder until the TMA-staged prefill kernel lands: reports itself unavailable so the
// dispatcher never selects it.
#include "vc1d_internal.h"

namespace vc1d {
bool tma_available() { return false; }
cudaError_t launch_prefill_tma(const vc1d_prefill_args&, cudaStream_t) { return cudaErrorNotSupported; }
}  // namespace vc1d
