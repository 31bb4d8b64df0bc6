// Instantiation of the TMA-staged prefill kernel for VC1D_F16 activations (see prefill_tma.cuh).
#include "prefill_tma.cuh"

namespace vc1d {
namespace tma {
template cudaError_t launch_dt<VC1D_F16>(const vc1d_prefill_args&, const TmaParams&, cudaStream_t);
}  // namespace tma
}  // namespace vc1d
