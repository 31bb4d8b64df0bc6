// Instantiation of the TMA-staged prefill backward kernel for VC1D_BF16 activations (see prefill_bwd_tma.cuh).
#include "prefill_bwd_tma.cuh"

namespace vc1d {
namespace tma {
template cudaError_t launch_bwd_dt<VC1D_BF16>(const vc1d_prefill_bwd_args&, const BwdParams&, cudaStream_t);
}  // namespace tma
}  // namespace vc1d
