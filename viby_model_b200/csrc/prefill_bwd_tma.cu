// Host side of the TMA-staged prefill backward kernel: fills the kernel parameters and dispatches
// into the per-dtype instantiations (prefill_bwd_tma_f32.cu, prefill_bwd_tma_bf16.cu,
// prefill_bwd_tma_f16.cu).
#include "prefill_bwd_tma.cuh"

namespace vc1d {
namespace tma {

extern template cudaError_t launch_bwd_dt<VC1D_F32>(const vc1d_prefill_bwd_args&, const BwdParams&, cudaStream_t);
extern template cudaError_t launch_bwd_dt<VC1D_BF16>(const vc1d_prefill_bwd_args&, const BwdParams&, cudaStream_t);
extern template cudaError_t launch_bwd_dt<VC1D_F16>(const vc1d_prefill_bwd_args&, const BwdParams&, cudaStream_t);

}  // namespace tma

cudaError_t launch_prefill_bwd_tma(const vc1d_prefill_bwd_args& a, cudaStream_t s) {
    const int eb = elem_bytes(a.dtype);
    tma::BwdParams p;
    p.dx = reinterpret_cast<char*>(a.dx);
    p.weight = a.weight;
    p.bias = a.bias;
    p.mask = a.mask;
    p.dweight = a.dweight;
    p.dbias = a.dbias;
    p.sched = nullptr;
    p.timeouts = tma::timeouts_ptr();
    if (p.timeouts == nullptr) return cudaErrorNotSupported;
    p.sdb = a.dx_stride_b * eb;
    p.sdt = a.dx_stride_t * eb;
    p.smb = a.mask_stride_b;
    p.smt = a.mask_stride_t;
    p.wsd = a.w_stride_d;
    p.wsw = a.w_stride_w;
    p.wdtype = a.wdtype;
    p.B = a.batch;
    p.D = a.dim;
    p.T = a.seqlen;
    p.n_ttile = p.n_rowtiles = p.ctas_per_slab = 0;
    p.mask_dtype = a.mask_dtype;
    p.residual = a.residual != 0;
    p.stages = 0;
    p.seg_mode = 0;
    if (a.seq_idx != nullptr) {
        // sequence ids travel the mask's path (per-row values, tile classes): a value other than one marks
        // the first row of a sequence
        p.mask = a.seq_idx;
        p.mask_dtype = VC1D_I32;
        p.smb = a.seq_stride_b;
        p.smt = a.seq_stride_t;
        p.seg_mode = 1;
    }
    switch (a.dtype) {
        case VC1D_F32: return tma::launch_bwd_dt<VC1D_F32>(a, p, s);
        case VC1D_BF16: return tma::launch_bwd_dt<VC1D_BF16>(a, p, s);
        default: return tma::launch_bwd_dt<VC1D_F16>(a, p, s);
    }
}

}  // namespace vc1d
