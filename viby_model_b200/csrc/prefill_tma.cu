// Host side of the TMA-staged prefill kernel: driver entry point for the tensor-map encoder, the
// device counter of expired waits, and the dispatch into the per-dtype instantiations
// (prefill_tma_f32.cu, prefill_tma_bf16.cu, prefill_tma_f16.cu).
#include <mutex>

#include "prefill_tma.cuh"

namespace vc1d {
namespace tma {

__device__ unsigned int g_tma_timeouts = 0;

EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(sym);
    });
    return fn;
}

// address of the counter on the current device (a __device__ variable exists once per device)
unsigned int* timeouts_ptr() {
    static std::atomic<unsigned int*> cache[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    if (dev >= 0 && dev < 64) {
        unsigned int* p = cache[dev].load(std::memory_order_acquire);
        if (p != nullptr) return p;
    }
    void* addr = nullptr;
    if (cudaGetSymbolAddress(&addr, g_tma_timeouts) != cudaSuccess) return nullptr;
    if (dev >= 0 && dev < 64) cache[dev].store(static_cast<unsigned int*>(addr), std::memory_order_release);
    return static_cast<unsigned int*>(addr);
}

extern template cudaError_t launch_dt<VC1D_F32>(const vc1d_prefill_args&, const TmaParams&, cudaStream_t);
extern template cudaError_t launch_dt<VC1D_BF16>(const vc1d_prefill_args&, const TmaParams&, cudaStream_t);
extern template cudaError_t launch_dt<VC1D_F16>(const vc1d_prefill_args&, const TmaParams&, cudaStream_t);

}  // namespace tma

bool tma_available() { return tma::encode_fn() != nullptr; }

unsigned int tma_timeouts() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, tma::g_tma_timeouts, sizeof(v)) != cudaSuccess) return 0xffffffffu;
    return v;
}

cudaError_t launch_prefill_tma(const vc1d_prefill_args& a, cudaStream_t s) {
    const int eb = elem_bytes(a.dtype);
    tma::TmaParams p = {};
    p.y = reinterpret_cast<char*>(a.y);
    p.syb = a.y_stride_b * eb;
    p.syt = a.y_stride_t * eb;
    p.x = reinterpret_cast<const char*>(a.x);
    p.res = reinterpret_cast<const char*>(a.residual);
    p.init = reinterpret_cast<const char*>(a.initial_state);
    p.init_len = a.init_len;
    p.weight = a.weight;
    p.bias = a.bias;
    p.mask = a.mask;
    p.fstate = reinterpret_cast<char*>(a.final_state);
    p.sched = nullptr;
    p.timeouts = tma::timeouts_ptr();
    if (p.timeouts == nullptr) return cudaErrorNotSupported;
    p.sxb = a.x_stride_b * eb;
    p.sxt = a.x_stride_t * eb;
    p.srb = a.r_stride_b * eb;
    p.srt = a.r_stride_t * eb;
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
    p.skip = (a.mask != nullptr && a.skip_masked_loads) ? 1 : 0;
    p.res_is_x = (a.residual != nullptr && a.residual == a.x && a.r_stride_b == a.x_stride_b &&
                  a.r_stride_t == a.x_stride_t)
                     ? 1
                     : 0;
    p.state_len = a.state_len;
    p.stages = 0;
    p.seg_mode = 0;
    p.chunk = 1;
    p.empty_tma = 0;
    if (a.seq_idx != nullptr) {
        // sequence ids travel the mask's path: per-row values fetched by the producer, tile classes
        // from the pre-pass; a row whose value is not one starts a new sequence
        p.mask = a.seq_idx;
        p.mask_dtype = VC1D_I32;
        p.smb = a.seq_stride_b;
        p.smt = a.seq_stride_t;
        p.skip = 0;
        p.seg_mode = 1;
    }
    switch (a.dtype) {
        case VC1D_F32: return tma::launch_dt<VC1D_F32>(a, p, s);
        case VC1D_BF16: return tma::launch_dt<VC1D_BF16>(a, p, s);
        default: return tma::launch_dt<VC1D_F16>(a, p, s);
    }
}

}  // namespace vc1d
