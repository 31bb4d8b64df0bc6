// vc1d_prefill_noalloc: the TMA-staged prefill kernel with dynamic tile claims, for callers that
// cannot hand the library a scratch buffer.
//
// The TMA-staged kernel balances its persistent CTAs by letting them claim tiles from one counter
// per channel slab, and (with an attention mask) reads one class byte per tile that a pre-pass
// wrote; both live in scratch memory that vc1d_prefill expects from the caller.  A caller that sits
// inside a serving loop with a frozen memory plan, or inside someone else's allocator callback, has
// no buffer to give and must not allocate one.  This entry point keeps the scratch in a
// fixed-size array in the library's own device image instead: no cudaMalloc, no cudaFree, no
// allocating library routine, on any call.
//
// There is no counterpart in the reference (its conv kernels come from an external package and use
// no scratch memory: model/model.py:20-30).
#include <cuda_runtime.h>

#include <atomic>

#include "../../include/vc1d.h"

namespace {

// Scheduler scratch of this entry point: 4096 bytes of claim counters, then one class byte per
// (sequence, 32-row time tile).  64 KB: up to 61 440 tiles, e.g. batch 32 x seqlen 61 440 or
// batch 512 x seqlen 3840.  One array per device (every device that loads the library has its own
// copy); every call on a device shares it.
constexpr long long kCounterBytes = 4096;
constexpr long long kScratchBytes = 64 * 1024;
constexpr long long kMaxTiles = kScratchBytes - kCounterBytes;
static_assert(kMaxTiles == VC1D_NOALLOC_MAX_TILES, "the header states this limit");

static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::atomic<void*> g_scratch_ptr[kMaxDevices];

// Address of the array on the current device.  The first call on a device asks the runtime (which
// may load the device image then: do it outside any stream capture); later calls read the cache.
cudaError_t scratch_of_current_device(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    void* p = g_scratch_ptr[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return e;
        if (p == nullptr) return cudaErrorInvalidSymbol;
        g_scratch_ptr[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return cudaSuccess;
}

}  // namespace

extern "C" VC1D_API int vc1d_prefill_noalloc(const vc1d_prefill_args* args, void* stream) {
    if (args == nullptr) return VC1D_E_NULL;
    if (args->struct_size != (int32_t)sizeof(vc1d_prefill_args)) return VC1D_E_STRUCT;
    if (args->batch < 0 || args->seqlen < 0 || args->dim < 0) return VC1D_E_SHAPE;
    // the limit: one class byte per (sequence, 32-row tile) must fit behind the counters
    const long long tiles = (long long)args->batch * ((args->seqlen + 31) / 32);
    if (tiles > kMaxTiles) return VC1D_E_TOO_LARGE;

    void* scratch = nullptr;
    cudaError_t e = scratch_of_current_device(&scratch);
    if (e != cudaSuccess) return (int)e;
    // The array keeps whatever the last call left.  The counters must start at zero; a call that
    // ended abnormally could have left them otherwise, so clear them on the caller's stream.  The
    // class bytes need no clearing: the pre-pass rewrites every one this call reads.
    e = cudaMemsetAsync(scratch, 0, (size_t)kCounterBytes, reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return (int)e;

    vc1d_prefill_args a = *args;
    a.kernel = VC1D_KERNEL_TMA;
    a.scratch = scratch;
    a.scratch_bytes = kScratchBytes;
    return vc1d_prefill(&a, stream);
}
