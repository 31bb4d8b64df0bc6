// Interface between the validating C-ABI layer (api.cu) and the per-kernel translation
// units.  Each launcher receives arguments that api.cu has already validated and that
// satisfy the layout preconditions listed beside it; it returns a cudaError_t.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/vc1d.h"

namespace vc1d {

// Number of SMs of the current device (cached per device ordinal).
int sm_count();

// Programmatic dependent launch between this library's kernels (on unless the environment sets
// VC1D_NO_PDL=1; read once).
bool pdl_enabled();

// Kernel launch bookkeeping shared by all launchers.
void note_launch(const char* kernel_name);
// what the calling thread's last prefill launch did with a class table in scratch: 0 none, 1 written, 2 kept
void note_class_table(int state);

// Channel-last prefill: x/y (and residual) have channel stride 1, dim % vec == 0, every
// base pointer and every batch/time stride is 16-byte aligned.
cudaError_t launch_prefill_channel_last(const vc1d_prefill_args& a, cudaStream_t s);

// Same preconditions as channel-last plus: dim*elem_size % 16 == 0
// (tensor-map stride rule).  Stages (rows + halo) x channel tiles through shared memory
// with cp.async.bulk.tensor.
cudaError_t launch_prefill_tma(const vc1d_prefill_args& a, cudaStream_t s);
bool tma_available();
// mbarrier waits that expired inside the TMA kernel since the process started (synchronising read).
unsigned int tma_timeouts();

// Time-major prefill: x/y have time stride 1, seqlen % vec == 0, aligned rows, none of
// mask / residual / initial_state / final_state.
cudaError_t launch_prefill_time_major(const vc1d_prefill_args& a, cudaStream_t s);

// Any strides, every option.
cudaError_t launch_prefill_generic(const vc1d_prefill_args& a, cudaStream_t s);

// Backward of prefill.  Generic: any strides.  TMA-staged: x, dy, dx channel-last (channel stride
// 1, 16-byte aligned rows), dim * elem_size a multiple of 16.
cudaError_t launch_prefill_bwd_generic(const vc1d_prefill_bwd_args& a, cudaStream_t s);
cudaError_t launch_prefill_bwd_tma(const vc1d_prefill_bwd_args& a, cudaStream_t s);

// Vectorised decode: x/y channel stride 1, conv_state strides (.., state_len, 1),
// dim % vec == 0, aligned, state_len in {1,2,3,4,8}, no cache_seqlens.
cudaError_t launch_update_vec(const vc1d_update_args& a, cudaStream_t s);
bool update_vec_supports(int state_len, int width);

// One channel per lane: x/y channel stride 1, conv_state strides (.., state_len, 1) and 16-byte
// aligned rows, state_len * elem_size 16 or 32 bytes; shifting or circular (cache_seqlens) state.
cudaError_t launch_update_lane(const vc1d_update_args& a, cudaStream_t s);
bool update_lane_supports(int dtype, int state_len, int width);

// Any strides, shifting or circular state.
cudaError_t launch_update_generic(const vc1d_update_args& a, cudaStream_t s);
// n independent problems of one I/O dtype in one launch; vec_ok[i] = problem i fits the vectorised code
cudaError_t launch_update_multi(const vc1d_update_args* calls, int n, const unsigned char* vec_ok, cudaStream_t s);

// Backward of one decode step: any strides, shifting or circular state.
cudaError_t launch_update_bwd(const vc1d_update_bwd_args& a, cudaStream_t s);

inline int elem_bytes(int dtype) {
    switch (dtype) {
        case VC1D_F32: return 4;
        case VC1D_BF16: return 2;
        case VC1D_F16: return 2;
        case VC1D_U8: return 1;
        case VC1D_I32: return 4;
        case VC1D_I64: return 8;
        default: return 0;
    }
}

}  // namespace vc1d
