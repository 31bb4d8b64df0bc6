/*
 * vc1d.h -- C ABI of the B200 (sm_100a) depthwise causal conv1d library that backs
 * Viby's Canon A/B/C/D layers.
 *
 * Every entry point takes plain pointers and sizes.  All data pointers are DEVICE
 * pointers owned by the caller; outputs are allocated by the caller; the library
 * allocates nothing and launches on the stream handle it is given (a cudaStream_t
 * cast to void*, NULL = the legacy default stream).  The caller guarantees that the
 * device owning the buffers is the current CUDA device of the calling thread.
 *
 * Return value of every launcher: 0 on success, a negative VC1D_E_* code for an
 * invalid argument (nothing was launched), or a positive cudaError_t value when the
 * CUDA runtime refused the launch.  vc1d_status_string() names either kind.
 *
 * Tap convention (reference: model/model.py:604-666 and
 * causal-conv1d-mps/causal_conv1d_mps/causal_conv1d.metal:160-179):
 *     y[b,d,t] = act( bias[d] + sum_{w<W} weight[d,w] * x[b,d,t-(W-1-w)] ),  x[t<0] = 0
 * accumulated in fp32 and rounded once to the I/O dtype.
 */
#ifndef VC1D_H_
#define VC1D_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VC1D_ABI_VERSION 1

#if defined(__GNUC__)
#define VC1D_API __attribute__((visibility("default")))
#else
#define VC1D_API
#endif

/* element types */
enum {
    VC1D_F32 = 0,
    VC1D_BF16 = 1,
    VC1D_F16 = 2,
    /* mask-only element types */
    VC1D_U8 = 8,  /* also torch.bool */
    VC1D_I32 = 9,
    VC1D_I64 = 10
};

/* activation */
enum { VC1D_ACT_NONE = 0, VC1D_ACT_SILU = 1 };

/* error codes (negative); positive return values are cudaError_t */
enum {
    VC1D_OK = 0,
    VC1D_E_NULL = -1,        /* a required pointer is NULL */
    VC1D_E_DTYPE = -2,       /* unsupported element type */
    VC1D_E_WIDTH = -3,       /* width not in {2,3,4} */
    VC1D_E_SHAPE = -4,       /* negative size, state_len < width-1, ... */
    VC1D_E_STRIDE = -5,      /* stride combination the kernels cannot address */
    VC1D_E_STRUCT = -6,      /* struct_size does not match this library */
    VC1D_E_ACTIVATION = -7,  /* unknown activation code */
    VC1D_E_ALIAS = -8,       /* in-place use that the kernel cannot honour */
    VC1D_E_TOO_LARGE = -9    /* size beyond what an entry point supports */
};

/* kernel selection override (0 = let the library choose) -- used by benches and tests */
enum {
    VC1D_KERNEL_AUTO = 0,
    VC1D_KERNEL_CHANNEL_LAST = 1, /* 128-bit accesses along channels, register sliding window */
    VC1D_KERNEL_TIME_MAJOR = 2,   /* 128-bit accesses along time ([B,D,T] contiguous) */
    VC1D_KERNEL_GENERIC = 3,      /* scalar, any strides */
    VC1D_KERNEL_TMA = 4           /* channel-last, TMA-staged tiles with (W-1)-row halo */
};

/*
 * Prefill: causal_conv1d_fn.
 * Replaces the external CUDA kernel the reference calls at model/model.py:460-466
 * (signature mirrored at causal-conv1d-mps/causal_conv1d_mps/autograd.py:501-510), and,
 * with the optional pointers set, the surrounding elementwise passes:
 *   mask       -> model/model.py:454-457 (x * mask before the conv),
 *   residual   -> model/model.py:491 / causal_conv1d.metal:334-336 (y += residual),
 *   final_state-> model/model.py:470-489 (right-aligned last state_len masked inputs),
 *   initial_state -> model/model.py:607-617 (history prepended instead of zeros).
 *
 * x, y: logical [batch, dim, seqlen]; element strides given per tensor, so both the
 * channel-last view the model passes (strides T*D, 1, D) and contiguous [B,D,T] work.
 * Masking zeroes INPUT rows (mask value 0) before the conv; outputs at masked
 * positions are still produced.  A non-zero mask value multiplies the input row and
 * the product is rounded to the I/O dtype, as `x * mask` does in the reference.
 */
typedef struct vc1d_prefill_args {
    uint32_t struct_size;   /* sizeof(vc1d_prefill_args) */
    int32_t dtype;          /* x, y, residual, states: VC1D_F32 | VC1D_BF16 | VC1D_F16 */
    int32_t wdtype;         /* weight and bias: same as dtype, or VC1D_F32 */
    int32_t activation;     /* VC1D_ACT_* */
    int32_t batch, dim, seqlen, width;
    const void* x;
    void* y;
    const void* weight;     /* [dim, width] */
    const void* bias;       /* [dim] or NULL */
    int64_t x_stride_b, x_stride_d, x_stride_t;   /* in elements */
    int64_t y_stride_b, y_stride_d, y_stride_t;
    int64_t w_stride_d, w_stride_w;
    /* optional fused pieces (NULL = absent) */
    const void* mask;       /* [batch, seqlen] */
    int32_t mask_dtype;     /* VC1D_U8 | VC1D_I32 | VC1D_I64 | VC1D_F32 | VC1D_BF16 | VC1D_F16 */
    int32_t skip_masked_loads; /* 1: rows whose mask is 0 are not read, they count as +0 */
    int64_t mask_stride_b, mask_stride_t;
    const void* residual;   /* added to y after the activation; may equal x */
    int64_t r_stride_b, r_stride_d, r_stride_t;
    const void* initial_state; /* [batch, dim, init_len] contiguous, last width-1 columns are history */
    int32_t init_len;
    int32_t state_len;      /* columns of final_state */
    void* final_state;      /* [batch, dim, state_len] contiguous */
    /* tuning / selection: 0 = automatic */
    int32_t kernel;         /* VC1D_KERNEL_* */
    int32_t rows_per_thread;
    int32_t block_threads;
    int32_t unroll;         /* rows a thread loads before computing: 0 auto, 4 or 8 */
    /* tuning of the TMA-staged kernel: 0 = automatic */
    int32_t tma_stages;          /* ring depth, 2..8 */
    int32_t tma_ctas_per_sm;     /* persistent CTAs per SM */
    int32_t tma_slab_bytes;      /* channel slab of a tile: 128 or 256 bytes */
    int32_t tma_rows_per_thread; /* 4 or 8 consecutive rows per thread and tile */
    /* Optional scratch for the TMA-staged kernel's dynamic tile scheduler: device memory, 16-byte
     * aligned, at least 4096 + batch * ceil(seqlen / 32) bytes; with 4096 + 4 * batch * ceil(seqlen / 32)
     * + 128 bytes tables of launches of different tile height do not overwrite each other (see
     * tma_kept_tables) and a masked launch of up to 4096 tiles gets its tiles as a list ordered by
     * cost.  Its first 4096 bytes (claim counters) must be ZERO before its first use; every launch
     * leaves them zeroed.  With a mask a small pre-pass kernel fills a table behind them (a class byte
     * per tile, or the ordered list).  Launches that may overlap on the GPU must not share it.  NULL,
     * too small, or more than 1015 channel slabs = static tile assignment. */
    void* scratch;
    int64_t scratch_bytes;
    /* Packed variable-length rows (the seq_idx argument of causal_conv1d_fn, signature at
     * causal-conv1d-mps/causal_conv1d_mps/autograd.py:501-510): seq_idx[batch, seqlen] int32 names the
     * sequence every time step belongs to; a tap contributes only when its step carries the same
     * value as the output step, so sequences laid end to end in one row never see each other.
     * NULL = absent.  Not combined with mask, initial_state or final_state (VC1D_E_SHAPE). */
    const int32_t* seq_idx;
    int64_t seq_stride_b, seq_stride_t;   /* in elements */
    /* more tuning of the TMA-staged kernel: 0 = automatic */
    int32_t tma_claim_chunk;     /* consecutive tiles a CTA takes per claim: 1, 2 or 4 */
    int32_t tma_empty_store;     /* tiles whose taps are all masked: 1 = stored by the consumer warps,
                                    2 = one bulk tensor store per tile from a constant tile in shared memory */
    int32_t tma_classify;        /* tile classes of a masked launch: 0 = pre-pass kernel, writing the ordered tile list
                                    where the launch is small enough for it; 1 = pre-pass kernel, class bytes only;
                                    2 = by every CTA itself while its first tile is in flight (small masks only) */
    int32_t tma_pdl;             /* main kernel launched as a programmatic dependent of whatever precedes it in
                                    the stream: 0 = always, 1 = only when the launch uses a tile table */
    int32_t tma_static_first;    /* tiles every CTA takes without a claim before it starts claiming */
    int32_t tma_test_expire;     /* self-test of the bounded waits: 1 = every CTA withholds its first tile and
                                    polls only 4096 times, so the waits for that tile expire, the kernel
                                    returns normally with y incomplete and vc1d_tma_timeouts() has grown */
    int32_t tma_kept_tables;     /* Class tables that earlier launches left in `scratch` and that are still current:
                                    bit k = the one of tile-height slot k (vc1d_last_class_table() names the slot a
                                    launch used).  A launch whose slot's bit is set runs no pre-pass.  The caller
                                    vouches for it: the launch that wrote the table had the same mask (or seq_idx)
                                    contents and strides, batch, seqlen, width, skip_masked_loads, tma_classify and the same
                                    presence of residual and initial_state, and nothing but vc1d_prefill has
                                    written to `scratch` since. */
    int32_t tma_reserved;        /* 0 */
} vc1d_prefill_args;

VC1D_API int vc1d_prefill(const vc1d_prefill_args* args, void* stream);

/*
 * Prefill for callers that can neither allocate device memory nor hand over a scratch buffer
 * (a serving loop whose memory plan is frozen, code running under another allocator's lock or
 * callback, a host language whose binding owns no device allocator).  No counterpart in the
 * reference.  Same arguments and results as vc1d_prefill with kernel = VC1D_KERNEL_TMA (so the
 * layout must be channel-last, else VC1D_E_STRIDE; every fused option of vc1d_prefill, initial_state
 * included, is accepted); `scratch`, `scratch_bytes` and `kernel` in *args are ignored.  The dynamic
 * tile scheduler's scratch is a fixed 64 KB array inside the library's device image, so the call
 * never allocates or frees.
 *  - Limit: batch * ceil(seqlen / 32) <= VC1D_NOALLOC_MAX_TILES, else VC1D_E_TOO_LARGE and nothing
 *    is launched.  The limit is checked, and the array's counters are cleared on the caller's
 *    stream, on every call -- also for launches that end up not using the array (no mask and few
 *    tiles per CTA: static tile assignment).
 *  - The first call on each device looks the array up (with that device current) and may make
 *    the runtime load the device image: make it before any stream capture begins.
 *  - One array per device, shared by every call on that device and holding the last call's
 *    contents (each call clears what it needs on its own stream): calls whose execution may
 *    overlap on one device -- different streams, different host threads -- race on it.  Order
 *    them, or use vc1d_prefill with a scratch buffer per stream.
 */
#define VC1D_NOALLOC_MAX_TILES 61440
VC1D_API int vc1d_prefill_noalloc(const vc1d_prefill_args* args, void* stream);

/*
 * Backward of prefill: gradients of causal_conv1d_fn with the fused mask / residual.
 * Replaces what the reference gets from torch.autograd through F.conv1d (model/model.py:664-670)
 * and from the backward kernels of its Metal package
 * (causal-conv1d-mps/causal_conv1d_mps/causal_conv1d.metal:803-854 and :1354-1483; host side
 * causal_conv1d_kernel.mm:517-670, 672-779; Python contract autograd.py:116-151, 305-338):
 *     pre[t]  = bias + sum_w weight[w] * (x*mask)[t-(W-1-w)]
 *     g[t]    = dy[t] * silu'(pre[t])                       (g = dy without activation)
 *     dx[t]   = (residual ? dy[t] : 0) + mask[t] * sum_w weight[w] * g[t+(W-1-w)]
 *     dweight[d,w] += sum_{b,t} (x*mask)[t-(W-1-w)] * g[t];    dbias[d] += sum_{b,t} g[t]
 * x, dy, dx: logical [batch, dim, seqlen], element strides per tensor.  dweight [dim, width] and
 * dbias [dim] are fp32, contiguous, and ACCUMULATED into (the caller zeroes them, or sets zero_grads),
 * as the reference accumulates in fp32 and casts afterwards (causal_conv1d_kernel.mm:553-557, 771-776).
 * Sums over (batch, time) use atomic adds of per-CTA partial sums: their order is not fixed.
 */
typedef struct vc1d_prefill_bwd_args {
    uint32_t struct_size;   /* sizeof(vc1d_prefill_bwd_args) */
    int32_t dtype;          /* x, dy, dx */
    int32_t wdtype;         /* weight and bias: same as dtype, or VC1D_F32 */
    int32_t activation;     /* VC1D_ACT_* of the forward pass */
    int32_t batch, dim, seqlen, width;
    const void* x;
    const void* dy;
    void* dx;               /* must not overlap x or dy */
    const void* weight;     /* [dim, width] */
    const void* bias;       /* [dim] or NULL (the forward bias: needed to rebuild pre[t]) */
    int64_t x_stride_b, x_stride_d, x_stride_t;   /* in elements */
    int64_t dy_stride_b, dy_stride_d, dy_stride_t;
    int64_t dx_stride_b, dx_stride_d, dx_stride_t;
    int64_t w_stride_d, w_stride_w;
    const void* mask;       /* [batch, seqlen] or NULL */
    int32_t mask_dtype;
    int32_t residual;       /* 1: the forward added x to its output, so dx += dy */
    int64_t mask_stride_b, mask_stride_t;
    float* dweight;         /* [dim, width] fp32, accumulated; NULL = not wanted */
    float* dbias;           /* [dim] fp32, accumulated; NULL = not wanted */
    int32_t kernel;         /* VC1D_KERNEL_AUTO | VC1D_KERNEL_GENERIC | VC1D_KERNEL_TMA */
    int32_t tma_stages;     /* tuning of the TMA-staged kernel: 0 = automatic */
    int32_t tma_ctas_per_sm;
    int32_t tma_variant;    /* thread geometry of the TMA-staged kernel: 0 = automatic, 1 = 8 bytes of channels per
                               thread, 2 = 4 bytes (16-bit I/O), 3 = 4 bytes with twice the consumer warps */
    void* scratch;          /* as in vc1d_prefill_args */
    int64_t scratch_bytes;
    /* History of a chunked continuation (model/model.py:607-617), as in vc1d_prefill_args: the
     * forward read its last width-1 columns instead of zeros left of t = 0.  dinitial_state, when
     * given, receives the gradient for every column (zero for columns no tap reads).  Launches with
     * an initial state take the generic kernel. */
    const void* initial_state;  /* [batch, dim, init_len] contiguous, or NULL */
    void* dinitial_state;       /* [batch, dim, init_len] contiguous, or NULL */
    int32_t init_len;
    int32_t zero_grads;         /* 1: the library clears dweight / dbias itself before accumulating (on the stream,
                                   folded into the tile-classification pre-pass when the launch has one) */
    /* Packed variable-length rows, as in vc1d_prefill_args: sequence id of every step; taps and their
     * gradients stay inside a run of equal ids.  Not combined with mask or initial_state
     * (VC1D_E_SHAPE). */
    const int32_t* seq_idx;
    int64_t seq_stride_b, seq_stride_t;
} vc1d_prefill_bwd_args;

VC1D_API int vc1d_prefill_bwd(const vc1d_prefill_bwd_args* args, void* stream);
VC1D_API uint32_t vc1d_sizeof_prefill_bwd_args(void);

/*
 * Decode: causal_conv1d_update.
 * Replaces the external CUDA kernel the reference calls at model/model.py:305-311 and
 * the PyTorch single step at model/model.py:372-398:
 *     cat = [conv_state | x];  y = act(bias + cat[..., -W:] . weight);
 *     conv_state <- cat[..., -state_len:]   (in place)
 * With cache_seqlens != NULL the state is the circular buffer of
 * causal_conv1d.metal:586-664 instead: write position = cache_seqlens[b] % state_len,
 * history read modulo state_len, nothing shifts.
 * residual != 0 adds x to y after the activation (causal_conv1d.metal:655-658).
 */
typedef struct vc1d_update_args {
    uint32_t struct_size;
    int32_t dtype;          /* x, y, conv_state */
    int32_t wdtype;
    int32_t activation;
    int32_t batch, dim, width, state_len;
    const void* x;          /* [batch, dim] */
    void* y;                /* [batch, dim] */
    void* conv_state;       /* [batch, dim, state_len], updated in place */
    const void* weight;
    const void* bias;
    int64_t x_stride_b, x_stride_d;
    int64_t y_stride_b, y_stride_d;
    int64_t s_stride_b, s_stride_d, s_stride_l;
    int64_t w_stride_d, w_stride_w;
    const int32_t* cache_seqlens; /* [batch] or NULL */
    int32_t residual;
    int32_t kernel;         /* VC1D_KERNEL_AUTO | VC1D_KERNEL_GENERIC */
    int32_t block_threads;
    int32_t reserved;
} vc1d_update_args;

VC1D_API int vc1d_update(const vc1d_update_args* args, void* stream);

/* Several independent decode steps in ONE kernel launch (a table of problems instead of a launch each): calls[i]
 * is a complete vc1d_update_args, with its own batch, dim, state_len, width, activation, strides and buffers; all
 * of one I/O dtype; at most VC1D_UPDATE_MULTI_MAX of them.  The problems must be independent of each other (none
 * reads what another writes): the Canon steps of one token of one network are NOT (each feeds the next), the
 * steps of several requests, networks or beams are.  Results are those of vc1d_update called on each, bit for
 * bit.  The reference has no counterpart; it launches one kernel per Canon step (model/model.py:305-311). */
#define VC1D_UPDATE_MULTI_MAX 80
VC1D_API int vc1d_update_multi(const vc1d_update_args* calls, int32_t n_calls, void* stream);

/*
 * Backward of one decode step (causal_conv1d_update), for the state the step STARTED from:
 *     win = last W entries of [conv_state | x] (or the circular history);  pre = bias + win . weight
 *     g = dy * silu'(pre);   dx = weight[W-1] * g (+ dy with residual);   dstate[col of tap w] = weight[w] * g
 *     dweight[d,w] += sum_b win[w] * g;   dbias[d] += sum_b g
 * Replaces short_conv_update_bwd of causal-conv1d-mps (causal_conv1d.metal:1738-1845, host side
 * causal_conv1d_kernel.mm:781-888, Python contract autograd.py:455-482).  dstate columns that no tap
 * reads are set to zero.  dweight / dbias: fp32, accumulated, caller-zeroed, as in vc1d_prefill_bwd.
 */
typedef struct vc1d_update_bwd_args {
    uint32_t struct_size;
    int32_t dtype;          /* x, conv_state, dy, dx, dstate */
    int32_t wdtype;
    int32_t activation;
    int32_t batch, dim, width, state_len;
    const void* x;          /* [batch, dim] */
    const void* conv_state; /* [batch, dim, state_len]: the state before the step */
    const void* dy;         /* [batch, dim] */
    void* dx;               /* [batch, dim] */
    void* dstate;           /* [batch, dim, state_len] contiguous, or NULL */
    const void* weight;
    const void* bias;
    int64_t x_stride_b, x_stride_d;
    int64_t dy_stride_b, dy_stride_d;
    int64_t dx_stride_b, dx_stride_d;
    int64_t s_stride_b, s_stride_d, s_stride_l;
    int64_t w_stride_d, w_stride_w;
    const int32_t* cache_seqlens; /* [batch] or NULL: circular state as in vc1d_update */
    int32_t residual;
    int32_t reserved;
    float* dweight;         /* [dim, width] fp32, accumulated; NULL = not wanted */
    float* dbias;           /* [dim] fp32, accumulated; NULL = not wanted */
} vc1d_update_bwd_args;

VC1D_API int vc1d_update_bwd(const vc1d_update_bwd_args* args, void* stream);
VC1D_API uint32_t vc1d_sizeof_update_bwd_args(void);

/* ABI version of the loaded library (VC1D_ABI_VERSION it was built with). */
VC1D_API int vc1d_abi_version(void);

/* sizeof() of the two argument structs as the library was built -- lets a binding
 * verify its own struct layout before the first launch. */
VC1D_API uint32_t vc1d_sizeof_prefill_args(void);
VC1D_API uint32_t vc1d_sizeof_update_args(void);

/* Name of a return code: VC1D_E_* or a cudaError_t.  Never NULL; static storage. */
VC1D_API const char* vc1d_status_string(int status);

/* Number of kernel launches this process has made through the library (all threads; the tile
 * classification pre-pass of a masked launch counts as a launch of its own).
 * The reference swallows kernel exceptions and silently falls back
 * (model/model.py:314-317, 492-495); callers use this to prove the kernels ran. */
VC1D_API uint64_t vc1d_launch_count(void);

/* Name of the kernel the most recent launcher call on this thread selected ("channel_last",
 * "time_major", "generic", "tma", "update_vec", "update_lane", "update_generic", "bwd_tma", "bwd_generic",
 * "update_bwd").  Per host thread: a backward pass run by an autograd worker thread does not show
 * up in the thread that called the forward. */
VC1D_API const char* vc1d_last_kernel(void);

/* What the calling thread's last vc1d_prefill did with tile-class tables in `scratch`.  Low byte: 0 = touched
   none, 1 = its pre-pass wrote the table of its tile-height slot, 2 = it read the one already there
   (tma_kept_tables), 3 = the buffer has room for one table only and the pre-pass wrote it at the front: no
   table there can be kept.  Bits 8 and up: the slot (0, 1, 2).  No reference counterpart. */
VC1D_API int vc1d_last_class_table(void);

/* Number of bounded mbarrier waits that expired inside the TMA-staged kernels since the process
 * started (0 in a healthy run; a CTA whose wait expires abandons its remaining tiles).  Reads a
 * device counter with a synchronising copy: call it after the stream has been synchronised. */
VC1D_API unsigned int vc1d_tma_timeouts(void);

/* Programmatic dependent launch between this library's kernels on one stream (a decode step's launch
 * overlapping the previous step's tail; a masked prefill's main kernel overlapping its
 * tile-classification pre-pass).  On by default unless the environment has VC1D_NO_PDL=1.
 * enabled: 1 = on, 0 = off, negative = back to the environment's choice.  Returns the setting that was
 * in effect before the call.  Process-wide; affects launches made after it returns.  (The reference
 * has no counterpart: its kernels come from an external package, model/model.py:20-30.) */
VC1D_API int vc1d_set_pdl(int enabled);

#ifdef __cplusplus
}
#endif
#endif /* VC1D_H_ */
