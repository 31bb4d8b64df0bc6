// Register-window prefill kernel for the channel-last layout the Canon layers pass
// (x.transpose(1,2) of a contiguous [B,T,D] tensor, reference model/model.py:459-466), with the
// fused options of the layer around it (mask model/model.py:454-457, residual :491, state
// :470-489, history :607-617).
//
// Work unit: one thread owns VB bytes of channels (8 = four bf16, or 16) and a chunk of R
// consecutive time rows.  Units are numbered with the channel slice fastest, so a warp reads
// 32*VB contiguous bytes per row, a 256-thread CTA 2-4 KB, and no lane idles whatever dim is.
// Weights and bias of the owned channels live in registers as fp32 pairs; the (W-1)-row
// history is a register window rotated by index, seeded by re-reading the W-1 rows before the
// chunk (L1/L2 hits: the thread of the chunk above streams them from HBM).  Loads are issued U
// rows at a time before any arithmetic, so a thread keeps U*VB bytes in flight and an SM, at
// ~900 resident threads, some 50 KB -- the depth at which this GPU's HBM streams best.  There
// is no shared memory and no barrier: the grid is many small CTAs and the hardware scheduler
// balances ragged (masked) batches and uneven SMs by itself.
//
// Masked rows are not read at all when skip_masked_loads is set; a chunk tail in which every
// tap of every row is masked stores act(bias) without any arithmetic.
#include "vc1d_common.cuh"
#include "vc1d_internal.h"

namespace vc1d {
namespace {

struct CLParams {
    const char* x;
    char* y;
    const char* res;
    const void* weight;
    const void* bias;
    const void* mask;
    const char* init;
    char* fstate;
    long long sxb, sxt;  // bytes
    long long syb, syt;
    long long srb, srt;
    long long smb, smt;  // elements
    long long wsd, wsw;  // elements
    long long total;
    int wdtype;
    int B, D, T;
    int nslice, nchunk, R;
    int mask_dtype;
    int skip;
    int init_len, state_len;
};

template <int DT, int W, int VB>
__device__ __forceinline__ void load_weights(const CLParams& p, int d0, float2 (&wp)[W][Slice<DT, VB>::kPairs],
                                             float2 (&bp)[Slice<DT, VB>::kPairs]) {
    using E = Elem<DT>;
    using T = typename E::type;
    constexpr int NE = Slice<DT, VB>::kElems;
    constexpr int NP = Slice<DT, VB>::kPairs;
    float wf[NE][W];
    float bf[NE];
#pragma unroll
    for (int c = 0; c < NE; ++c) {
#pragma unroll
        for (int w = 0; w < W; ++w) {
            const long long idx = (long long)(d0 + c) * p.wsd + (long long)w * p.wsw;
            wf[c][w] = (p.wdtype == VC1D_F32) ? __ldg(reinterpret_cast<const float*>(p.weight) + idx)
                                              : E::to_float(__ldg(reinterpret_cast<const T*>(p.weight) + idx));
        }
        bf[c] = 0.f;
        if (p.bias != nullptr) {
            bf[c] = (p.wdtype == VC1D_F32) ? __ldg(reinterpret_cast<const float*>(p.bias) + d0 + c)
                                           : E::to_float(__ldg(reinterpret_cast<const T*>(p.bias) + d0 + c));
        }
    }
#pragma unroll
    for (int q = 0; q < NP; ++q) {
#pragma unroll
        for (int w = 0; w < W; ++w) wp[w][q] = make_float2(wf[2 * q][w], wf[2 * q + 1][w]);
        bp[q] = make_float2(bf[2 * q], bf[2 * q + 1]);
    }
}

// raw row -> fp32 pairs, with the multiplicative mask of the reference (x * mask, rounded to the
// I/O dtype) when the mask value is not exactly 1
template <int DT, int VB>
__device__ __forceinline__ void decode_row(const uint32_t (&raw)[Slice<DT, VB>::kWords], bool masked, float mk,
                                           float2 (&f)[Slice<DT, VB>::kPairs]) {
    using S = Slice<DT, VB>;
    S::unpack(raw, f);
    if (masked && mk != 1.0f) {
        const float2 m2 = make_float2(mk, mk);
#pragma unroll
        for (int q = 0; q < S::kPairs; ++q) f[q] = S::round_trip(mul2(f[q], m2));
    }
}

// one column of an initial state [B, D, init_len] for this thread's channels, as a raw row
template <int DT, int VB>
__device__ __forceinline__ void load_init_column(const char* init, long long row0, int init_len, int col,
                                                 uint32_t (&raw)[Slice<DT, VB>::kWords]) {
    using T = typename Elem<DT>::type;
    constexpr int NE = Slice<DT, VB>::kElems;
    T vals[NE];
    const T* in = reinterpret_cast<const T*>(init);
#pragma unroll
    for (int c = 0; c < NE; ++c) vals[c] = in[(row0 + c) * init_len + col];
    const uint32_t* w = reinterpret_cast<const uint32_t*>(vals);
#pragma unroll
    for (int i = 0; i < Slice<DT, VB>::kWords; ++i) raw[i] = w[i];
}

template <int DT, int W, int VB, int U, bool ACT, bool MASK, bool RES>
__global__ void __launch_bounds__(256, (VB == 8 && !MASK) ? 3 : 2) k_prefill_window(const CLParams p) {
    using E = Elem<DT>;
    using S = Slice<DT, VB>;
    constexpr int NE = S::kElems;
    constexpr int NP = S::kPairs;
    constexpr int NW = S::kWords;
    constexpr int H = W - 1;
    constexpr int HS = H > 0 ? H : 1;

    const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= p.total) return;
    const int slice = (int)(g % p.nslice);
    const long long q0 = g / p.nslice;
    const int chunk = (int)(q0 % p.nchunk);
    const int b = (int)(q0 / p.nchunk);
    const int d0 = slice * NE;
    const int t0 = chunk * p.R;
    const int t1 = min(t0 + p.R, p.T);

    float2 wp[W][NP];
    float2 bp[NP];
    load_weights<DT, W, VB>(p, d0, wp, bp);

    const char* xb = p.x + (long long)b * p.sxb + (long long)d0 * E::kBytes;
    char* yb = p.y + (long long)b * p.syb + (long long)d0 * E::kBytes;
    const char* rb = RES ? p.res + (long long)b * p.srb + (long long)d0 * E::kBytes : nullptr;
    const long long mrow = (long long)b * p.smb;
    const long long row0 = (long long)b * p.D + d0;  // first owned row of a [B*D, L] state

    // ---- history: the W-1 rows before the chunk; hist[j] is the row W-1-j steps back ... oldest first
    float2 hist[HS][NP];
    int zero_run = 0;  // trailing rows known to be +0 because their mask is 0 and loads are skipped
#pragma unroll
    for (int j = 0; j < H; ++j) {
        const int t = t0 - H + j;
        uint32_t raw[NW];
#pragma unroll
        for (int i = 0; i < NW; ++i) raw[i] = 0u;
        float mk = 1.0f;
        bool zero = false;
        if (t >= 0) {
            if (MASK) mk = load_mask(p.mask, mrow + (long long)t * p.smt, p.mask_dtype);
            if (MASK && p.skip && mk == 0.0f)
                zero = true;
            else
                S::ldg(xb + (long long)t * p.sxt, raw);
        } else if (p.init != nullptr) {
            load_init_column<DT, VB>(p.init, row0, p.init_len, p.init_len + t, raw);
        } else {
            zero = true;  // causal left padding
        }
        decode_row<DT, VB>(raw, MASK && t >= 0 && !zero, mk, hist[j]);
        zero_run = zero ? zero_run + 1 : 0;
    }

    // value of a row whose W taps are all +0: act(bias)
    uint32_t const_row[NW];
    {
        float2 c[NP];
#pragma unroll
        for (int qq = 0; qq < NP; ++qq) c[qq] = ACT ? silu2<E::kPreciseSilu>(bp[qq]) : bp[qq];
        S::pack(c, const_row);
    }

    // ---- main sweep, U rows at a time ------------------------------------------------------
    float mk_next[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
        mk_next[k] = 1.0f;
        if (MASK && t0 + k < t1) mk_next[k] = load_mask(p.mask, mrow + (long long)(t0 + k) * p.smt, p.mask_dtype);
    }
    for (int tb = t0; tb < t1; tb += U) {
        float mk[U];
        bool skip_row[U];
        bool any_live = false;
        uint32_t raw[U][NW];
        uint32_t rres[RES ? U : 1][NW];
#pragma unroll
        for (int k = 0; k < U; ++k) {
            mk[k] = mk_next[k];
            const bool in = tb + k < t1;
            skip_row[k] = !in || (MASK && p.skip && mk[k] == 0.0f);
            any_live |= in && !skip_row[k];
#pragma unroll
            for (int i = 0; i < NW; ++i) raw[k][i] = 0u;
            if (!skip_row[k]) S::ldg(xb + (long long)(tb + k) * p.sxt, raw[k]);
            if (RES) {
#pragma unroll
                for (int i = 0; i < NW; ++i) rres[k][i] = 0u;
                if (in) S::ldg(rb + (long long)(tb + k) * p.srt, rres[k]);
            }
        }
        if (MASK) {
            // the mask values of the next batch travel while this batch is computed
#pragma unroll
            for (int k = 0; k < U; ++k) {
                mk_next[k] = 1.0f;
                if (tb + U + k < t1)
                    mk_next[k] = load_mask(p.mask, mrow + (long long)(tb + U + k) * p.smt, p.mask_dtype);
            }
        }
        if (MASK && !RES && !any_live && zero_run >= H) {
            // every tap of every row of this batch is +0
#pragma unroll
            for (int k = 0; k < U; ++k)
                if (tb + k < t1) S::stg(yb + (long long)(tb + k) * p.syt, const_row);
            zero_run += U;
            continue;  // hist stays all-zero
        }
        static_for<0, U>([&](auto kc) {
            constexpr int k = decltype(kc)::value;
            if (tb + k < t1) {
                float2 cur[NP];
                decode_row<DT, VB>(raw[k], MASK && !skip_row[k], mk[k], cur);
                float2 acc[NP];
#pragma unroll
                for (int qq = 0; qq < NP; ++qq) {
                    acc[qq] = bp[qq];
#pragma unroll
                    for (int w = 0; w < H; ++w) acc[qq] = fma2(wp[w][qq], hist[(k + w) % HS][qq], acc[qq]);
                    acc[qq] = fma2(wp[H][qq], cur[qq], acc[qq]);
                    if (ACT) acc[qq] = silu2<E::kPreciseSilu>(acc[qq]);
                }
                if (RES) {
                    // same roundings as the unfused `x + y`: y rounded to the I/O dtype, then the sum
                    float2 rr[NP];
                    S::unpack(rres[k], rr);
#pragma unroll
                    for (int qq = 0; qq < NP; ++qq) acc[qq] = add2(S::round_trip(acc[qq]), rr[qq]);
                }
                uint32_t outw[NW];
                S::pack(acc, outw);
                S::stg(yb + (long long)(tb + k) * p.syt, outw);
                if (H > 0) {
#pragma unroll
                    for (int qq = 0; qq < NP; ++qq) hist[k % HS][qq] = cur[qq];
                }
                zero_run = skip_row[k] ? zero_run + 1 : 0;
            }
        });
        // the batch advanced the window by U rows: bring the oldest row back to slot 0
        // (rows past t1 only occur in the last batch, after which the window is dead)
        if (H > 1 && (U % HS) != 0) {
            float2 tmp[HS][NP];
#pragma unroll
            for (int w = 0; w < H; ++w)
#pragma unroll
                for (int qq = 0; qq < NP; ++qq) tmp[w][qq] = hist[(U + w) % HS][qq];
#pragma unroll
            for (int w = 0; w < H; ++w)
#pragma unroll
                for (int qq = 0; qq < NP; ++qq) hist[w][qq] = tmp[w][qq];
        }
    }

    // ---- final state: right-aligned last state_len masked inputs ------------------------
    if (p.fstate != nullptr && t1 == p.T) {
        using T = typename E::type;
        const int L = p.state_len;
        T* out = reinterpret_cast<T*>(p.fstate) + row0 * L;
        for (int j = 0; j < L; ++j) {
            const int t = p.T - L + j;
            uint32_t raw[NW];
#pragma unroll
            for (int i = 0; i < NW; ++i) raw[i] = 0u;
            if (t >= 0) {
                S::ldg(xb + (long long)t * p.sxt, raw);
                if (MASK) {
                    const float mkv = load_mask(p.mask, mrow + (long long)t * p.smt, p.mask_dtype);
                    if (mkv != 1.0f) {
                        float2 f[NP];
                        S::unpack(raw, f);
                        const float2 m2 = make_float2(mkv, mkv);
#pragma unroll
                        for (int qq = 0; qq < NP; ++qq) f[qq] = mul2(f[qq], m2);
                        S::pack(f, raw);
                    }
                }
            } else if (p.init != nullptr && p.init_len + t >= 0) {
                load_init_column<DT, VB>(p.init, row0, p.init_len, p.init_len + t, raw);
            }
            const T* vals = reinterpret_cast<const T*>(raw);
#pragma unroll
            for (int c = 0; c < NE; ++c) out[(long long)c * L + j] = vals[c];
        }
    }
}

template <int DT, int W, int VB, bool ACT>
cudaError_t launch_flags(const CLParams& p, bool mask, bool res, int block, cudaStream_t s) {
    constexpr int U = 8;
    const long long blocks = (p.total + block - 1) / block;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    const dim3 grid((unsigned)blocks);
    if (mask && res)
        k_prefill_window<DT, W, VB, U, ACT, true, true><<<grid, block, 0, s>>>(p);
    else if (mask)
        k_prefill_window<DT, W, VB, U, ACT, true, false><<<grid, block, 0, s>>>(p);
    else if (res)
        k_prefill_window<DT, W, VB, U, ACT, false, true><<<grid, block, 0, s>>>(p);
    else
        k_prefill_window<DT, W, VB, U, ACT, false, false><<<grid, block, 0, s>>>(p);
    return cudaGetLastError();
}

template <int DT, int W>
cudaError_t launch_w(const CLParams& base, const vc1d_prefill_args& a, int block, cudaStream_t s) {
    const bool mask = a.mask != nullptr, res = a.residual != nullptr;
    const bool act = a.activation == VC1D_ACT_SILU;
    CLParams p = base;
    // bytes of channels per thread: 8 by default (more resident threads), 16 on request
    const int vb = (a.unroll == 16) ? 16 : 8;
    const int eb = Elem<DT>::kBytes;
    p.nslice = a.dim * eb / vb;
    p.total = (long long)a.batch * p.nchunk * p.nslice;
    if constexpr (DT == VC1D_BF16 && W == 4) {
        if (vb == 16)
            return act ? launch_flags<DT, W, 16, true>(p, mask, res, block, s)
                       : launch_flags<DT, W, 16, false>(p, mask, res, block, s);
    }
    p.nslice = a.dim * eb / 8;
    p.total = (long long)a.batch * p.nchunk * p.nslice;
    return act ? launch_flags<DT, W, 8, true>(p, mask, res, block, s)
               : launch_flags<DT, W, 8, false>(p, mask, res, block, s);
}

template <int DT>
cudaError_t launch_dt(const CLParams& p, const vc1d_prefill_args& a, int block, cudaStream_t s) {
    switch (a.width) {
        case 2: return launch_w<DT, 2>(p, a, block, s);
        case 3: return launch_w<DT, 3>(p, a, block, s);
        default: return launch_w<DT, 4>(p, a, block, s);
    }
}

}  // namespace

cudaError_t launch_prefill_channel_last(const vc1d_prefill_args& a, cudaStream_t s) {
    const int eb = elem_bytes(a.dtype);
    CLParams p;
    p.x = reinterpret_cast<const char*>(a.x);
    p.y = reinterpret_cast<char*>(a.y);
    p.res = reinterpret_cast<const char*>(a.residual);
    p.weight = a.weight;
    p.bias = a.bias;
    p.mask = a.mask;
    p.init = reinterpret_cast<const char*>(a.initial_state);
    p.fstate = reinterpret_cast<char*>(a.final_state);
    p.sxb = a.x_stride_b * eb;
    p.sxt = a.x_stride_t * eb;
    p.syb = a.y_stride_b * eb;
    p.syt = a.y_stride_t * eb;
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
    p.mask_dtype = a.mask_dtype;
    p.skip = (a.mask != nullptr && a.skip_masked_loads) ? 1 : 0;
    p.init_len = a.init_len;
    p.state_len = a.state_len;

    int block = a.block_threads > 0 ? a.block_threads : 256;
    if (block > 256) block = 256;
    block = (block + 31) / 32 * 32;

    // Rows per thread: long enough to amortise the weight load and the halo re-read, short
    // enough that the grid has several waves of CTAs on every SM.
    int R = a.rows_per_thread;
    if (R <= 0) {
        R = 64;
        const long long nslice = (long long)a.dim * eb / 8;
        const long long want_threads = (long long)sm_count() * 1024 * 6;
        while (R > 8 && (long long)a.batch * nslice * ((a.seqlen + R - 1) / R) < want_threads) R /= 2;
    }
    if (R > a.seqlen) R = a.seqlen;
    p.R = R;
    p.nchunk = (a.seqlen + R - 1) / R;
    p.nslice = 0;
    p.total = 0;
    note_launch("channel_last");
    switch (a.dtype) {
        case VC1D_F32: return launch_dt<VC1D_F32>(p, a, block, s);
        case VC1D_BF16: return launch_dt<VC1D_BF16>(p, a, block, s);
        default: return launch_dt<VC1D_F16>(p, a, block, s);
    }
}

}  // namespace vc1d
