// Prefill kernel for the channel-last layout the Canon layers pass
// (x.transpose(1,2) of a contiguous [B,T,D] tensor, reference model/model.py:459-466).
//
// Work unit: one thread owns one 128-bit channel vector (8 bf16 / 4 fp32 channels) and a
// chunk of consecutive time rows.  Units are numbered with the channel vector fastest, so
// a warp reads 512 contiguous bytes per row and no lane idles whatever dim is.  Weights
// and bias of the owned channels live in registers as fp32 pairs; the (W-1)-row history
// is a register sliding window, seeded by re-reading the W-1 rows before the chunk (they
// come from L1/L2: another thread of the grid streams them from HBM).  Loads are issued
// U rows at a time before any arithmetic so that every thread keeps U*16 bytes in flight.
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
    int nvec, nchunk, R;
    int act;
    int mask_dtype;
    int skip;
    int init_len, state_len;
    int w_fast;  // weights contiguous [D,W], same dtype as x, 16-byte aligned
};

template <int DT, int W>
__device__ __forceinline__ void load_weights(const CLParams& p, int d0,
                                             float2 (&wp)[W][Pack<DT>::kPairs],
                                             float2 (&bp)[Pack<DT>::kPairs]) {
    using E = Elem<DT>;
    using T = typename E::type;
    constexpr int VEC = E::kVec;
    constexpr int PAIRS = Pack<DT>::kPairs;
    float wf[VEC * W];
    if (p.w_fast) {
        // VEC channels x W taps are VEC*W consecutive elements = W 128-bit vectors
        const char* base = reinterpret_cast<const char*>(p.weight) + (long long)d0 * W * E::kBytes;
#pragma unroll
        for (int j = 0; j < W; ++j) {
            const uint4 v = ld_vec(base + j * 16);
            float2 f[PAIRS];
            Pack<DT>::unpack(v, f);
#pragma unroll
            for (int q = 0; q < PAIRS; ++q) {
                wf[j * VEC + 2 * q] = f[q].x;
                wf[j * VEC + 2 * q + 1] = f[q].y;
            }
        }
    } else {
#pragma unroll
        for (int c = 0; c < VEC; ++c) {
#pragma unroll
            for (int w = 0; w < W; ++w) {
                const long long idx = (long long)(d0 + c) * p.wsd + (long long)w * p.wsw;
                wf[c * W + w] = (p.wdtype == VC1D_F32)
                                    ? __ldg(reinterpret_cast<const float*>(p.weight) + idx)
                                    : E::to_float(__ldg(reinterpret_cast<const T*>(p.weight) + idx));
            }
        }
    }
#pragma unroll
    for (int w = 0; w < W; ++w) {
#pragma unroll
        for (int q = 0; q < PAIRS; ++q) {
            wp[w][q] = make_float2(wf[(2 * q) * W + w], wf[(2 * q + 1) * W + w]);
        }
    }
    if (p.bias != nullptr) {
        float bf[VEC];
#pragma unroll
        for (int c = 0; c < VEC; ++c) {
            bf[c] = (p.wdtype == VC1D_F32)
                        ? __ldg(reinterpret_cast<const float*>(p.bias) + d0 + c)
                        : E::to_float(__ldg(reinterpret_cast<const T*>(p.bias) + d0 + c));
        }
#pragma unroll
        for (int q = 0; q < PAIRS; ++q) bp[q] = make_float2(bf[2 * q], bf[2 * q + 1]);
    } else {
#pragma unroll
        for (int q = 0; q < PAIRS; ++q) bp[q] = make_float2(0.f, 0.f);
    }
}

// raw 128-bit row -> fp32 pairs, with the multiplicative mask of the reference
// (x * mask, rounded to the I/O dtype) when the mask value is not exactly 1
template <int DT, bool MASK>
__device__ __forceinline__ void decode_row(const uint4& raw, float mk,
                                           float2 (&f)[Pack<DT>::kPairs]) {
    Pack<DT>::unpack(raw, f);
    if (MASK) {
        if (mk != 1.0f) {
            const float2 m2 = make_float2(mk, mk);
#pragma unroll
            for (int q = 0; q < Pack<DT>::kPairs; ++q) f[q] = Pack<DT>::round_trip(mul2(f[q], m2));
        }
    }
}

template <int DT>
__device__ __forceinline__ void store_channel_column(char* fstate, long long row0, int L, int j,
                                                     const uint4& raw) {
    // fstate is [B, D, L] contiguous; this thread owns channels row0 .. row0+VEC-1
    using T = typename Elem<DT>::type;
    constexpr int VEC = Elem<DT>::kVec;
    T vals[VEC];
    *reinterpret_cast<uint4*>(vals) = raw;
    T* out = reinterpret_cast<T*>(fstate);
#pragma unroll
    for (int c = 0; c < VEC; ++c) out[(row0 + c) * L + j] = vals[c];
}

template <int DT>
__device__ __forceinline__ uint4 load_init_column(const char* init, long long row0, int init_len,
                                                  int col) {
    using T = typename Elem<DT>::type;
    constexpr int VEC = Elem<DT>::kVec;
    T vals[VEC];
    const T* in = reinterpret_cast<const T*>(init);
#pragma unroll
    for (int c = 0; c < VEC; ++c) vals[c] = in[(row0 + c) * init_len + col];
    return *reinterpret_cast<uint4*>(vals);
}

template <int DT, int W, int U, bool MASK, bool RES>
__global__ void __launch_bounds__(256) k_prefill_channel_last(const CLParams p) {
    using E = Elem<DT>;
    using PK = Pack<DT>;
    constexpr int VEC = E::kVec;
    constexpr int PAIRS = PK::kPairs;
    constexpr int H = W - 1;

    const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= p.total) return;
    const int lane = (int)(g % p.nvec);
    const long long q = g / p.nvec;
    const int chunk = (int)(q % p.nchunk);
    const int b = (int)(q / p.nchunk);
    const int d0 = lane * VEC;
    const int t0 = chunk * p.R;
    const int t1 = min(t0 + p.R, p.T);

    float2 wp[W][PAIRS];
    float2 bp[PAIRS];
    load_weights<DT, W>(p, d0, wp, bp);

    const char* xb = p.x + (long long)b * p.sxb + (long long)d0 * E::kBytes;
    char* yb = p.y + (long long)b * p.syb + (long long)d0 * E::kBytes;
    const char* rb = RES ? p.res + (long long)b * p.srb + (long long)d0 * E::kBytes : nullptr;
    const long long mrow = (long long)b * p.smb;
    const long long row0 = (long long)b * p.D + d0;  // first owned row of a [B*D, L] state

    // ---- history: the W-1 rows before the chunk --------------------------------------
    float2 hist[H][PAIRS];
#pragma unroll
    for (int j = 0; j < H; ++j) {
        const int t = t0 - H + j;
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        float mk = 1.0f;
        if (t >= 0) {
            if (MASK) mk = load_mask(p.mask, mrow + (long long)t * p.smt, p.mask_dtype);
            if (!MASK || !p.skip || mk != 0.0f) raw = ld_vec(xb + (long long)t * p.sxt);
        } else if (p.init != nullptr) {
            raw = load_init_column<DT>(p.init, row0, p.init_len, p.init_len + t);
        }
        decode_row<DT, MASK>(raw, mk, hist[j]);
    }

    // ---- main sweep ------------------------------------------------------------------
    for (int tb = t0; tb < t1; tb += U) {
        uint4 raw[U];
        uint4 rres[RES ? U : 1];
        float mk[U];
#pragma unroll
        for (int k = 0; k < U; ++k) {
            const int t = tb + k;
            const bool in = t < t1;
            mk[k] = 1.0f;
            if (MASK) mk[k] = in ? load_mask(p.mask, mrow + (long long)t * p.smt, p.mask_dtype) : 0.0f;
            const bool need = in && (!MASK || !p.skip || mk[k] != 0.0f);
            raw[k] = make_uint4(0u, 0u, 0u, 0u);
            if (need) raw[k] = ld_vec(xb + (long long)t * p.sxt);
            if (RES) {
                rres[k] = make_uint4(0u, 0u, 0u, 0u);
                if (in) rres[k] = ld_vec(rb + (long long)t * p.srt);
            }
        }
#pragma unroll
        for (int k = 0; k < U; ++k) {
            const int t = tb + k;
            if (t < t1) {
                float2 cur[PAIRS];
                decode_row<DT, MASK>(raw[k], mk[k], cur);
                float2 acc[PAIRS];
#pragma unroll
                for (int qq = 0; qq < PAIRS; ++qq) {
                    acc[qq] = bp[qq];
#pragma unroll
                    for (int w = 0; w < H; ++w) acc[qq] = fma2(wp[w][qq], hist[w][qq], acc[qq]);
                    acc[qq] = fma2(wp[H][qq], cur[qq], acc[qq]);
                    if (p.act) acc[qq] = silu2<E::kPreciseSilu>(acc[qq]);
                }
                if (RES) {
                    // same roundings as the unfused `x + y`: y rounded to the I/O dtype, then the sum
                    float2 rr[PAIRS];
                    PK::unpack(rres[k], rr);
#pragma unroll
                    for (int qq = 0; qq < PAIRS; ++qq) acc[qq] = add2(PK::round_trip(acc[qq]), rr[qq]);
                }
                st_vec_stream(yb + (long long)t * p.syt, PK::pack(acc));
#pragma unroll
                for (int w = 0; w + 1 < H; ++w) {
#pragma unroll
                    for (int qq = 0; qq < PAIRS; ++qq) hist[w][qq] = hist[w + 1][qq];
                }
                if (H > 0) {
#pragma unroll
                    for (int qq = 0; qq < PAIRS; ++qq) hist[H - 1][qq] = cur[qq];
                }
            }
        }
    }

    // ---- final state: right-aligned last state_len masked inputs ------------------------
    if (p.fstate != nullptr && t1 == p.T) {
        const int L = p.state_len;
        for (int j = 0; j < L; ++j) {
            const int t = p.T - L + j;
            uint4 raw = make_uint4(0u, 0u, 0u, 0u);
            if (t >= 0) {
                raw = ld_vec(xb + (long long)t * p.sxt);
                if (MASK) {
                    const float mk = load_mask(p.mask, mrow + (long long)t * p.smt, p.mask_dtype);
                    if (mk != 1.0f) {
                        float2 f[PAIRS];
                        PK::unpack(raw, f);
                        const float2 m2 = make_float2(mk, mk);
#pragma unroll
                        for (int qq = 0; qq < PAIRS; ++qq) f[qq] = mul2(f[qq], m2);
                        raw = PK::pack(f);
                    }
                }
            } else if (p.init != nullptr && p.init_len + t >= 0) {
                raw = load_init_column<DT>(p.init, row0, p.init_len, p.init_len + t);
            }
            store_channel_column<DT>(p.fstate, row0, L, j, raw);
        }
    }
}

template <int DT, int W, int U>
cudaError_t launch_u(const CLParams& p, bool mask, bool res, int block, cudaStream_t s) {
    const long long blocks = (p.total + block - 1) / block;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    const dim3 grid((unsigned)blocks);
    if (mask && res)
        k_prefill_channel_last<DT, W, U, true, true><<<grid, block, 0, s>>>(p);
    else if (mask)
        k_prefill_channel_last<DT, W, U, true, false><<<grid, block, 0, s>>>(p);
    else if (res)
        k_prefill_channel_last<DT, W, U, false, true><<<grid, block, 0, s>>>(p);
    else
        k_prefill_channel_last<DT, W, U, false, false><<<grid, block, 0, s>>>(p);
    return cudaGetLastError();
}

template <int DT, int W>
cudaError_t launch_w(const CLParams& p, bool mask, bool res, int block, int unroll, cudaStream_t s) {
    if (unroll == 4) return launch_u<DT, W, 4>(p, mask, res, block, s);
    return launch_u<DT, W, 8>(p, mask, res, block, s);
}

template <int DT>
cudaError_t launch_dt(const CLParams& p, int width, bool mask, bool res, int block, int unroll,
                      cudaStream_t s) {
    switch (width) {
        case 2: return launch_w<DT, 2>(p, mask, res, block, unroll, s);
        case 3: return launch_w<DT, 3>(p, mask, res, block, unroll, s);
        default: return launch_w<DT, 4>(p, mask, res, block, unroll, s);
    }
}

}  // namespace

cudaError_t launch_prefill_channel_last(const vc1d_prefill_args& a, cudaStream_t s) {
    const int eb = elem_bytes(a.dtype);
    const int vec = 16 / eb;
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
    p.nvec = a.dim / vec;
    p.act = a.activation;
    p.mask_dtype = a.mask_dtype;
    p.skip = (a.mask != nullptr && a.skip_masked_loads) ? 1 : 0;
    p.init_len = a.init_len;
    p.state_len = a.state_len;
    p.w_fast = (a.wdtype == a.dtype && a.w_stride_w == 1 && a.w_stride_d == a.width &&
                (reinterpret_cast<uintptr_t>(a.weight) & 15u) == 0)
                   ? 1
                   : 0;

    int block = a.block_threads > 0 ? a.block_threads : 256;
    if (block > 256) block = 256;
    block = (block + 31) / 32 * 32;

    // Rows per thread: long enough to amortise the weight load and the halo re-read,
    // short enough that the grid has several waves of CTAs on every SM.
    int R = a.rows_per_thread;
    if (R <= 0) {
        R = 32;
        const long long want_threads = (long long)sm_count() * 2048 * 4;
        while (R > 8 && (long long)a.batch * p.nvec * ((a.seqlen + R - 1) / R) < want_threads) R /= 2;
    }
    if (R > a.seqlen) R = a.seqlen;
    p.R = R;
    p.nchunk = (a.seqlen + R - 1) / R;
    p.total = (long long)a.batch * p.nchunk * p.nvec;

    const bool mask = a.mask != nullptr;
    const bool res = a.residual != nullptr;
    const int unroll = (a.unroll == 4) ? 4 : 8;
    note_launch("channel_last");
    switch (a.dtype) {
        case VC1D_F32: return launch_dt<VC1D_F32>(p, a.width, mask, res, block, unroll, s);
        case VC1D_BF16: return launch_dt<VC1D_BF16>(p, a.width, mask, res, block, unroll, s);
        default: return launch_dt<VC1D_F16>(p, a.width, mask, res, block, unroll, s);
    }
}

}  // namespace vc1d
