// Scalar prefill kernel for every case the vectorised kernels decline: arbitrary strides,
// dim or seqlen not a multiple of the vector width, unaligned pointers.  One thread per
// output element, indexed so that consecutive threads walk the unit-stride dimension of x.
// Supports every fused option with the same semantics as the channel-last kernel.
#include "vc1d_common.cuh"
#include "vc1d_internal.h"

namespace vc1d {
namespace {

struct GParams {
    const void* x;
    void* y;
    const void* res;
    const void* weight;
    const void* bias;
    const void* mask;
    const void* init;
    const int* seq;  // sequence id of every time step (packed variable-length rows), or NULL
    void* fstate;
    long long ssb, sst;
    long long sxb, sxd, sxt;  // elements
    long long syb, syd, syt;
    long long srb, srd, srt;
    long long smb, smt;
    long long wsd, wsw;
    long long total;
    int wdtype;
    int B, D, T, W;
    int act;
    int mask_dtype;
    int skip;
    int init_len, state_len;
    int time_fastest;
};

template <int DT>
__device__ __forceinline__ float masked_input(const GParams& p, const typename Elem<DT>::type* x,
                                              long long b, int d, int t) {
    using E = Elem<DT>;
    using T = typename E::type;
    if (t < 0) {
        if (p.init != nullptr && p.init_len + t >= 0) {
            const T* in = reinterpret_cast<const T*>(p.init);
            return E::to_float(in[(b * p.D + d) * p.init_len + (p.init_len + t)]);
        }
        return 0.f;
    }
    float mk = 1.f;
    if (p.mask != nullptr) {
        mk = load_mask(p.mask, b * p.smb + (long long)t * p.smt, p.mask_dtype);
        if (mk == 0.f && p.skip) return 0.f;
    }
    float v = E::to_float(x[b * p.sxb + (long long)d * p.sxd + (long long)t * p.sxt]);
    if (mk != 1.f) v = E::to_float(E::from_float(v * mk));
    return v;
}

template <int DT>
__global__ void __launch_bounds__(256) k_prefill_generic(const GParams p) {
    using E = Elem<DT>;
    using T = typename E::type;
    const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= p.total) return;
    int d, t;
    long long b;
    if (p.time_fastest) {
        t = (int)(g % p.T);
        const long long q = g / p.T;
        d = (int)(q % p.D);
        b = q / p.D;
    } else {
        d = (int)(g % p.D);
        const long long q = g / p.D;
        t = (int)(q % p.T);
        b = q / p.T;
    }
    const T* x = reinterpret_cast<const T*>(p.x);
    T* y = reinterpret_cast<T*>(p.y);

    float acc = 0.f;
    if (p.bias != nullptr) {
        acc = (p.wdtype == VC1D_F32) ? reinterpret_cast<const float*>(p.bias)[d]
                                     : E::to_float(reinterpret_cast<const T*>(p.bias)[d]);
    }
    // packed rows: only the steps right above t that carry its sequence id are taps
    int reach = p.W - 1;
    if (p.seq != nullptr) {
        const int* ids = p.seq + b * p.ssb;
        const int mine = ids[(long long)t * p.sst];
        reach = 0;
        while (reach < p.W - 1 && t - reach - 1 >= 0 && ids[(long long)(t - reach - 1) * p.sst] == mine) ++reach;
    }
    for (int w = 0; w < p.W; ++w) {
        const long long widx = (long long)d * p.wsd + (long long)w * p.wsw;
        const float wv = (p.wdtype == VC1D_F32) ? reinterpret_cast<const float*>(p.weight)[widx]
                                                : E::to_float(reinterpret_cast<const T*>(p.weight)[widx]);
        const int back = p.W - 1 - w;
        if (back > reach) continue;  // the tap lies in another sequence of the same packed row
        acc = fmaf(wv, masked_input<DT>(p, x, b, d, t - back), acc);
    }
    if (p.act) acc = silu1<E::kPreciseSilu>(acc);
    if (p.res != nullptr) {
        const T* r = reinterpret_cast<const T*>(p.res);
        acc = E::to_float(E::from_float(acc)) +
              E::to_float(r[b * p.srb + (long long)d * p.srd + (long long)t * p.srt]);
    }
    y[b * p.syb + (long long)d * p.syd + (long long)t * p.syt] = E::from_float(acc);

    // final state [B, D, L]: column j holds masked input row T-L+j (initial state or zero before row 0)
    if (p.fstate != nullptr) {
        const int L = p.state_len;
        T* fs = reinterpret_cast<T*>(p.fstate) + (b * p.D + d) * L;
        const int j = t - (p.T - L);
        if (j >= 0) {
            T v = x[b * p.sxb + (long long)d * p.sxd + (long long)t * p.sxt];
            if (p.mask != nullptr) {
                const float mk = load_mask(p.mask, b * p.smb + (long long)t * p.smt, p.mask_dtype);
                if (mk != 1.f) v = E::from_float(E::to_float(v) * mk);
            }
            fs[j] = v;
        }
        if (t == 0) {
            for (int jj = 0; jj < L - p.T; ++jj) {
                const int tt = p.T - L + jj;  // negative
                T v = E::from_float(0.f);
                if (p.init != nullptr && p.init_len + tt >= 0)
                    v = reinterpret_cast<const T*>(p.init)[(b * p.D + d) * p.init_len + (p.init_len + tt)];
                fs[jj] = v;
            }
        }
    }
}

}  // namespace

cudaError_t launch_prefill_generic(const vc1d_prefill_args& a, cudaStream_t s) {
    GParams p;
    p.x = a.x;
    p.y = a.y;
    p.res = a.residual;
    p.weight = a.weight;
    p.bias = a.bias;
    p.mask = a.mask;
    p.init = a.initial_state;
    p.seq = a.seq_idx;
    p.ssb = a.seq_stride_b;
    p.sst = a.seq_stride_t;
    p.fstate = a.final_state;
    p.sxb = a.x_stride_b;
    p.sxd = a.x_stride_d;
    p.sxt = a.x_stride_t;
    p.syb = a.y_stride_b;
    p.syd = a.y_stride_d;
    p.syt = a.y_stride_t;
    p.srb = a.r_stride_b;
    p.srd = a.r_stride_d;
    p.srt = a.r_stride_t;
    p.smb = a.mask_stride_b;
    p.smt = a.mask_stride_t;
    p.wsd = a.w_stride_d;
    p.wsw = a.w_stride_w;
    p.wdtype = a.wdtype;
    p.B = a.batch;
    p.D = a.dim;
    p.T = a.seqlen;
    p.W = a.width;
    p.act = a.activation;
    p.mask_dtype = a.mask_dtype;
    p.skip = (a.mask != nullptr && a.skip_masked_loads) ? 1 : 0;
    p.init_len = a.init_len;
    p.state_len = a.state_len;
    p.time_fastest = (a.x_stride_t == 1 && a.x_stride_d != 1) ? 1 : 0;
    p.total = (long long)a.batch * a.dim * a.seqlen;
    const int block = 256;
    const long long blocks = (p.total + block - 1) / block;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    note_launch("generic");
    const dim3 grid((unsigned)blocks);
    switch (a.dtype) {
        case VC1D_F32: k_prefill_generic<VC1D_F32><<<grid, block, 0, s>>>(p); break;
        case VC1D_BF16: k_prefill_generic<VC1D_BF16><<<grid, block, 0, s>>>(p); break;
        default: k_prefill_generic<VC1D_F16><<<grid, block, 0, s>>>(p); break;
    }
    return cudaGetLastError();
}

}  // namespace vc1d
