// Prefill kernel for time-contiguous input ([B,D,T] contiguous, the layout of the
// reference's stand-alone forward, causal-conv1d-mps/causal_conv1d_mps/__init__.py:81-151
// and causal_conv1d.metal:130-180).
//
// Work unit: one warp owns K*32 consecutive 128-bit vectors of one (batch, channel) row, so
// the weights of the row are four broadcast scalars and each load instruction of the warp
// covers 512 contiguous bytes.  The W-1 elements before a vector come from the lane to the
// left by shuffle; lane 0 takes them from lane 31 of the previous step, or re-reads the
// vector before the segment.
#include "vc1d_common.cuh"
#include "vc1d_internal.h"

namespace vc1d {
namespace {

struct TMParams {
    const char* x;
    char* y;
    const void* weight;
    const void* bias;
    long long sxb, sxd;  // bytes
    long long syb, syd;
    long long wsd, wsw;  // elements
    long long nwarps;
    int wdtype;
    int D, T;
    int nvt;   // vectors per row
    int nseg;  // warp segments per row
    int act;
};

constexpr int kVecsPerLane = 4;

template <int DT, int W>
__global__ void __launch_bounds__(256) k_prefill_time_major(const TMParams p) {
    using E = Elem<DT>;
    using T = typename E::type;
    using PK = Pack<DT>;
    constexpr int VEC = E::kVec;
    constexpr int PAIRS = PK::kPairs;
    constexpr int H = W - 1;
    constexpr int K = kVecsPerLane;

    const long long wg = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (wg >= p.nwarps) return;  // whole warps leave together
    const int lane = threadIdx.x & 31;
    const int seg = (int)(wg % p.nseg);
    const long long row = wg / p.nseg;
    const int d = (int)(row % p.D);
    const long long b = row / p.D;

    float wv[W];
#pragma unroll
    for (int w = 0; w < W; ++w) {
        const long long idx = (long long)d * p.wsd + (long long)w * p.wsw;
        wv[w] = (p.wdtype == VC1D_F32) ? __ldg(reinterpret_cast<const float*>(p.weight) + idx)
                                       : E::to_float(__ldg(reinterpret_cast<const T*>(p.weight) + idx));
    }
    float bv = 0.f;
    if (p.bias != nullptr) {
        bv = (p.wdtype == VC1D_F32) ? __ldg(reinterpret_cast<const float*>(p.bias) + d)
                                    : E::to_float(__ldg(reinterpret_cast<const T*>(p.bias) + d));
    }

    const char* xr = p.x + b * p.sxb + (long long)d * p.sxd;
    char* yr = p.y + b * p.syb + (long long)d * p.syd;
    const int j0 = seg * 32 * K;

    uint4 raw[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
        const int j = j0 + k * 32 + lane;
        raw[k] = make_uint4(0u, 0u, 0u, 0u);
        if (j < p.nvt) raw[k] = ld_vec_stream(xr + (long long)j * 16);
    }
    uint4 carry = make_uint4(0u, 0u, 0u, 0u);
    if (lane == 0 && j0 > 0) carry = ld_vec(xr + (long long)(j0 - 1) * 16);

#pragma unroll
    for (int k = 0; k < K; ++k) {
        const int j = j0 + k * 32 + lane;
        // vector to the left of mine
        uint4 prev;
        prev.x = 0u;
        prev.y = __shfl_up_sync(0xffffffffu, raw[k].y, 1);
        prev.z = __shfl_up_sync(0xffffffffu, raw[k].z, 1);
        prev.w = __shfl_up_sync(0xffffffffu, raw[k].w, 1);
        if (lane == 0) prev = carry;
        // lane 31's vector becomes lane 0's left neighbour at the next step
        uint4 nxt;
        nxt.x = 0u;
        nxt.y = __shfl_sync(0xffffffffu, raw[k].y, 31);
        nxt.z = __shfl_sync(0xffffffffu, raw[k].z, 31);
        nxt.w = __shfl_sync(0xffffffffu, raw[k].w, 31);
        carry = nxt;

        if (j < p.nvt) {
            float2 pf[PAIRS], cf[PAIRS];
            PK::unpack(prev, pf);
            PK::unpack(raw[k], cf);
            float xx[VEC + H];
#pragma unroll
            for (int i = 0; i < H; ++i) {
                const int e = VEC - H + i;  // element of the previous vector
                xx[i] = (e & 1) ? pf[e >> 1].y : pf[e >> 1].x;
            }
#pragma unroll
            for (int i = 0; i < VEC; ++i) xx[H + i] = (i & 1) ? cf[i >> 1].y : cf[i >> 1].x;
            float2 out[PAIRS];
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                float acc = bv;
#pragma unroll
                for (int w = 0; w < W; ++w) acc = fmaf(wv[w], xx[i + w], acc);
                if (p.act) acc = silu1<E::kPreciseSilu>(acc);
                if (i & 1)
                    out[i >> 1].y = acc;
                else
                    out[i >> 1].x = acc;
            }
            st_vec_stream(yr + (long long)j * 16, PK::pack(out));
        }
    }
}

template <int DT>
cudaError_t launch_dt(const TMParams& p, int width, int block, cudaStream_t s) {
    const long long threads = p.nwarps * 32;
    const long long blocks = (threads + block - 1) / block;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    const dim3 grid((unsigned)blocks);
    switch (width) {
        case 2: k_prefill_time_major<DT, 2><<<grid, block, 0, s>>>(p); break;
        case 3: k_prefill_time_major<DT, 3><<<grid, block, 0, s>>>(p); break;
        default: k_prefill_time_major<DT, 4><<<grid, block, 0, s>>>(p); break;
    }
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_prefill_time_major(const vc1d_prefill_args& a, cudaStream_t s) {
    const int eb = elem_bytes(a.dtype);
    const int vec = 16 / eb;
    TMParams p;
    p.x = reinterpret_cast<const char*>(a.x);
    p.y = reinterpret_cast<char*>(a.y);
    p.weight = a.weight;
    p.bias = a.bias;
    p.sxb = a.x_stride_b * eb;
    p.sxd = a.x_stride_d * eb;
    p.syb = a.y_stride_b * eb;
    p.syd = a.y_stride_d * eb;
    p.wsd = a.w_stride_d;
    p.wsw = a.w_stride_w;
    p.wdtype = a.wdtype;
    p.D = a.dim;
    p.T = a.seqlen;
    p.nvt = a.seqlen / vec;
    p.nseg = (p.nvt + 32 * kVecsPerLane - 1) / (32 * kVecsPerLane);
    p.nwarps = (long long)a.batch * a.dim * p.nseg;
    p.act = a.activation;
    int block = a.block_threads > 0 ? a.block_threads : 256;
    if (block > 256) block = 256;
    block = (block + 31) / 32 * 32;
    note_launch("time_major");
    switch (a.dtype) {
        case VC1D_F32: return launch_dt<VC1D_F32>(p, a.width, block, s);
        case VC1D_BF16: return launch_dt<VC1D_BF16>(p, a.width, block, s);
        default: return launch_dt<VC1D_F16>(p, a.width, block, s);
    }
}

}  // namespace vc1d
