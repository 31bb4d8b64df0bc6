// Backward of one decode step (causal_conv1d_update).
//
//     win = last W entries of [conv_state | x] (or the circular history);  pre = bias + win . weight
//     g = dy * silu'(pre);   dx = weight[W-1] * g (+ dy with residual);   dstate[col of tap w] = weight[w] * g
//     dweight[d,w] += sum_b win[w] * g;   dbias[d] += sum_b g
// (reference: causal-conv1d-mps/causal_conv1d_mps/causal_conv1d.metal:1738-1845, which adds every
// product to dweight with a global atomic per (sequence, channel, tap)).
//
// One thread owns one channel and walks a strided share of the batch, so its dweight / dbias sums
// stay in registers and reach memory with W + 1 atomic adds per thread.  Training through single
// decode steps is rare; this kernel is written for any strides, not tuned.
#include "vc1d_common.cuh"
#include "vc1d_internal.h"

namespace vc1d {
namespace {

struct UBParams {
    const void* x;
    const void* state;
    const void* dy;
    void* dx;
    void* dstate;
    const void* weight;
    const void* bias;
    const int32_t* seqlens;
    float* dweight;
    float* dbias;
    long long sxb, sxd, sgb, sgd, sdb, sdd;
    long long ssb, ssd, ssl;
    long long wsd, wsw;
    int wdtype;
    int B, D, W, L;
    int act, residual;
};

template <int MODE>
__device__ __forceinline__ float silu_grad_scalar(float z) {
    float s;
    if (MODE == 0) {
        s = 1.0f / (1.0f + expf(-z));
    } else {
        s = rcp_approx(1.0f + ex2_approx(z * -1.4426950408889634f));
    }
    return s * fmaf(z, fmaf(s, -1.0f, 1.0f), 1.0f);
}

template <int DT>
__global__ void __launch_bounds__(128) k_update_bwd(const UBParams p) {
    using E = Elem<DT>;
    using T = typename E::type;
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= p.D) return;
    const int W = p.W, L = p.L;
    const T* x = reinterpret_cast<const T*>(p.x);
    const T* dy = reinterpret_cast<const T*>(p.dy);
    const T* st = reinterpret_cast<const T*>(p.state);
    T* dx = reinterpret_cast<T*>(p.dx);
    T* dst = reinterpret_cast<T*>(p.dstate);

    float wt[4] = {0.f, 0.f, 0.f, 0.f};
    for (int w = 0; w < W; ++w) {
        const long long idx = (long long)d * p.wsd + (long long)w * p.wsw;
        wt[w] = (p.wdtype == VC1D_F32) ? reinterpret_cast<const float*>(p.weight)[idx]
                                       : E::to_float(reinterpret_cast<const T*>(p.weight)[idx]);
    }
    float bv = 0.f;
    if (p.bias != nullptr)
        bv = (p.wdtype == VC1D_F32) ? reinterpret_cast<const float*>(p.bias)[d]
                                    : E::to_float(reinterpret_cast<const T*>(p.bias)[d]);
    float dw[4] = {0.f, 0.f, 0.f, 0.f};
    float db = 0.f;
    for (long long b = blockIdx.y; b < p.B; b += gridDim.y) {
        const T* srow = st + b * p.ssb + (long long)d * p.ssd;
        int pos = 0;
        if (p.seqlens != nullptr) {
            pos = p.seqlens[b] % L;
            if (pos < 0) pos += L;
        }
        // column of the state that tap w (< W-1) reads
        auto col = [&](int w) -> int {
            if (p.seqlens == nullptr) return L + 1 - W + w;
            int h = (pos - (W - 1 - w)) % L;
            return h < 0 ? h + L : h;
        };
        const float xv = E::to_float(x[b * p.sxb + (long long)d * p.sxd]);
        float win[4] = {0.f, 0.f, 0.f, 0.f};
        for (int w = 0; w < W - 1; ++w) win[w] = E::to_float(srow[(long long)col(w) * p.ssl]);
        win[W - 1] = xv;
        const float gy = E::to_float(dy[b * p.sgb + (long long)d * p.sgd]);
        float g = gy;
        if (p.act) {
            float pre = bv;
            for (int w = 0; w < W; ++w) pre = fmaf(wt[w], win[w], pre);
            g *= silu_grad_scalar<E::kPreciseSilu ? 0 : 1>(pre);
        }
        float dxv = wt[W - 1] * g;
        if (p.residual) dxv += gy;
        dx[b * p.sdb + (long long)d * p.sdd] = E::from_float(dxv);
        if (dst != nullptr) {
            T* drow = dst + (b * p.D + d) * (long long)L;
            for (int l = 0; l < L; ++l) drow[l] = E::from_float(0.f);
            for (int w = 0; w < W - 1; ++w) drow[col(w)] = E::from_float(wt[w] * g);
        }
        for (int w = 0; w < W; ++w) dw[w] = fmaf(win[w], g, dw[w]);
        db += g;
    }
    if (p.dweight != nullptr)
        for (int w = 0; w < W; ++w) atomicAdd(p.dweight + (long long)d * W + w, dw[w]);
    if (p.dbias != nullptr) atomicAdd(p.dbias + d, db);
}

}  // namespace

cudaError_t launch_update_bwd(const vc1d_update_bwd_args& a, cudaStream_t s) {
    UBParams p;
    p.x = a.x; p.state = a.conv_state; p.dy = a.dy; p.dx = a.dx; p.dstate = a.dstate;
    p.weight = a.weight; p.bias = a.bias; p.seqlens = a.cache_seqlens;
    p.dweight = a.dweight; p.dbias = a.dbias;
    p.sxb = a.x_stride_b; p.sxd = a.x_stride_d;
    p.sgb = a.dy_stride_b; p.sgd = a.dy_stride_d;
    p.sdb = a.dx_stride_b; p.sdd = a.dx_stride_d;
    p.ssb = a.s_stride_b; p.ssd = a.s_stride_d; p.ssl = a.s_stride_l;
    p.wsd = a.w_stride_d; p.wsw = a.w_stride_w;
    p.wdtype = a.wdtype;
    p.B = a.batch; p.D = a.dim; p.W = a.width; p.L = a.state_len;
    p.act = a.activation == VC1D_ACT_SILU;
    p.residual = a.residual != 0;
    const dim3 block(128);
    // enough batch slices to fill the GPU, few enough that each thread amortises its atomics
    const int dblocks = (a.dim + 127) / 128;
    int slices = (sm_count() * 8 + dblocks - 1) / dblocks;
    if (slices > a.batch) slices = a.batch;
    if (slices < 1) slices = 1;
    if (slices > 65535) slices = 65535;
    note_launch("update_bwd");
    const dim3 grid((unsigned)dblocks, (unsigned)slices);
    switch (a.dtype) {
        case VC1D_F32: k_update_bwd<VC1D_F32><<<grid, block, 0, s>>>(p); break;
        case VC1D_BF16: k_update_bwd<VC1D_BF16><<<grid, block, 0, s>>>(p); break;
        default: k_update_bwd<VC1D_F16><<<grid, block, 0, s>>>(p); break;
    }
    return cudaGetLastError();
}

}  // namespace vc1d
