// Decode kernels: one new token per sequence against the rolling conv_state
// (reference call site model/model.py:305-311, PyTorch restatement model/model.py:372-398,
// circular variant causal_conv1d.metal:586-664).
//
// Vectorised kernel: one thread owns one 128-bit vector of channels (8 bf16 / 4 fp32).
// conv_state is [B, D, L] with L innermost, so the state of those channels is L
// consecutive 128-bit vectors: the thread reads them, shifts every channel's window left
// by one element in registers, appends x and writes the L vectors back -- state read,
// shift and write-back in one pass, the state elements moved as raw bits (no float round
// trip), y accumulated in fp32.
#include "vc1d_common.cuh"
#include "vc1d_internal.h"

namespace vc1d {
namespace {

struct UParams {
    const char* x;
    char* y;
    char* state;
    const void* weight;
    const void* bias;
    const int32_t* seqlens;
    long long sxb, sxd;  // elements
    long long syb, syd;
    long long ssb, ssd, ssl;
    long long wsd, wsw;
    long long total;
    int wdtype;
    int B, D, W, L;
    int nvec;
    int act;
    int residual;
    int nb;      // sequences one thread of the vectorised kernel walks
    int w_fast;  // weights contiguous [D,W] (and bias) in the I/O dtype, 16-byte aligned
    int vec;     // (several problems in one launch) this problem takes the vectorised code
};

template <int DT, int W, int L>
__device__ __forceinline__ void update_vec_body(const UParams& p, unsigned block) {
    using E = Elem<DT>;
    using T = typename E::type;
    using PK = Pack<DT>;
    constexpr int VEC = E::kVec;
    constexpr int UB = 2;  // sequences in flight per thread
    const long long g = (long long)block * blockDim.x + threadIdx.x;
    if (g >= p.total) return;
    const int lane = (int)(g % p.nvec);
    const long long grp = g / p.nvec;
    const int d0 = lane * VEC;

    // weights and bias of the owned channels, once per thread: the thread then walks nb sequences
    float wf[VEC][W];
    float bf[VEC];
    if (p.w_fast) {
        // VEC channels x W taps are VEC*W consecutive elements = W 128-bit vectors
        float flat[VEC * W];
        const char* base = reinterpret_cast<const char*>(p.weight) + (long long)d0 * W * E::kBytes;
#pragma unroll
        for (int j = 0; j < W; ++j) {
            float2 f[PK::kPairs];
            PK::unpack(ld_vec(base + j * 16), f);
#pragma unroll
            for (int q = 0; q < PK::kPairs; ++q) {
                flat[j * VEC + 2 * q] = f[q].x;
                flat[j * VEC + 2 * q + 1] = f[q].y;
            }
        }
#pragma unroll
        for (int c = 0; c < VEC; ++c)
#pragma unroll
            for (int w = 0; w < W; ++w) wf[c][w] = flat[c * W + w];
    } else {
#pragma unroll
        for (int c = 0; c < VEC; ++c) {
#pragma unroll
            for (int w = 0; w < W; ++w) {
                const long long idx = (long long)(d0 + c) * p.wsd + (long long)w * p.wsw;
                wf[c][w] = (p.wdtype == VC1D_F32) ? __ldg(reinterpret_cast<const float*>(p.weight) + idx)
                                                  : E::to_float(__ldg(reinterpret_cast<const T*>(p.weight) + idx));
            }
        }
    }
#pragma unroll
    for (int c = 0; c < VEC; ++c) bf[c] = 0.f;
    if (p.bias != nullptr) {
        if (p.w_fast) {
            float2 f[PK::kPairs];
            PK::unpack(ld_vec(reinterpret_cast<const char*>(p.bias) + (long long)d0 * E::kBytes), f);
#pragma unroll
            for (int q = 0; q < PK::kPairs; ++q) {
                bf[2 * q] = f[q].x;
                bf[2 * q + 1] = f[q].y;
            }
        } else {
#pragma unroll
            for (int c = 0; c < VEC; ++c)
                bf[c] = (p.wdtype == VC1D_F32) ? __ldg(reinterpret_cast<const float*>(p.bias) + d0 + c)
                                               : E::to_float(__ldg(reinterpret_cast<const T*>(p.bias) + d0 + c));
        }
    }

    const long long b0 = grp * p.nb;
    const long long b1 = (b0 + p.nb < p.B) ? b0 + p.nb : p.B;
    for (long long bb = b0; bb < b1; bb += UB) {
        // issue every load first
        T st[UB][VEC * L];
        T xv[UB][VEC];
#pragma unroll
        for (int u = 0; u < UB; ++u) {
            if (bb + u < b1) {
                const char* sp = p.state + ((bb + u) * p.ssb + (long long)d0 * L) * E::kBytes;
#pragma unroll
                for (int j = 0; j < L; ++j)
                    reinterpret_cast<uint4*>(st[u])[j] = *reinterpret_cast<const uint4*>(sp + j * 16);
                *reinterpret_cast<uint4*>(xv[u]) = ld_vec(p.x + ((bb + u) * p.sxb + d0) * E::kBytes);
            }
        }
#pragma unroll
        for (int u = 0; u < UB; ++u) {
            if (bb + u < b1) {
                T ns[VEC * L];
                T yv[VEC];
#pragma unroll
                for (int c = 0; c < VEC; ++c) {
                    // cat = [state | x]; taps are cat[L+1-W .. L]
                    float acc = bf[c];
#pragma unroll
                    for (int w = 0; w < W; ++w) {
                        const int i = L + 1 - W + w;
                        const float v = (i < L) ? E::to_float(st[u][c * L + i]) : E::to_float(xv[u][c]);
                        acc = fmaf(wf[c][w], v, acc);
                    }
                    if (p.act) acc = silu1<E::kPreciseSilu>(acc);
                    if (p.residual) acc = E::to_float(E::from_float(acc)) + E::to_float(xv[u][c]);
                    yv[c] = E::from_float(acc);
#pragma unroll
                    for (int j = 0; j + 1 < L; ++j) ns[c * L + j] = st[u][c * L + j + 1];
                    ns[c * L + L - 1] = xv[u][c];
                }
                char* spw = p.state + ((bb + u) * p.ssb + (long long)d0 * L) * E::kBytes;
#pragma unroll
                for (int j = 0; j < L; ++j)
                    *reinterpret_cast<uint4*>(spw + j * 16) = reinterpret_cast<const uint4*>(ns)[j];
                st_vec(p.y + ((bb + u) * p.syb + d0) * E::kBytes, *reinterpret_cast<const uint4*>(yv));
            }
        }
    }
}

template <int DT, int W, int L>
__global__ void __launch_bounds__(256, 2) k_update_vec(const UParams p) {
    // Launched with programmatic stream serialization: consecutive decode steps depend on each other
    // through conv_state, so every thread waits for the previous kernel before its first access,
    // while the launch itself and the scheduling of the CTAs overlap the previous step's tail.
    griddep_wait();
    griddep_launch_dependents();
    update_vec_body<DT, W, L>(p, blockIdx.x);
}

// One channel per lane, for states whose state_len columns of one channel are one or two 128-bit
// vectors (state_len 8 in bf16 / fp16, 4 or 8 in fp32: what the reference's PyTorch and Metal
// branches keep, model/model.py:286 and 541).  Consecutive lanes own consecutive channels, so the
// state of a warp's 32 channels is 512 (or 1024) contiguous bytes: every state access is one fully
// coalesced 128-bit load or store per lane, x and y are one element per lane.  The window moves as
// raw bits.  Shifting state: the vector is shifted by one element and x appended.  Circular state
// (cache_seqlens, causal_conv1d.metal:586-664): the history columns are picked out of the vector by
// position, x replaces the column at cache_seqlens[b] % state_len, and the vector is written back
// whole (the partial sector a 2-byte store would dirty costs the same write-back).
template <int EB, int NWORDS>
__device__ __forceinline__ uint32_t state_elem(const uint32_t (&wd)[NWORDS], int idx) {
    // element idx of the window, as raw bits in the low EB bytes
    const int wi = (EB == 4) ? idx : (idx >> 1);
    uint32_t r = wd[0];
#pragma unroll
    for (int k = 1; k < NWORDS; ++k) r = (wi == k) ? wd[k] : r;
    if (EB == 2) r = (idx & 1) ? (r >> 16) : (r & 0xffffu);
    return r;
}
template <int EB, int NWORDS>
__device__ __forceinline__ void state_put(uint32_t (&wd)[NWORDS], int idx, uint32_t bits) {
    const int wi = (EB == 4) ? idx : (idx >> 1);
#pragma unroll
    for (int k = 0; k < NWORDS; ++k) {
        uint32_t nv = bits;
        if (EB == 2) nv = (idx & 1) ? ((wd[k] & 0xffffu) | (bits << 16)) : ((wd[k] & 0xffff0000u) | bits);
        wd[k] = (wi == k) ? nv : wd[k];
    }
}
template <int DT>
__device__ __forceinline__ float bits_to_float(uint32_t bits) {
    if constexpr (DT == VC1D_F32) return __uint_as_float(bits);
    if constexpr (DT == VC1D_BF16) return __uint_as_float(bits << 16);
    if constexpr (DT == VC1D_F16) return __half2float(__ushort_as_half((unsigned short)bits));
    return 0.f;
}
template <int DT>
__device__ __forceinline__ uint32_t float_to_bits(float v) {
    if constexpr (DT == VC1D_F32) return __float_as_uint(v);
    if constexpr (DT == VC1D_BF16) return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v));
    if constexpr (DT == VC1D_F16) return (uint32_t)__half_as_ushort(__float2half_rn(v));
    return 0u;
}

template <int DT, int W, int NV>
__global__ void __launch_bounds__(256) k_update_lane(const UParams p) {
    using E = Elem<DT>;
    using T = typename E::type;
    constexpr int EB = E::kBytes;
    constexpr int NWORDS = 4 * NV;
    constexpr int L = NV * 16 / EB;
    constexpr int UB = 2;  // sequences in flight per thread
    griddep_wait();
    griddep_launch_dependents();
    const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= p.total) return;
    const int d = (int)(g % p.D);
    const long long grp = g / p.D;

    float wf[W];
    float bf = 0.f;
#pragma unroll
    for (int w = 0; w < W; ++w) {
        const long long idx = (long long)d * p.wsd + (long long)w * p.wsw;
        wf[w] = (p.wdtype == VC1D_F32) ? __ldg(reinterpret_cast<const float*>(p.weight) + idx)
                                       : E::to_float(__ldg(reinterpret_cast<const T*>(p.weight) + idx));
    }
    if (p.bias != nullptr)
        bf = (p.wdtype == VC1D_F32) ? __ldg(reinterpret_cast<const float*>(p.bias) + d)
                                    : E::to_float(__ldg(reinterpret_cast<const T*>(p.bias) + d));

    const bool circular = p.seqlens != nullptr;
    const long long b0 = grp * p.nb;
    const long long b1 = (b0 + p.nb < p.B) ? b0 + p.nb : p.B;
    for (long long bb = b0; bb < b1; bb += UB) {
        uint32_t wd[UB][NWORDS];
        uint32_t xb[UB];
        int pos[UB];
#pragma unroll
        for (int u = 0; u < UB; ++u) {
            xb[u] = 0u;
            pos[u] = 0;
            if (bb + u < b1) {
                const uint4* sp = reinterpret_cast<const uint4*>(p.state + ((bb + u) * p.ssb + (long long)d * L) * EB);
#pragma unroll
                for (int j = 0; j < NV; ++j) {
                    const uint4 v = sp[j];
                    wd[u][4 * j] = v.x;
                    wd[u][4 * j + 1] = v.y;
                    wd[u][4 * j + 2] = v.z;
                    wd[u][4 * j + 3] = v.w;
                }
                const T xe = __ldg(reinterpret_cast<const T*>(p.x) + (bb + u) * p.sxb + d);
                if constexpr (EB == 4) xb[u] = __float_as_uint(xe);
                else xb[u] = (uint32_t)(*reinterpret_cast<const unsigned short*>(&xe));
                if (circular) {
                    int q = __ldg(p.seqlens + bb + u) % L;
                    pos[u] = q < 0 ? q + L : q;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < UB; ++u) {
            if (bb + u < b1) {
                const float xf = bits_to_float<DT>(xb[u]);
                float acc = bf;
                if (!circular) {
#pragma unroll
                    for (int w = 0; w < W - 1; ++w)
                        acc = fmaf(wf[w], bits_to_float<DT>(state_elem<EB, NWORDS>(wd[u], L + 1 - W + w)), acc);
                    acc = fmaf(wf[W - 1], xf, acc);
                    // shift the window left by one element, append x
                    if constexpr (EB == 4) {
#pragma unroll
                        for (int k = 0; k + 1 < NWORDS; ++k) wd[u][k] = wd[u][k + 1];
                        wd[u][NWORDS - 1] = xb[u];
                    } else {
#pragma unroll
                        for (int k = 0; k + 1 < NWORDS; ++k) wd[u][k] = __funnelshift_r(wd[u][k], wd[u][k + 1], 16);
                        wd[u][NWORDS - 1] = (wd[u][NWORDS - 1] >> 16) | (xb[u] << 16);
                    }
                } else {
#pragma unroll
                    for (int w = 0; w < W - 1; ++w) {
                        int h = pos[u] - (W - 1 - w);
                        h = h < 0 ? h + L : h;
                        acc = fmaf(wf[w], bits_to_float<DT>(state_elem<EB, NWORDS>(wd[u], h)), acc);
                    }
                    acc = fmaf(wf[W - 1], xf, acc);
                    state_put<EB, NWORDS>(wd[u], pos[u], xb[u]);
                }
                if (p.act) acc = silu1<E::kPreciseSilu>(acc);
                if (p.residual) acc = E::to_float(E::from_float(acc)) + xf;
                uint4* spw = reinterpret_cast<uint4*>(p.state + ((bb + u) * p.ssb + (long long)d * L) * EB);
#pragma unroll
                for (int j = 0; j < NV; ++j)
                    spw[j] = make_uint4(wd[u][4 * j], wd[u][4 * j + 1], wd[u][4 * j + 2], wd[u][4 * j + 3]);
                reinterpret_cast<T*>(p.y)[(bb + u) * p.syb + d] = E::from_float(acc);
            }
        }
    }
}

// Scalar kernel: any strides, any state_len >= width-1, shifting or circular state.
template <int DT>
__device__ __forceinline__ void update_generic_body(const UParams& p, unsigned block) {
    using E = Elem<DT>;
    using T = typename E::type;
    const long long g = (long long)block * blockDim.x + threadIdx.x;
    if (g >= p.total) return;
    const int d = (int)(g % p.D);
    const long long b = g / p.D;
    const T* x = reinterpret_cast<const T*>(p.x);
    T* y = reinterpret_cast<T*>(p.y);
    T* st = reinterpret_cast<T*>(p.state) + b * p.ssb + (long long)d * p.ssd;
    const int W = p.W, L = p.L;

    const T xr = x[b * p.sxb + (long long)d * p.sxd];
    float acc = 0.f;
    if (p.bias != nullptr) {
        acc = (p.wdtype == VC1D_F32) ? reinterpret_cast<const float*>(p.bias)[d]
                                     : E::to_float(reinterpret_cast<const T*>(p.bias)[d]);
    }
    auto wgt = [&](int w) -> float {
        const long long idx = (long long)d * p.wsd + (long long)w * p.wsw;
        return (p.wdtype == VC1D_F32) ? reinterpret_cast<const float*>(p.weight)[idx]
                                      : E::to_float(reinterpret_cast<const T*>(p.weight)[idx]);
    };
    if (p.seqlens == nullptr) {
        // taps first (they read the old state), then shift left by one and append
        for (int w = 0; w < W; ++w) {
            const int i = L + 1 - W + w;
            const float v = (i < L) ? E::to_float(st[(long long)i * p.ssl]) : E::to_float(xr);
            acc = fmaf(wgt(w), v, acc);
        }
        for (int j = 0; j + 1 < L; ++j) st[(long long)j * p.ssl] = st[(long long)(j + 1) * p.ssl];
        st[(long long)(L - 1) * p.ssl] = xr;
    } else {
        int pos = p.seqlens[b] % L;
        if (pos < 0) pos += L;
        for (int w = 0; w < W; ++w) {
            float v;
            if (w == W - 1) {
                v = E::to_float(xr);
            } else {
                int h = (pos - (W - 1 - w)) % L;
                if (h < 0) h += L;
                v = E::to_float(st[(long long)h * p.ssl]);
            }
            acc = fmaf(wgt(w), v, acc);
        }
        st[(long long)pos * p.ssl] = xr;
    }
    if (p.act) acc = silu1<E::kPreciseSilu>(acc);
    if (p.residual) acc = E::to_float(E::from_float(acc)) + E::to_float(xr);
    y[b * p.syb + (long long)d * p.syd] = E::from_float(acc);
}

template <int DT>
__global__ void __launch_bounds__(256) k_update_generic(const UParams p) {
    update_generic_body<DT>(p, blockIdx.x);
}

// Several independent problems in one launch.  Their parameters sit in the kernel's parameter space; the
// blocks of all problems are numbered through (first_block[i] = blocks of the problems before i), so a
// block finds its problem by bisection and no block is launched for nothing.  A problem that fits the
// vectorised code for this instantiation's width and state length takes it; every other one takes the
// scalar code.
constexpr int kMultiMax = VC1D_UPDATE_MULTI_MAX;
struct UMulti {
    UParams calls[kMultiMax];
    unsigned first_block[kMultiMax + 1];
    int n;
};
template <int DT, int W, int L>
__global__ void __launch_bounds__(256, 2) k_update_multi(const __grid_constant__ UMulti m) {
    griddep_wait();
    griddep_launch_dependents();
    int lo = 0, hi = m.n;  // the problem i with first_block[i] <= blockIdx.x < first_block[i + 1]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (m.first_block[mid] <= blockIdx.x)
            lo = mid;
        else
            hi = mid;
    }
    const UParams& p = m.calls[lo];
    const unsigned block = blockIdx.x - m.first_block[lo];
    if (p.vec)
        update_vec_body<DT, W, L>(p, block);
    else
        update_generic_body<DT>(p, block);
}

UParams make_params(const vc1d_update_args& a) {
    UParams p;
    p.x = reinterpret_cast<const char*>(a.x);
    p.y = reinterpret_cast<char*>(a.y);
    p.state = reinterpret_cast<char*>(a.conv_state);
    p.weight = a.weight;
    p.bias = a.bias;
    p.seqlens = a.cache_seqlens;
    p.sxb = a.x_stride_b;
    p.sxd = a.x_stride_d;
    p.syb = a.y_stride_b;
    p.syd = a.y_stride_d;
    p.ssb = a.s_stride_b;
    p.ssd = a.s_stride_d;
    p.ssl = a.s_stride_l;
    p.wsd = a.w_stride_d;
    p.wsw = a.w_stride_w;
    p.wdtype = a.wdtype;
    p.B = a.batch;
    p.D = a.dim;
    p.W = a.width;
    p.L = a.state_len;
    p.act = a.activation;
    p.residual = a.residual;
    p.nvec = 0;
    p.total = 0;
    p.nb = 1;
    p.vec = 0;
    p.w_fast = (a.wdtype == a.dtype && a.w_stride_w == 1 && a.w_stride_d == a.width &&
                (reinterpret_cast<uintptr_t>(a.weight) & 15u) == 0 &&
                (a.bias == nullptr || (reinterpret_cast<uintptr_t>(a.bias) & 15u) == 0))
                   ? 1
                   : 0;
    return p;
}

template <class Kernel>
cudaError_t launch_pdl(Kernel kernel, const UParams& p, dim3 grid, int block, cudaStream_t s) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3((unsigned)block);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, p);
}

template <int DT, int W>
cudaError_t launch_vec_l(const UParams& p, dim3 grid, int block, cudaStream_t s) {
    switch (p.L) {
        case 1:
            if (W == 2) return launch_pdl(k_update_vec<DT, (W == 2 ? W : 2), 1>, p, grid, block, s);
            return cudaErrorInvalidValue;
        case 2:
            if (W <= 3) return launch_pdl(k_update_vec<DT, (W <= 3 ? W : 2), 2>, p, grid, block, s);
            return cudaErrorInvalidValue;
        case 3: return launch_pdl(k_update_vec<DT, W, 3>, p, grid, block, s);
        case 4: return launch_pdl(k_update_vec<DT, W, 4>, p, grid, block, s);
        case 8: return launch_pdl(k_update_vec<DT, W, 8>, p, grid, block, s);
        default: return cudaErrorInvalidValue;
    }
}

template <int DT>
cudaError_t launch_vec_w(const UParams& p, dim3 grid, int block, cudaStream_t s) {
    switch (p.W) {
        case 2: return launch_vec_l<DT, 2>(p, grid, block, s);
        case 3: return launch_vec_l<DT, 3>(p, grid, block, s);
        default: return launch_vec_l<DT, 4>(p, grid, block, s);
    }
}

}  // namespace

bool update_vec_supports(int state_len, int width) {
    if (state_len < width - 1) return false;
    return state_len == 1 || state_len == 2 || state_len == 3 || state_len == 4 || state_len == 8;
}

cudaError_t launch_update_vec(const vc1d_update_args& a, cudaStream_t s) {
    UParams p = make_params(a);
    const int vec = 16 / elem_bytes(a.dtype);
    p.nvec = a.dim / vec;
    // a thread keeps its channels' weights in registers and walks nb sequences; small batches keep
    // one sequence per thread so that the grid still fills the GPU
    const long long threads1 = (long long)a.batch * p.nvec;
    long long nb = threads1 / ((long long)sm_count() * 2048);
    if (nb < 1) nb = 1;
    if (nb > 16) nb = 16;
    if (a.reserved > 0) nb = a.reserved;  // tuning override
    p.nb = (int)nb;
    const long long ngroups = (a.batch + nb - 1) / nb;
    p.total = ngroups * p.nvec;
    int block = a.block_threads > 0 ? a.block_threads : 128;
    if (block > 256) block = 256;
    block = (block + 31) / 32 * 32;
    const long long blocks = (p.total + block - 1) / block;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    note_launch("update_vec");
    const dim3 grid((unsigned)blocks);
    switch (a.dtype) {
        case VC1D_F32: return launch_vec_w<VC1D_F32>(p, grid, block, s);
        case VC1D_BF16: return launch_vec_w<VC1D_BF16>(p, grid, block, s);
        default: return launch_vec_w<VC1D_F16>(p, grid, block, s);
    }
}

// n problems (all of one I/O dtype) in one launch.  vec_ok[i]: problem i meets the layout conditions of the
// vectorised kernel.  The vectorised code is instantiated for the width and state length that most of those
// problems share; the others run the scalar code.
namespace {
template <int DT, int W, int L>
cudaError_t launch_multi_wl(const UMulti& m, dim3 grid, int block, cudaStream_t s) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3((unsigned)block);
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, k_update_multi<DT, W, L>, m);
}
template <int DT>
cudaError_t launch_multi_dt(const UMulti& m, int W, int L, dim3 grid, int block, cudaStream_t s) {
#define VC1D_MULTI(WW, LL) \
    if (W == WW && L == LL) return launch_multi_wl<DT, WW, LL>(m, grid, block, s);
    VC1D_MULTI(2, 1) VC1D_MULTI(2, 2) VC1D_MULTI(2, 3) VC1D_MULTI(2, 4) VC1D_MULTI(2, 8)
    VC1D_MULTI(3, 2) VC1D_MULTI(3, 3) VC1D_MULTI(3, 4) VC1D_MULTI(3, 8)
    VC1D_MULTI(4, 3) VC1D_MULTI(4, 4) VC1D_MULTI(4, 8)
#undef VC1D_MULTI
    return launch_multi_wl<DT, 4, 3>(m, grid, block, s);  // no problem takes the vectorised code
}
}  // namespace

cudaError_t launch_update_multi(const vc1d_update_args* calls, int n, const unsigned char* vec_ok, cudaStream_t s) {
    if (n < 1 || n > kMultiMax) return cudaErrorInvalidValue;
    // the (width, state length) pair most vectorisable problems have
    int best_w = 4, best_l = 3, best_n = 0;
    for (int i = 0; i < n; ++i) {
        if (!vec_ok[i]) continue;
        int cnt = 0;
        for (int j = 0; j < n; ++j)
            if (vec_ok[j] && calls[j].width == calls[i].width && calls[j].state_len == calls[i].state_len) ++cnt;
        if (cnt > best_n) {
            best_n = cnt;
            best_w = calls[i].width;
            best_l = calls[i].state_len;
        }
    }
    static thread_local UMulti m;  // 15 KB: not on the stack
    const int block = 128;
    long long n_blocks = 0;
    m.n = n;
    for (int i = 0; i < n; ++i) {
        const vc1d_update_args& a = calls[i];
        UParams p = make_params(a);
        p.vec = (best_n > 0 && vec_ok[i] && a.width == best_w && a.state_len == best_l) ? 1 : 0;
        if (p.vec) {
            const int vec = 16 / elem_bytes(a.dtype);
            p.nvec = a.dim / vec;
            p.nb = 1;  // decode batches that share a launch are small: one sequence per thread
            p.total = (long long)a.batch * p.nvec;
        } else {
            p.total = (long long)a.batch * a.dim;
        }
        m.first_block[i] = (unsigned)n_blocks;
        n_blocks += (p.total + block - 1) / block;
        if (n_blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
        m.calls[i] = p;
    }
    m.first_block[n] = (unsigned)n_blocks;
    note_launch("update_multi");
    const dim3 grid((unsigned)n_blocks);
    switch (calls[0].dtype) {
        case VC1D_F32: return launch_multi_dt<VC1D_F32>(m, best_w, best_l, grid, block, s);
        case VC1D_BF16: return launch_multi_dt<VC1D_BF16>(m, best_w, best_l, grid, block, s);
        default: return launch_multi_dt<VC1D_F16>(m, best_w, best_l, grid, block, s);
    }
}

bool update_lane_supports(int dtype, int state_len, int width) {
    const int bytes = state_len * elem_bytes(dtype);
    return state_len >= width - 1 && state_len >= 1 && (bytes == 16 || bytes == 32);
}

cudaError_t launch_update_lane(const vc1d_update_args& a, cudaStream_t s) {
    UParams p = make_params(a);
    // a thread keeps its channel's weights in registers and walks nb sequences
    const long long threads1 = (long long)a.batch * a.dim;
    long long nb = threads1 / ((long long)sm_count() * 2048 * 4);
    if (nb < 2) nb = 2;
    if (nb > 16) nb = 16;
    if (a.batch < nb) nb = a.batch;
    if (a.reserved > 0) nb = a.reserved;  // tuning override
    p.nb = (int)nb;
    const long long ngroups = (a.batch + nb - 1) / nb;
    p.total = ngroups * a.dim;
    int block = a.block_threads > 0 ? a.block_threads : 256;
    if (block > 256) block = 256;
    block = (block + 31) / 32 * 32;
    const long long blocks = (p.total + block - 1) / block;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    note_launch("update_lane");
    const dim3 grid((unsigned)blocks);
    const int nv = a.state_len * elem_bytes(a.dtype) / 16;
#define VC1D_LANE(DT)                                                                          \
    switch (a.width) {                                                                         \
        case 2: return nv == 1 ? launch_pdl(k_update_lane<DT, 2, 1>, p, grid, block, s)        \
                               : launch_pdl(k_update_lane<DT, 2, 2>, p, grid, block, s);       \
        case 3: return nv == 1 ? launch_pdl(k_update_lane<DT, 3, 1>, p, grid, block, s)        \
                               : launch_pdl(k_update_lane<DT, 3, 2>, p, grid, block, s);       \
        default: return nv == 1 ? launch_pdl(k_update_lane<DT, 4, 1>, p, grid, block, s)       \
                                : launch_pdl(k_update_lane<DT, 4, 2>, p, grid, block, s);      \
    }
    switch (a.dtype) {
        case VC1D_F32: VC1D_LANE(VC1D_F32)
        case VC1D_BF16: VC1D_LANE(VC1D_BF16)
        default: VC1D_LANE(VC1D_F16)
    }
#undef VC1D_LANE
}

cudaError_t launch_update_generic(const vc1d_update_args& a, cudaStream_t s) {
    UParams p = make_params(a);
    p.total = (long long)a.batch * a.dim;
    const int block = 256;
    const long long blocks = (p.total + block - 1) / block;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    note_launch("update_generic");
    const dim3 grid((unsigned)blocks);
    switch (a.dtype) {
        case VC1D_F32: k_update_generic<VC1D_F32><<<grid, block, 0, s>>>(p); break;
        case VC1D_BF16: k_update_generic<VC1D_BF16><<<grid, block, 0, s>>>(p); break;
        default: k_update_generic<VC1D_F16><<<grid, block, 0, s>>>(p); break;
    }
    return cudaGetLastError();
}

}  // namespace vc1d
