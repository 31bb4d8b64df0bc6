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
};

template <int DT, int W, int L>
__global__ void __launch_bounds__(256, 2) k_update_vec(const UParams p) {
    using E = Elem<DT>;
    using T = typename E::type;
    using PK = Pack<DT>;
    constexpr int VEC = E::kVec;
    constexpr int UB = 2;  // sequences in flight per thread
    // Launched with programmatic stream serialization: consecutive decode steps depend on each other
    // through conv_state, so every thread waits for the previous kernel before its first access,
    // while the launch itself and the scheduling of the CTAs overlap the previous step's tail.
    griddep_wait();
    griddep_launch_dependents();
    const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
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

// Scalar kernel: any strides, any state_len >= width-1, shifting or circular state.
template <int DT>
__global__ void __launch_bounds__(256) k_update_generic(const UParams p) {
    using E = Elem<DT>;
    using T = typename E::type;
    const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
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
