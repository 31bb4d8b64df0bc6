// Backward of prefill, scalar kernel for any strides and every option.
//
//     pre[t] = bias + sum_w weight[w] * xm[t-(W-1-w)]         xm = x * mask (rounded to the I/O dtype)
//     g[t]   = dy[t] * silu'(pre[t])                            (g = dy without activation)
//     dx[t]  = (residual ? dy[t] : 0) + mask[t] * sum_w weight[w] * g[t+(W-1-w)]
//     dweight[d,w] += sum_{b,t} xm[t-(W-1-w)] * g[t];    dbias[d] += sum_{b,t} g[t]
// (reference: causal-conv1d-mps/causal_conv1d_mps/causal_conv1d.metal:1354-1483).
//
// One thread owns one channel and a chunk of kChunk consecutive rows of one sequence.  It walks
// the chunk plus W-1 rows past it with two register windows (the last W masked inputs and the last
// W values of g), so every pre[t] is built once per chunk and neither x nor dy is re-read; the
// thread's partial dweight / dbias go to the fp32 accumulators with one atomic add each.
#include "vc1d_common.cuh"
#include "vc1d_internal.h"

namespace vc1d {
namespace {

constexpr int kChunk = 128;

struct BGParams {
    const void* x;
    const void* dy;
    void* dx;
    const void* weight;
    const void* bias;
    const void* mask;
    const void* init;   // [B, D, init_len] history, or NULL
    void* dinit;        // its gradient, or NULL
    float* dweight;
    float* dbias;
    const int* seq;     // sequence id of every step (packed rows), or NULL
    long long ssb, sst;
    long long sxb, sxd, sxt;  // elements
    long long sgb, sgd, sgt;
    long long sdb, sdd, sdt;
    long long smb, smt;
    long long wsd, wsw;
    int wdtype;
    int B, D, T, W;
    int act;
    int mask_dtype;
    int residual;
    int n_chunks;
    int init_len;
};

// MODE 0: expf and an IEEE division (fp32 I/O); 1: ex2.approx + rcp.approx (fp16 I/O);
// 2: s = 0.5 + 0.5 * tanh.approx(z / 2) (bf16 I/O) -- the same three forms, operation for
// operation, as the TMA-staged kernel, so that both kernels return the same bits.
template <int MODE>
__device__ __forceinline__ float silu_grad(float z) {
    // d/dz [z * s(z)] = s(z) * (1 + z * (1 - s(z)))
    float s;
    if (MODE == 0) {
        s = 1.0f / (1.0f + expf(-z));
    } else if (MODE == 1) {
        s = rcp_approx(1.0f + ex2_approx(z * -1.4426950408889634f));
    } else {
        float th;
        const float t = z * 0.5f;
        asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(t));
        s = fmaf(th, 0.5f, 0.5f);
    }
    const float u = fmaf(s, -1.0f, 1.0f);
    return s * fmaf(z, u, 1.0f);
}

template <int DT>
__global__ void __launch_bounds__(128) k_prefill_bwd_generic(const BGParams p) {
    using E = Elem<DT>;
    using T = typename E::type;
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= p.D) return;
    const int W = p.W, H = W - 1;
    const T* x = reinterpret_cast<const T*>(p.x);
    const T* dy = reinterpret_cast<const T*>(p.dy);
    T* dx = reinterpret_cast<T*>(p.dx);

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

    // work items of this thread: (sequence, chunk) pairs strided over gridDim.y
    const long long n_items = (long long)p.B * p.n_chunks;
    float dw[4] = {0.f, 0.f, 0.f, 0.f};
    float db = 0.f;
    for (long long item = blockIdx.y; item < n_items; item += gridDim.y) {
        const long long b = item / p.n_chunks;
        const int c0 = (int)(item - b * p.n_chunks) * kChunk;
        const int c1 = min(c0 + kChunk, p.T);

        auto masked_x = [&](int t, float& mk) -> float {
            mk = 1.f;
            if (t < 0) {  // history of a chunked continuation, already masked when it was stored
                if (p.init == nullptr || p.init_len + t < 0) return 0.f;
                return E::to_float(reinterpret_cast<const T*>(p.init)[(b * p.D + d) * p.init_len + (p.init_len + t)]);
            }
            if (t >= p.T) return 0.f;
            if (p.mask != nullptr) mk = load_mask(p.mask, b * p.smb + (long long)t * p.smt, p.mask_dtype);
            if (mk == 0.f) return 0.f;
            float v = E::to_float(x[b * p.sxb + (long long)d * p.sxd + (long long)t * p.sxt]);
            if (mk != 1.f) v = E::to_float(E::from_float(v * mk));
            return v;
        };

        if (c0 == 0 && p.dinit != nullptr) {  // history columns that no tap reads get no gradient
            T* drow = reinterpret_cast<T*>(p.dinit) + (b * p.D + d) * p.init_len;
            for (int col = 0; col < p.init_len - H; ++col) drow[col] = E::from_float(0.f);
        }
        // sequence id of a row (packed rows): a tap counts only between rows of one sequence
        auto seq_id = [&](int t) -> int {
            if (p.seq == nullptr || t < 0 || t >= p.T) return 0;
            return p.seq[b * p.ssb + (long long)t * p.sst];
        };
        // xw[3] is xm[j], xw[2] xm[j-1], ...; gw likewise for g, idw for the sequence ids
        float xw[4] = {0.f, 0.f, 0.f, 0.f};
        float gw[4] = {0.f, 0.f, 0.f, 0.f};
        int idw[4] = {0, 0, 0, 0};
        float mk_unused;
        for (int i = 0; i < H; ++i) {  // rows before the chunk
            xw[4 - H + i] = masked_x(c0 - H + i, mk_unused);
            idw[4 - H + i] = seq_id(c0 - H + i);
        }
        float mkw[4] = {1.f, 1.f, 1.f, 1.f};  // mask of rows j-3 .. j (for dx of row j-H)
        for (int j = c0; j < c1 + H; ++j) {
            xw[0] = xw[1]; xw[1] = xw[2]; xw[2] = xw[3];
            mkw[0] = mkw[1]; mkw[1] = mkw[2]; mkw[2] = mkw[3];
            idw[0] = idw[1]; idw[1] = idw[2]; idw[2] = idw[3];
            xw[3] = masked_x(j, mkw[3]);
            idw[3] = seq_id(j);
            if (p.seq != nullptr) {
                // inputs above the start of row j's sequence (the run of equal ids that ends at j) are no taps
                // of row j, nor of any later row
                bool cut = false;
                for (int i = 2; i >= 0; --i) {
                    cut |= (idw[i] != idw[3]);
                    if (cut) xw[i] = 0.f;
                }
            }
            float g = 0.f;
            if (j < p.T) {
                g = E::to_float(dy[b * p.sgb + (long long)d * p.sgd + (long long)j * p.sgt]);
                if (p.act) {
                    float pre = bv;
                    for (int w = 0; w < W; ++w) pre = fmaf(wt[w], xw[4 - W + w], pre);
                    g *= silu_grad<(DT == VC1D_F32) ? 0 : (DT == VC1D_F16 ? 1 : 2)>(pre);
                }
            }
            gw[0] = gw[1]; gw[1] = gw[2]; gw[2] = gw[3];
            gw[3] = g;
            if (j < c1) {  // rows of this chunk: parameter gradients
                for (int w = 0; w < W; ++w) dw[w] = fmaf(xw[4 - W + w], g, dw[w]);
                db += g;
            }
            const int t = j - H;
            if (t < 0 && c0 == 0 && p.dinit != nullptr && p.init_len + t >= 0) {
                // gradient of the history rows: the taps of the first W-1 outputs that reached back
                float acc = 0.f;
                for (int w = 0; w < W; ++w) acc = fmaf(wt[w], gw[3 - w], acc);
                reinterpret_cast<T*>(p.dinit)[(b * p.D + d) * p.init_len + (p.init_len + t)] = E::from_float(acc);
            }
            if (t >= c0) {  // t < c1 holds by the loop bound
                float acc = 0.f;
                // g of row j - w = t + (H - w) reaches input row t through weight[w]; with packed rows only
                // while the run of equal ids that row t belongs to lasts
                int reach = H;
                if (p.seq != nullptr) {
                    reach = 0;
                    while (reach < H && idw[3 - H + reach + 1] == idw[3 - H]) ++reach;
                }
                for (int w = 0; w < W; ++w)
                    if (H - w <= reach) acc = fmaf(wt[w], gw[3 - w], acc);
                acc *= mkw[3 - H];
                if (p.residual) acc += E::to_float(dy[b * p.sgb + (long long)d * p.sgd + (long long)t * p.sgt]);
                dx[b * p.sdb + (long long)d * p.sdd + (long long)t * p.sdt] = E::from_float(acc);
            }
        }
    }
    if (p.dweight != nullptr)
        for (int w = 0; w < W; ++w) atomicAdd(p.dweight + (long long)d * W + w, dw[w]);
    if (p.dbias != nullptr) atomicAdd(p.dbias + d, db);
}

}  // namespace

cudaError_t launch_prefill_bwd_generic(const vc1d_prefill_bwd_args& a, cudaStream_t s) {
    BGParams p;
    p.x = a.x; p.dy = a.dy; p.dx = a.dx;
    p.weight = a.weight; p.bias = a.bias; p.mask = a.mask;
    p.init = a.initial_state; p.dinit = a.dinitial_state; p.init_len = a.init_len;
    p.dweight = a.dweight; p.dbias = a.dbias;
    p.seq = a.seq_idx; p.ssb = a.seq_stride_b; p.sst = a.seq_stride_t;
    p.sxb = a.x_stride_b; p.sxd = a.x_stride_d; p.sxt = a.x_stride_t;
    p.sgb = a.dy_stride_b; p.sgd = a.dy_stride_d; p.sgt = a.dy_stride_t;
    p.sdb = a.dx_stride_b; p.sdd = a.dx_stride_d; p.sdt = a.dx_stride_t;
    p.smb = a.mask_stride_b; p.smt = a.mask_stride_t;
    p.wsd = a.w_stride_d; p.wsw = a.w_stride_w;
    p.wdtype = a.wdtype;
    p.B = a.batch; p.D = a.dim; p.T = a.seqlen; p.W = a.width;
    p.act = a.activation == VC1D_ACT_SILU;
    p.mask_dtype = a.mask_dtype;
    p.residual = a.residual != 0;
    p.n_chunks = (a.seqlen + kChunk - 1) / kChunk;
    const long long n_items = (long long)a.batch * p.n_chunks;
    const dim3 block(128);
    const dim3 grid((unsigned)((a.dim + 127) / 128), (unsigned)(n_items < 65535 ? n_items : 65535));
    if (a.zero_grads) {
        cudaError_t e = a.dweight != nullptr ? cudaMemsetAsync(a.dweight, 0, sizeof(float) * (size_t)a.dim * a.width, s)
                                             : cudaSuccess;
        if (e == cudaSuccess && a.dbias != nullptr) e = cudaMemsetAsync(a.dbias, 0, sizeof(float) * (size_t)a.dim, s);
        if (e != cudaSuccess) return e;
    }
    note_launch("bwd_generic");
    switch (a.dtype) {
        case VC1D_F32: k_prefill_bwd_generic<VC1D_F32><<<grid, block, 0, s>>>(p); break;
        case VC1D_BF16: k_prefill_bwd_generic<VC1D_BF16><<<grid, block, 0, s>>>(p); break;
        default: k_prefill_bwd_generic<VC1D_F16><<<grid, block, 0, s>>>(p); break;
    }
    return cudaGetLastError();
}

}  // namespace vc1d
