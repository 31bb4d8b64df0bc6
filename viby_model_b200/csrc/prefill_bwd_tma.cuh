// Backward of channel-last prefill on the TMA pipeline of the forward kernel.
//
//     pre[t] = bias + sum_w weight[w] * xm[t-(W-1-w)]         xm = x * mask (rounded to the I/O dtype)
//     g[t]   = dy[t] * silu'(pre[t])                            (g = dy without activation)
//     dx[t]  = (residual ? dy[t] : 0) + mask[t] * sum_w weight[w] * g[t+(W-1-w)]
//     dweight[d,w] += sum_{b,t} xm[t-(W-1-w)] * g[t];    dbias[d] += sum_{b,t} g[t]
// (reference: causal-conv1d-mps/causal_conv1d_mps/causal_conv1d.metal:803-854, 1354-1483, which
// rebuilds pre[] of every future position per output element and adds every product to dweight
// with a global atomic.)
//
// Here a tile is 64 rows x one channel slab of one sequence.  The producer warp brings in two
// boxes per tile with bulk tensor copies: x rows [t0-H, t0+64+H) and dy rows [t0, t0+64+H), H = W-1
// (rows outside the sequence arrive as zeros, which is both the causal padding of x and "no
// gradient from beyond the end").  A consumer thread owns 4 or 8 bytes of channels and 8 or 16
// consecutive rows (BwdGeometry); it walks its rows + H once with two register windows (masked
// inputs, g), so each pre[t] is built once per thread, each g[t] feeds the W outputs that use it,
// and nothing is re-read.  The
// thread's dweight / dbias partial sums stay in registers across all tiles of its CTA (a CTA keeps
// its channel slab); at the end the CTA adds them up through shared memory and issues one atomic
// add per (channel, tap).  HBM traffic is the algorithmic minimum: x and dy read once, dx written once.
#pragma once

#include "prefill_tma.cuh"

namespace vc1d {
namespace tma {

struct BwdParams {
    char* dx;
    const void* weight;
    const void* bias;
    const void* mask;
    float* dweight;
    float* dbias;
    unsigned int* sched;     // per-slab claim counters in scratch memory (NULL: static assignment)
    const unsigned char* gtable;  // class byte per (sequence, time tile) from the pre-pass, or NULL
    unsigned int* timeouts;
    long long sdb, sdt;      // dx strides in bytes
    long long smb, smt;      // mask strides in elements
    long long wsd, wsw;
    int wdtype;
    int B, D, T;
    int n_ttile, n_rowtiles, ctas_per_slab;
    int mask_dtype;
    int residual;
    int stages;
    int seg_mode;  // mask holds int32 sequence ids (packed rows): no multipliers, taps stay inside a run of equal ids
};

// VARIANT 0: a thread owns 8 bytes of channels and 8 consecutive rows.  VARIANT 1 (16-bit I/O): 4
// bytes of channels (one pair) and 8 rows, so a tile is half as tall and a third CTA fits an SM.
// VARIANT 2 (16-bit I/O): 4 bytes of channels and 16 rows: tiles as tall as variant 0, three CTAs per
// SM with a two-stage ring, and the W-1 rows of g below a thread's own rows, which it has to work
// out a second time, are spread over 16 rows instead of 8.
template <int DT, int W, int SLAB_BYTES, int VARIANT = 0>
struct BwdGeometry {
    static constexpr int kVB = (VARIANT == 0) ? 8 : 4;
    static constexpr int kH = W - 1;
    static constexpr int kRows = (VARIANT == 2) ? 16 : 8;
    static constexpr int kLanesPerRow = SLAB_BYTES / kVB;
    static constexpr int kConsumerWarps = 8;
    static constexpr int kConsumerThreads = kConsumerWarps * 32;
    static constexpr int kThreads = kConsumerThreads + 32;
    static constexpr int kGroups = kConsumerThreads / kLanesPerRow;
    static constexpr int kTileRows = kGroups * kRows;
    static constexpr int kXRows = kTileRows + 2 * kH;  // x box: H rows above the tile, H below
    static constexpr int kGRows = kTileRows + kH;      // dy box: H rows below the tile
    static constexpr int kRowBytes = SLAB_BYTES;
    static constexpr int kSlabElems = SLAB_BYTES / Elem<DT>::kBytes;
    static constexpr int kXBytes = kXRows * kRowBytes;
    static constexpr int kGBytes = kGRows * kRowBytes;
    static constexpr int kStageBytes = kXBytes + kGBytes;  // rows are 128 or 256 bytes: stays 128-byte aligned
    // fp32 I/O (one channel pair per thread) fits 72 registers: 3 CTAs per SM with a 2-stage ring.  16-bit I/O
    // (two pairs) needs 96: 2 CTAs per SM with 3 stages; squeezed to 72 it spills and runs at half the speed.
    static constexpr int kCtasPerSm = (DT == VC1D_F32 || VARIANT != 0) ? 3 : 2;
    static constexpr int kDefaultStages = ((DT == VC1D_F32 && VARIANT == 0) || VARIANT == 2) ? 2 : 3;
    // layout for S stages: stages | full[S], done[S] | tile descriptor[S]
    __host__ __device__ static constexpr int off_bars(int S) { return S * kStageBytes; }
    __host__ __device__ static constexpr int off_flags(int S) { return off_bars(S) + 2 * S * 8; }
    __host__ __device__ static constexpr int smem_bytes(int S) { return off_flags(S) + S * 32 + 128; }
};

// silu'(z) = s * (1 + z * (1 - s)), s = sigmoid(z), for a pair of lanes.
// MODE 0: expf and an IEEE division (fp32 I/O).  MODE 1: ex2.approx + rcp.approx (fp16 I/O).
// MODE 2: s = 0.5 + 0.5 * tanh.approx(z / 2), one special-function op per element instead of two;
// its absolute error of 2.5e-4 in s (4e-4 in silu') is 1/20 of a bf16 step at 1, so bf16 I/O uses it.
template <int MODE>
__device__ __forceinline__ float2 silu_grad2(float2 z) {
    float2 s;
    if constexpr (MODE == 0) {
        s = make_float2(1.0f / (1.0f + expf(-z.x)), 1.0f / (1.0f + expf(-z.y)));
    } else if constexpr (MODE == 1) {
        const float2 t = mul2(z, make_float2(-1.4426950408889634f, -1.4426950408889634f));
        float2 e = make_float2(ex2_approx(t.x), ex2_approx(t.y));
        e = add2(e, make_float2(1.0f, 1.0f));
        s = make_float2(rcp_approx(e.x), rcp_approx(e.y));
    } else {
        const float2 half = make_float2(0.5f, 0.5f);
        const float2 t = mul2(z, half);
        float2 th;
        asm("tanh.approx.f32 %0, %1;" : "=f"(th.x) : "f"(t.x));
        asm("tanh.approx.f32 %0, %1;" : "=f"(th.y) : "f"(t.y));
        s = fma2(th, half, half);
    }
    const float2 one = make_float2(1.0f, 1.0f);
    const float2 u = fma2(s, make_float2(-1.0f, -1.0f), one);  // 1 - s
    return mul2(s, fma2(z, u, one));
}

__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

template <int DT, int W, int SLAB_BYTES, bool ACT, int VARIANT = 0>
__global__ void __launch_bounds__(BwdGeometry<DT, W, SLAB_BYTES, VARIANT>::kThreads,
                                  BwdGeometry<DT, W, SLAB_BYTES, VARIANT>::kCtasPerSm)
    k_prefill_bwd_tma(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_g,
                      const BwdParams p) {
    using E = Elem<DT>;
    using G = BwdGeometry<DT, W, SLAB_BYTES, VARIANT>;
    constexpr int VB = G::kVB;
    using S = Slice<DT, VB>;
    constexpr int NE = S::kElems;
    constexpr int NP = S::kPairs;
    constexpr int NW = S::kWords;
    constexpr int H = G::kH;
    constexpr int R = G::kRows;
    constexpr int LPR = G::kLanesPerRow;
    constexpr int GL = LPR < 32 ? LPR : 32;  // lanes of one row group inside a warp
    static_assert(R + 2 * H <= GL, "one mask value per lane of a row group");

    extern __shared__ __align__(128) unsigned char smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 127u) & ~127u;
    unsigned char* const base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const int kStages = p.stages;
    const uint32_t bars = base + G::off_bars(kStages);
    const uint32_t flags = base + G::off_flags(kStages);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int slab = blockIdx.x;
    const int j0 = blockIdx.y;
    const int stride = p.ctas_per_slab;
    const int slab_ch0 = slab * G::kSlabElems;
    const int n_my = (j0 < p.n_rowtiles) ? (p.n_rowtiles - j0 + stride - 1) / stride : 0;

    if (threadIdx.x == G::kConsumerWarps * 32) {
        prefetch_tensormap(&tmap_x);
        prefetch_tensormap(&tmap_g);
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bars + 8 * s, 1);
            mbar_init(bars + 8 * (kStages + s), G::kConsumerWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // launched as a programmatic dependent of whatever precedes it in the stream (the tile-classification
    // pre-pass when there is one): nothing above touched global memory
    griddep_wait();
    __syncthreads();

    if (warp == G::kConsumerWarps) {
        // ================================ producer warp ==================================
        int s_ring = 0, n_ring = 0;
        uint32_t ph_ring = 0;
        auto claim = [&]() -> bool {
            if (n_ring >= kStages) {
                const bool ok = mbar_wait(bars + 8 * (kStages + s_ring), ph_ring ^ 1);
                if (!ok && lane == 0) atomicAdd(p.timeouts, 1u);
                if (!ok) return false;
            }
            return true;
        };
        auto advance = [&]() {
            ++n_ring;
            if (++s_ring == kStages) {
                s_ring = 0;
                ph_ring ^= 1;
            }
        };
        const bool dynamic = p.sched != nullptr;
        int n_issued = 0;
        auto next_tile = [&]() -> int {
            unsigned raw;
            if (dynamic) {
                raw = 0u;
                if (lane == 0) raw = atomicAdd(p.sched + slab, 1u);
                raw = __shfl_sync(0xffffffffu, raw, 0);
            } else {
                raw = n_issued < n_my ? (unsigned)(j0 + n_issued * stride) : 0xffffffffu;
            }
            ++n_issued;
            return raw < (unsigned)p.n_rowtiles ? (int)raw : -1;
        };
        bool live = true;
        int rt = next_tile();
        while (live && rt >= 0) {
            const int b = rt / p.n_ttile;
            const int t0 = (rt - b * p.n_ttile) * G::kTileRows;
            // a tile whose x rows are all masked out needs no x: only its dy box is copied
            // class from the pre-pass: all mask rows one, mixed, or every x row masked out (no x box)
            const int cls_now = p.gtable != nullptr ? (int)__ldcg(p.gtable + rt)  // written by the pre-pass while this grid was resident: no read-only path
                                                    : (p.mask != nullptr ? (int)TILE_MIXED : (int)TILE_FULL);
            const bool need_x = cls_now != TILE_EMPTY;
            rt = next_tile();  // fetched while this tile waits for its slot
            live = claim();
            if (!live) break;
            const int s = s_ring;
            if (lane == 0) {
                const long long off = (long long)b * p.sdb + (long long)t0 * p.sdt;
                sts_desc(flags + 32 * s, cls_now, p.T - t0, off);
                sts_s32(flags + 32 * s + 16, b);
                sts_s32(flags + 32 * s + 20, t0);
                const uint32_t full = bars + 8 * s;
                const uint32_t dst = base + s * G::kStageBytes;
                mbar_arrive_expect_tx(full, (need_x ? G::kXBytes : 0) + G::kGBytes);
                if (need_x) tma_load_3d(dst, &tmap_x, slab_ch0, t0 - H, b, full);
                tma_load_3d(dst + G::kXBytes, &tmap_g, slab_ch0, t0, b, full);
            }
            __syncwarp();
            advance();
        }
        // every tile of this CTA is on its way: a dependent launch of the stream may take the slots that CTAs
        // free as they finish
        griddep_launch_dependents();
        if (live && claim()) {
            if (lane == 0) {
                sts_desc(flags + 32 * s_ring, TILE_END, 0, 0);
                mbar_arrive(bars + 8 * s_ring);
            }
            __syncwarp();
        }
        if (dynamic && lane == 0) {
            // the last CTA to finish claiming leaves the counters zeroed for the next launch
            const unsigned n_ctas = gridDim.x * gridDim.y;
            __threadfence();
            const unsigned done = atomicAdd(p.sched + gridDim.x, 1u);
            if (done == n_ctas - 1) {
                for (unsigned k = 0; k <= gridDim.x; ++k) p.sched[k] = 0u;
                __threadfence();
            }
        }
        return;
    }

    // ================================ consumer warps =====================================
    const int grp = threadIdx.x / LPR;
    const int cl = threadIdx.x % LPR;
    const int d0 = slab_ch0 + cl * NE;
    const bool ch_ok = d0 < p.D;
    const int rbase = grp * R;

    float2 wp[W][NP];
    float2 bp[NP];
    {
        TmaParams wparams = {};  // load_weights reads these fields only
        wparams.weight = p.weight;
        wparams.bias = p.bias;
        wparams.wsd = p.wsd;
        wparams.wsw = p.wsw;
        wparams.wdtype = p.wdtype;
        load_weights<DT, W, VB>(wparams, d0, ch_ok, wp, bp);
    }
    float2 dwp[W][NP];
    float2 dbp[NP];
    float2 sgb[NP];  // silu'(bias): the factor of g in rows whose inputs are all masked out
#pragma unroll
    for (int q = 0; q < NP; ++q) {
        sgb[q] = ACT ? silu_grad2<(DT == VC1D_F32) ? 0 : (DT == VC1D_F16 ? 1 : 2)>(bp[q]) : make_float2(1.0f, 1.0f);
        dbp[q] = make_float2(0.f, 0.f);
#pragma unroll
        for (int w = 0; w < W; ++w) dwp[w][q] = make_float2(0.f, 0.f);
    }

    char* const dxbase = p.dx + (long long)rbase * p.sdt + (long long)d0 * E::kBytes;
    const unsigned pitch = (unsigned)p.sdt;
    const uint32_t tbase = base + rbase * G::kRowBytes + cl * VB;
    const int rbase_lim = ch_ok ? rbase : (1 << 28);
    const bool masked = p.mask != nullptr;
    const int msrc = lane & ~(GL - 1);
    const int mj = lane & (GL - 1);

    int s = -1;
    uint32_t ph = 0;
    uint32_t xrow = tbase - G::kStageBytes;
    for (;;) {
        xrow += G::kStageBytes;
        if (++s == kStages) {
            s = 0;
            ph ^= 1;
            xrow = tbase;
        }
        if (!mbar_wait(bars + 8 * s, ph)) {
            if (lane == 0) atomicAdd(p.timeouts, 1u);
            break;
        }
        int cls, rows_valid;
        long long off;
        lds_desc(flags + 32 * s, cls, rows_valid, off);
        if (cls == TILE_END) break;
        const int rows_ok = min(R, max(0, rows_valid - rbase_lim));
        char* dxrow = dxbase + off;
        const uint32_t grow = xrow + G::kXBytes;  // this thread's first dy row
        // x box row n of this thread is time tfirst - H + n (n = 0 .. R+2H-1); dy box row n is tfirst + n
        float mkv = 1.0f;
        if (cls == TILE_MIXED) {  // only mixed tiles look at their mask rows
            const int b = lds_s32(flags + 32 * s + 16);
            const int tfirst = lds_s32(flags + 32 * s + 20) + rbase;
            TmaParams mp = {};
            mp.mask = p.mask;
            mp.smt = p.smt;
            mp.mask_dtype = p.mask_dtype;
            mp.T = p.T;
            mp.seg_mode = p.seg_mode;
            if (mj < R + 2 * H) mkv = tile_mask(mp, (long long)b * p.smb, tfirst - H + mj);
        }
        // rows of this warp whose mask values are all one take the code without mask arithmetic
        const bool warp_masked = cls == TILE_MIXED && !__all_sync(0xffffffffu, mkv == 1.0f);
        // x box row n has just been put into its window slot.  With a mask: multiply it.  With packed rows a
        // value other than one means that a sequence starts at this row: the rows above it are no taps of it
        // or of anything after it, so the other slots of the window are cleared.
        auto mask_row = [&](float2 (&xw)[W][NP], int n, float mk) {
            if (p.seg_mode) {
                if (mk != 1.0f) {
#pragma unroll
                    for (int v = 1; v < W; ++v)
#pragma unroll
                        for (int q = 0; q < NP; ++q) xw[(n + v) % W][q] = make_float2(0.f, 0.f);
                }
            } else {
                apply_mask<DT, VB>(xw[n % W], mk, 1);
            }
        };
        auto rows = [&](auto mk_c) {
            constexpr bool MK = decltype(mk_c)::value;
            float2 xw[W][NP];  // masked inputs: row n lives in slot n % W
            float2 gw[W][NP];  // g: row jj lives in slot jj % W
    #pragma unroll
            for (int n = 0; n < H; ++n) {
                uint32_t raw[NW];
                S::lds(xrow + n * G::kRowBytes, raw);
                S::unpack(raw, xw[n % W]);
                if constexpr (MK) mask_row(xw, n, __shfl_sync(0xffffffffu, mkv, msrc + n));
            }
            static_for<0, R + H>([&](auto jc) {
                constexpr int jj = decltype(jc)::value;
                constexpr int n = H + jj;  // x box row of this step
                {
                    uint32_t raw[NW];
                    S::lds(xrow + n * G::kRowBytes, raw);
                    S::unpack(raw, xw[n % W]);
                    if constexpr (MK) mask_row(xw, n, __shfl_sync(0xffffffffu, mkv, msrc + n));
                }
                float2 g[NP];
                {
                    uint32_t raw[NW];
                    S::lds(grow + jj * G::kRowBytes, raw);
                    S::unpack(raw, g);
                }
                if constexpr (ACT) {
    #pragma unroll
                    for (int q = 0; q < NP; ++q) {
                        float2 pre = bp[q];
    #pragma unroll
                        for (int w = 0; w < W; ++w) pre = fma2(wp[w][q], xw[(n + 1 + w) % W][q], pre);
                        g[q] = mul2(g[q], silu_grad2<(DT == VC1D_F32) ? 0 : (DT == VC1D_F16 ? 1 : 2)>(pre));
                    }
                }
    #pragma unroll
                for (int q = 0; q < NP; ++q) gw[jj % W][q] = g[q];
                if constexpr (jj < R) {
                    // rows of this thread's own share of the tile: parameter gradients
    #pragma unroll
                    for (int q = 0; q < NP; ++q) {
    #pragma unroll
                        for (int w = 0; w < W; ++w) dwp[w][q] = fma2(xw[(n + 1 + w) % W][q], g[q], dwp[w][q]);
                        dbp[q] = add2(dbp[q], g[q]);
                    }
                }
                if constexpr (jj >= H) {
                    constexpr int k = jj - H;  // output row: dx[t] = sum_w weight[w] * g[t + (W-1-w)], t + H = jj
                    float2 acc[NP];
                    // g of row k + H - w reaches input row k through weight[w]; with packed rows only while
                    // the sequence of row k lasts, i.e. for the first `reach` rows behind it
                    int reach = H;
                    if constexpr (MK) {
                        if (p.seg_mode) {
                            reach = 0;
                            bool open = true;
    #pragma unroll
                            for (int u = 1; u <= H; ++u) {
                                open = open && (__shfl_sync(0xffffffffu, mkv, msrc + H + k + u) == 1.0f);
                                if (open) reach = u;
                            }
                        }
                    }
    #pragma unroll
                    for (int q = 0; q < NP; ++q) {
                        acc[q] = (reach == H) ? mul2(wp[0][q], gw[jj % W][q]) : make_float2(0.f, 0.f);
    #pragma unroll
                        for (int w = 1; w < W; ++w)
                            if (H - w <= reach) acc[q] = fma2(wp[w][q], gw[(jj - w + W) % W][q], acc[q]);
                    }
                    if constexpr (MK) {
                        if (!p.seg_mode) {
                            const float mk = __shfl_sync(0xffffffffu, mkv, msrc + H + k);
    #pragma unroll
                            for (int q = 0; q < NP; ++q) acc[q] = mul2(acc[q], make_float2(mk, mk));
                        }
                    }
                    if (p.residual) {
                        uint32_t raw[NW];
                        float2 dyk[NP];
                        S::lds(grow + k * G::kRowBytes, raw);
                        S::unpack(raw, dyk);
    #pragma unroll
                        for (int q = 0; q < NP; ++q) acc[q] = add2(acc[q], dyk[q]);
                    }
                    uint32_t outw[NW];
                    S::pack(acc, outw);
                    S::template stg_row<k>(row_addr<k>(dxrow, pitch), outw, rows_ok);
                }
            });
        };
        // rows whose inputs are all masked out: pre = bias, so g = dy * silu'(bias); no gradient reaches
        // the weights or, residual aside, the inputs
        // (a tile the producer classed as empty arrives without its x box: it must take this path)
        const bool warp_zero = cls == TILE_EMPTY || (cls == TILE_MIXED && __all_sync(0xffffffffu, mj >= R + 2 * H || mkv == 0.0f));
        if (warp_zero) {
            static_for<0, R>([&](auto kc) {
                constexpr int k = decltype(kc)::value;
                uint32_t raw[NW];
                float2 g[NP];
                S::lds(grow + k * G::kRowBytes, raw);
                S::unpack(raw, g);
                if (!p.residual) {
#pragma unroll
                    for (int i = 0; i < NW; ++i) raw[i] = 0u;
                }
                S::template stg_row<k>(row_addr<k>(dxrow, pitch), raw, rows_ok);  // dx = dy (residual) or +0
#pragma unroll
                for (int q = 0; q < NP; ++q) dbp[q] = fma2(g[q], sgb[q], dbp[q]);
            });
        } else if (warp_masked) {
            rows(std::true_type{});
        } else {
            rows(std::false_type{});
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + 8 * (kStages + s));
    }

    // ---- parameter gradients: add up the row groups of the CTA, one atomic per (channel, tap) ----
    if (p.dweight != nullptr || p.dbias != nullptr) {
        constexpr int NACC = NE * (W + 1);
        static_assert(G::kConsumerThreads * NACC * 4 <= G::kStageBytes, "the reduction reuses the first stage");
        float* red = reinterpret_cast<float*>(base_ptr);
        named_barrier_sync(1, G::kConsumerThreads);  // every consumer warp has left the ring
        float* mine = red + threadIdx.x * NACC;
#pragma unroll
        for (int q = 0; q < NP; ++q) {
#pragma unroll
            for (int w = 0; w < W; ++w) {
                mine[(2 * q) * (W + 1) + w] = dwp[w][q].x;
                mine[(2 * q + 1) * (W + 1) + w] = dwp[w][q].y;
            }
            mine[(2 * q) * (W + 1) + W] = dbp[q].x;
            mine[(2 * q + 1) * (W + 1) + W] = dbp[q].y;
        }
        named_barrier_sync(1, G::kConsumerThreads);
        if (threadIdx.x < LPR && ch_ok) {
#pragma unroll
            for (int c = 0; c < NE; ++c) {
#pragma unroll
                for (int w = 0; w <= W; ++w) {
                    float sum = 0.f;
                    for (int gi = 0; gi < G::kGroups; ++gi) sum += red[(gi * LPR + cl) * NACC + c * (W + 1) + w];
                    if (w < W) {
                        if (p.dweight != nullptr) atomicAdd(p.dweight + (long long)(d0 + c) * W + w, sum);
                    } else if (p.dbias != nullptr) {
                        atomicAdd(p.dbias + d0 + c, sum);
                    }
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
template <int DT, int W, int SLAB_BYTES, bool ACT, int VARIANT = 0>
cudaError_t launch_bwd_kernel(const vc1d_prefill_bwd_args& a, const BwdParams& base, cudaStream_t s) {
    using G = BwdGeometry<DT, W, SLAB_BYTES, VARIANT>;
    const int eb = Elem<DT>::kBytes;
    BwdParams p = base;
    const int slab_ch = G::kSlabElems;
    const int n_slab = (a.dim + slab_ch - 1) / slab_ch;
    p.n_ttile = (a.seqlen + G::kTileRows - 1) / G::kTileRows;
    const long long n_rowtiles = (long long)a.batch * p.n_ttile;
    if (n_rowtiles > 0x7fffffffLL) return cudaErrorNotSupported;
    p.n_rowtiles = (int)n_rowtiles;
    if (a.dx_stride_t < 0 || (long long)a.dx_stride_t * eb >= (1LL << 28)) return cudaErrorNotSupported;

    EncodeFn enc = encode_fn();
    if (enc == nullptr) return cudaErrorNotSupported;
    const CUtensorMapDataType dt = (DT == VC1D_F32)    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : (DT == VC1D_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                       : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    auto make_map = [&](CUtensorMap* m, const void* ptr, long long st_t, long long st_b, int rows) -> bool {
        const cuuint64_t dims[3] = {(cuuint64_t)a.dim, (cuuint64_t)a.seqlen, (cuuint64_t)a.batch};
        const cuuint32_t estr[3] = {1u, 1u, 1u};
        cuuint64_t st[2] = {(cuuint64_t)st_t * eb, (cuuint64_t)st_b * eb};
        if (a.seqlen == 1) st[0] = (cuuint64_t)a.dim * eb;
        if (a.batch == 1) st[1] = st[0] * (cuuint64_t)a.seqlen;
        if (st[0] % 16 != 0 || st[1] % 16 != 0) return false;
        const cuuint32_t box[3] = {(cuuint32_t)slab_ch, (cuuint32_t)rows, 1u};
        return enc(m, dt, 3, const_cast<void*>(ptr), dims, st, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    };
    CUtensorMap tmap_x, tmap_g;
    if (!make_map(&tmap_x, a.x, a.x_stride_t, a.x_stride_b, G::kXRows)) return cudaErrorNotSupported;
    if (!make_map(&tmap_g, a.dy, a.dy_stride_t, a.dy_stride_b, G::kGRows)) return cudaErrorNotSupported;

    int stages = a.tma_stages > 0 ? a.tma_stages : G::kDefaultStages;
    if (stages < 2) stages = 2;
    if (stages > kMaxStages) stages = kMaxStages;
    const int per_sm = (a.tma_ctas_per_sm > 0 && a.tma_ctas_per_sm <= 8) ? a.tma_ctas_per_sm : G::kCtasPerSm;
    p.stages = stages;
    const bool use_sched = a.scratch != nullptr && 4LL * (n_slab + 1) <= kSchedCounterBytes &&
                           a.scratch_bytes >= kSchedCounterBytes && (reinterpret_cast<uintptr_t>(a.scratch) & 15u) == 0;
    // CTAs per slab: with dynamic claims round up, so that no resident slot stays empty (a CTA that
    // starts late simply claims what is left); with static assignment round down
    const long long slots = (long long)sm_count() * per_sm;
    long long g = use_sched ? (slots + n_slab - 1) / n_slab : slots / n_slab;
    if (g < 1) g = 1;
    if (g > n_rowtiles) g = n_rowtiles;
    if (g > 65535) g = 65535;
    p.ctas_per_slab = (int)g;
    const int smem = G::smem_bytes(stages);
    {
        static std::atomic<int> granted[64];
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev < 0 || dev >= 64 || granted[dev].load(std::memory_order_acquire) < smem) {
            const cudaError_t e = cudaFuncSetAttribute(k_prefill_bwd_tma<DT, W, SLAB_BYTES, ACT, VARIANT>,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (e != cudaSuccess) return e == cudaErrorInvalidValue ? cudaErrorNotSupported : e;
            if (dev >= 0 && dev < 64) granted[dev].store(smem, std::memory_order_release);
        }
    }
    p.sched = nullptr;
    p.gtable = nullptr;
    // gradient accumulators the caller asked the library to clear: by the pre-pass when there is one
    // (no extra launch), else by memsets on the stream
    bool zero_pending = a.zero_grads != 0;
    const int n_dw = a.dweight != nullptr ? a.dim * a.width : 0;
    const int n_db = a.dbias != nullptr ? a.dim : 0;
    if (use_sched) {
        p.sched = reinterpret_cast<unsigned int*>(a.scratch);
        if (p.mask != nullptr && a.scratch_bytes >= kSchedCounterBytes + n_rowtiles) {
            // class of every tile from its R + 2H mask rows (pre-pass shared with the forward kernel)
            TmaParams cp = {};
            cp.mask = p.mask;
            cp.smb = p.smb;
            cp.smt = p.smt;
            cp.mask_dtype = p.mask_dtype;
            cp.seg_mode = p.seg_mode;
            cp.B = a.batch;
            cp.T = a.seqlen;
            cp.n_ttile = p.n_ttile;
            cp.skip = 1;
            cp.res = nullptr;
            cp.init = nullptr;
            unsigned char* tab = reinterpret_cast<unsigned char*>(a.scratch) + kSchedCounterBytes;
            const long long threads = n_rowtiles * 32;
            // (the pre-pass waits for its predecessor before it writes anything: it may start while that one drains)
            cudaLaunchAttribute pattr[1];
            pattr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            pattr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
            cudaLaunchConfig_t pcfg = {};
            pcfg.gridDim = dim3((unsigned)((threads + 255) / 256));
            pcfg.blockDim = dim3(256);
            pcfg.stream = s;
            pcfg.attrs = pattr;
            pcfg.numAttrs = 1;
            const cudaError_t e = cudaLaunchKernelEx(
                &pcfg, k_classify_tiles, cp, tab, (int)G::kTileRows, (int)G::kH, (int)G::kXRows,
                zero_pending ? a.dweight : (float*)nullptr, zero_pending ? n_dw : 0, zero_pending ? a.dbias : (float*)nullptr,
                zero_pending ? n_db : 0, (unsigned short*)nullptr, (unsigned int*)nullptr);
            if (e != cudaSuccess) return e;
            zero_pending = false;
            note_launch("classify");
            p.gtable = tab;
        }
    }
    if (zero_pending) {
        cudaError_t e = n_dw > 0 ? cudaMemsetAsync(a.dweight, 0, sizeof(float) * (size_t)n_dw, s) : cudaSuccess;
        if (e == cudaSuccess && n_db > 0) e = cudaMemsetAsync(a.dbias, 0, sizeof(float) * (size_t)n_db, s);
        if (e != cudaSuccess) return e;
    }
    note_launch("bwd_tma");
    // the main kernel is a programmatic dependent of its predecessor (the pre-pass when there is one): its launch
    // and prologue overlap it
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)n_slab, (unsigned)g);
    cfg.blockDim = dim3(G::kThreads);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, k_prefill_bwd_tma<DT, W, SLAB_BYTES, ACT, VARIANT>, tmap_x, tmap_g, p);
}

template <int DT, int W>
cudaError_t launch_bwd_w(const vc1d_prefill_bwd_args& a, const BwdParams& p, cudaStream_t s) {
    const int eb = Elem<DT>::kBytes;
    const int wide = 256 / eb, narrow = 128 / eb;
    const bool use_wide = (a.dim % wide == 0) || (a.dim % narrow != 0);
    const bool act = a.activation == VC1D_ACT_SILU;
    if constexpr (DT != VC1D_F32) {
        // 16-bit I/O, full-width slabs: one channel pair per thread (see BwdGeometry).  With SiLU the
        // kernel is bound by instruction issue and 16 rows per thread save the most work; without it 8
        // rows per thread measured fastest.
        const int variant = a.tma_variant != 0 ? a.tma_variant : (act ? 3 : 2);
        if (use_wide && variant == 2)
            return act ? launch_bwd_kernel<DT, W, 256, true, 1>(a, p, s) : launch_bwd_kernel<DT, W, 256, false, 1>(a, p, s);
        if (use_wide && variant == 3)
            return act ? launch_bwd_kernel<DT, W, 256, true, 2>(a, p, s) : launch_bwd_kernel<DT, W, 256, false, 2>(a, p, s);
    }
    if (use_wide)
        return act ? launch_bwd_kernel<DT, W, 256, true>(a, p, s) : launch_bwd_kernel<DT, W, 256, false>(a, p, s);
    return act ? launch_bwd_kernel<DT, W, 128, true>(a, p, s) : launch_bwd_kernel<DT, W, 128, false>(a, p, s);
}

template <int DT>
cudaError_t launch_bwd_dt(const vc1d_prefill_bwd_args& a, const BwdParams& p, cudaStream_t s) {
    switch (a.width) {
        case 2: return launch_bwd_w<DT, 2>(a, p, s);
        case 3: return launch_bwd_w<DT, 3>(a, p, s);
        default: return launch_bwd_w<DT, 4>(a, p, s);
    }
}

}  // namespace tma
}  // namespace vc1d
