// TMA-staged prefill kernel for the channel-last layout (reference call site
// model/model.py:459-466; fused mask / residual / final state: model/model.py:454-457,
// 491, 470-489).  Device code and the templated launcher; prefill_tma_<dtype>.cu instantiate it
// per element type, prefill_tma.cu holds the tensor-map encoder and the dispatch.
//
// Geometry.  A tile is kTileRows time rows x one 128- or 256-byte slab of channels of one
// sequence.  Its input box, (kTileRows + W-1) rows starting W-1 rows ABOVE the tile, arrives in
// shared memory by one cp.async.bulk.tensor.3d load (no multicast); rows before t = 0 are
// out of bounds for the tensor map and are zero-filled by the hardware, which is exactly the
// causal left padding.  The grid is (channel slabs) x (persistent CTAs per slab): a CTA keeps
// the weights of its slab in registers for its whole life and walks row tiles
// j, j + G, j + 2G, ... of that slab, so neighbouring CTAs touch neighbouring rows and the
// (W-1)-row halo of a tile is an L2 hit.
//
// Pipeline.  One producer warp and eight consumer warps share a ring of stages guarded by
// full/done mbarriers.  The producer fetches the tile's mask rows two tiles ahead (32 lanes, a
// few loads each) and classifies the tile: all rows valid, mixed, or nothing to read.  A tile
// with nothing to read never enters the ring: no byte of it is requested from HBM and the
// producer warp stores its outputs, act(bias), itself.  Bytes in flight are set by the ring
// depth, not by registers.  Each consumer thread owns 8 bytes of channels and 8 consecutive
// rows of the tile: a register window over shared memory rotated by index, fp32x2 FMAs, fused
// mask / bias / SiLU / residual epilogue, streaming 8-byte stores (a warp writes 256 contiguous
// bytes per row).  No consumer warp waits on HBM for its input, and none waits for another
// warp: the only synchronisation is the pair of mbarriers per stage.
//
// Every mbarrier wait is bounded; on expiry the warp records the event in a device counter
// (read by vc1d_tma_timeouts()) and leaves its loop.
#pragma once

#include <cuda.h>

#include <atomic>
#include <type_traits>

#include "vc1d_common.cuh"
#include "vc1d_internal.h"

namespace vc1d {
namespace tma {

constexpr int kMaxStages = 8;
constexpr unsigned kSpinLimit = 1u << 24;

enum : int { TILE_EMPTY = 0, TILE_MIXED = 1, TILE_FULL = 2, TILE_END = 3 };

struct TmaParams {
    char* y;
    long long syb, syt;
    const char* x;  // for the final-state pass
    const char* res;
    const void* weight;
    const void* bias;
    const void* mask;
    char* fstate;
    unsigned int* timeouts;  // device counter of expired waits
    long long sxb, sxt;  // bytes
    long long srb, srt;
    long long smb, smt;  // elements
    long long wsd, wsw;
    int wdtype;
    int B, D, T;
    int n_ttile, n_rowtiles, ctas_per_slab;
    int mask_dtype;
    int skip;
    int res_is_x;
    int state_len;
    int stages;      // ring depth (2..kMaxStages)
};

// ---- raw PTX wrappers -----------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the limit expired.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (unsigned i = 0; i < kSpinLimit; ++i) {
        if (mbar_test(bar, parity)) return true;
        if (i > 64) __nanosleep(64);
    }
    return false;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
        : "memory");
}
__device__ __forceinline__ float lds_f32(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ int lds_s32(uint32_t a) {
    int v;
    asm volatile("ld.volatile.shared.s32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts_s32(uint32_t a, int v) {
    asm volatile("st.volatile.shared.s32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}
__device__ __forceinline__ void sts_f32(uint32_t a, float v) {
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory");
}

// Walks the row tiles j0, j0 + G, j0 + 2G, ... of one CTA without a division per tile.  Tile
// number rt means sequence b = rt / n_ttile and time position (rt % n_ttile + b) % n_ttile: the
// position is rotated by the sequence index so that a CTA does not keep meeting the same position
// of every sequence (with right-padded batches the late positions are the cheap, masked ones).
struct TileIter {
    int b, r, brot;        // sequence, rt % n_ttile, b % n_ttile
    int n, sb, sr, sbrot;  // n_ttile, G / n_ttile, G % n_ttile, sb % n_ttile
    __device__ __forceinline__ void init(int rt, int n_ttile, int stride) {
        n = n_ttile;
        b = rt / n;
        r = rt - b * n;
        brot = b % n;
        sb = stride / n;
        sr = stride - sb * n;
        sbrot = sb % n;
    }
    __device__ __forceinline__ void next() {
        b += sb;
        brot += sbrot;
        if (brot >= n) brot -= n;
        r += sr;
        if (r >= n) {
            r -= n;
            ++b;
            if (++brot == n) brot = 0;
        }
    }
    __device__ __forceinline__ int t0(int tile_rows) const {
        int tt = r + brot;
        if (tt >= n) tt -= n;
        return tt * tile_rows;
    }
};

template <int DT, int W, int SLAB_BYTES, int VB, int RPT>
struct Geometry {
    static constexpr int kH = W - 1;
    static constexpr int kRows = RPT;  // consecutive rows one thread computes per tile
    static constexpr int kLanesPerRow = SLAB_BYTES / VB;
    static constexpr int kConsumerWarps = (VB == 16) ? 4 : 8;
    static constexpr int kConsumerThreads = kConsumerWarps * 32;
    static constexpr int kThreads = kConsumerThreads + 32;
    static constexpr int kGroups = kConsumerThreads / kLanesPerRow;  // row groups per tile
    static constexpr int kTileRows = kGroups * RPT;
    static constexpr int kBoxRows = kTileRows + kH;
    static constexpr int kRowBytes = SLAB_BYTES;
    static constexpr int kSlabElems = SLAB_BYTES / Elem<DT>::kBytes;
    static constexpr int kStageBytes = ((kBoxRows * kRowBytes + 127) / 128) * 128;
    static constexpr int kMaskFloats = ((kBoxRows + 31) / 32) * 32;
    // layout for S stages: stages | mask floats | full[S], done[S] | {class, b, t0}[S], abort
    __host__ __device__ static constexpr int off_mask(int S) { return S * kStageBytes; }
    __host__ __device__ static constexpr int off_bars(int S) { return off_mask(S) + S * kMaskFloats * 4; }
    __host__ __device__ static constexpr int off_flags(int S) { return off_bars(S) + 2 * S * 8; }
    __host__ __device__ static constexpr int smem_bytes(int S) {
        return off_flags(S) + (3 * S + 1) * 4 + 128 /* base alignment slack */;
    }
};

// Weights and bias of this thread's channels as fp32 pairs; zeros for channels past dim.
template <int DT, int W, int VB>
__device__ __forceinline__ void load_weights(const TmaParams& p, int d0, bool in_range,
                                             float2 (&wp)[W][Slice<DT, VB>::kPairs],
                                             float2 (&bp)[Slice<DT, VB>::kPairs]) {
    using E = Elem<DT>;
    using T = typename E::type;
    constexpr int NE = Slice<DT, VB>::kElems;
    constexpr int NP = Slice<DT, VB>::kPairs;
    float wf[NE][W];
    float bf[NE];
#pragma unroll
    for (int c = 0; c < NE; ++c) {
        bf[c] = 0.f;
#pragma unroll
        for (int w = 0; w < W; ++w) wf[c][w] = 0.f;
    }
    if (in_range) {
#pragma unroll
        for (int c = 0; c < NE; ++c) {
#pragma unroll
            for (int w = 0; w < W; ++w) {
                const long long idx = (long long)(d0 + c) * p.wsd + (long long)w * p.wsw;
                wf[c][w] = (p.wdtype == VC1D_F32) ? __ldg(reinterpret_cast<const float*>(p.weight) + idx)
                                                  : E::to_float(__ldg(reinterpret_cast<const T*>(p.weight) + idx));
            }
            if (p.bias != nullptr) {
                bf[c] = (p.wdtype == VC1D_F32) ? __ldg(reinterpret_cast<const float*>(p.bias) + d0 + c)
                                               : E::to_float(__ldg(reinterpret_cast<const T*>(p.bias) + d0 + c));
            }
        }
    }
#pragma unroll
    for (int q = 0; q < NP; ++q) {
#pragma unroll
        for (int w = 0; w < W; ++w) wp[w][q] = make_float2(wf[2 * q][w], wf[2 * q + 1][w]);
        bp[q] = make_float2(bf[2 * q], bf[2 * q + 1]);
    }
}

// One staged row -> fp32 pairs with the reference's multiplicative mask (x * mask rounded to the
// I/O dtype); with skip_masked_loads a zero mask makes the row +0 whatever it holds.
template <int DT, int VB>
__device__ __forceinline__ void apply_mask(float2 (&f)[Slice<DT, VB>::kPairs], float mk, int skip) {
    constexpr int NP = Slice<DT, VB>::kPairs;
    if (mk != 1.0f) {
        if (mk == 0.0f && skip) {
#pragma unroll
            for (int q = 0; q < NP; ++q) f[q] = make_float2(0.f, 0.f);
        } else {
            const float2 m2 = make_float2(mk, mk);
#pragma unroll
            for (int q = 0; q < NP; ++q) f[q] = Slice<DT, VB>::round_trip(mul2(f[q], m2));
        }
    }
}

// The R rows of one thread in one tile.  GENERAL adds the per-row mask and the residual.  Results go
// straight to global memory with streaming stores (yrow is the address of the thread's first row).
template <int DT, int W, int VB, int RPT, bool ACT, bool GENERAL, int ROW_BYTES>
__device__ __forceinline__ void process_rows(uint32_t trow, uint32_t mk_addr, const TmaParams& p, bool mixed,
                                             const char* rb, char* yrow, int tfirst, int rows_ok,
                                             float2 (&hist)[W - 1 > 0 ? W - 1 : 1][Slice<DT, VB>::kPairs],
                                             const float2 (&wp)[W][Slice<DT, VB>::kPairs],
                                             const float2 (&bp)[Slice<DT, VB>::kPairs]) {
    using S = Slice<DT, VB>;
    using E = Elem<DT>;
    constexpr int NP = S::kPairs;
    constexpr int NW = S::kWords;
    constexpr int H = W - 1;
    // Unrolled at the language level: every index below is a compile-time constant, and the history
    // window rotates by index (row k overwrites slot k % H, the oldest) instead of by moving registers.
    static_for<0, RPT>([&](auto kc) {
        constexpr int k = decltype(kc)::value;
        const uint32_t slot = trow + (H + k) * ROW_BYTES;
        uint32_t raw[NW];
        S::lds(slot, raw);
        float2 cur[NP];
        S::unpack(raw, cur);
        if constexpr (GENERAL) {
            if (mixed) apply_mask<DT, VB>(cur, lds_f32(mk_addr + (H + k) * 4), p.skip);
        }
        float2 acc[NP];
#pragma unroll
        for (int q = 0; q < NP; ++q) {
            acc[q] = bp[q];
#pragma unroll
            for (int w = 0; w < H; ++w) acc[q] = fma2(wp[w][q], hist[(k + w) % (H > 0 ? H : 1)][q], acc[q]);
            acc[q] = fma2(wp[H][q], cur[q], acc[q]);
            if constexpr (ACT) acc[q] = silu2<E::kPreciseSilu>(acc[q]);
        }
        if constexpr (GENERAL) {
            if (p.res != nullptr) {
                float2 rr[NP];
                if (p.res_is_x) {
                    S::unpack(raw, rr);  // the unmasked input, already on chip
                } else {
                    uint32_t rv[NW];
#pragma unroll
                    for (int i = 0; i < NW; ++i) rv[i] = 0u;
                    const int t = tfirst + k;
                    if (rb != nullptr && t < p.T) {
                        const uint32_t* src = reinterpret_cast<const uint32_t*>(rb + (long long)t * p.srt);
#pragma unroll
                        for (int i = 0; i < NW; ++i) rv[i] = __ldg(src + i);
                    }
                    S::unpack(rv, rr);
                }
#pragma unroll
                for (int q = 0; q < NP; ++q) acc[q] = add2(S::round_trip(acc[q]), rr[q]);
            }
        }
        uint32_t outw[NW];
        S::pack(acc, outw);
        if (rows_ok > k) S::stg(yrow + (long long)k * p.syt, outw);
        if constexpr (H > 0) {
#pragma unroll
            for (int q = 0; q < NP; ++q) hist[k % H][q] = cur[q];
        }
    });
}

// Mask values of one tile's box rows, kBoxRows spread over the 32 lanes of the producer warp.
template <int NMK, int BOX_ROWS, int H, int TILE_ROWS>
__device__ __forceinline__ void fetch_mask(const TmaParams& p, int b, int t0, int lane, float (&mk)[NMK]) {
#pragma unroll
    for (int q = 0; q < NMK; ++q) {
        const int jrow = lane + 32 * q;
        const int t = t0 - H + jrow;
        float v = 1.0f;                        // rows before t = 0 are zero-filled data: any multiplier works
        if (jrow < BOX_ROWS) {
            if (t >= p.T) v = 0.0f;            // rows past the end are never stored
            else if (t >= 0) v = load_mask(p.mask, (long long)b * p.smb + (long long)t * p.smt, p.mask_dtype);
        }
        mk[q] = v;
    }
}

template <int DT, int W, int SLAB_BYTES, int VB, int RPT, bool ACT>
__global__ void __launch_bounds__(Geometry<DT, W, SLAB_BYTES, VB, RPT>::kThreads)
    k_prefill_tma(const __grid_constant__ CUtensorMap tmap_x, const TmaParams p) {
    using E = Elem<DT>;
    using S = Slice<DT, VB>;
    using G = Geometry<DT, W, SLAB_BYTES, VB, RPT>;
    constexpr int NE = S::kElems;
    constexpr int NP = S::kPairs;
    constexpr int NW = S::kWords;
    constexpr int H = G::kH;
    constexpr int R = RPT;
    constexpr int LPR = G::kLanesPerRow;
    constexpr int NMK = (G::kBoxRows + 31) / 32;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 127u) & ~127u;
    const int kStages = p.stages;  // ring depth of this launch
    const uint32_t mask_base = base + G::off_mask(kStages);
    const uint32_t bars = base + G::off_bars(kStages);    // full[s] at bars + 8 s, done[s] at bars + 8 (kStages + s)
    const uint32_t flags = base + G::off_flags(kStages);  // per stage {class, sequence, first row}; then the abort flag
    const uint32_t abort_c = flags + 12 * kStages;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int slab = blockIdx.x;
    const int j0 = blockIdx.y;
    const int stride = p.ctas_per_slab;
    const int slab_ch0 = slab * G::kSlabElems;
    const int n_my = (j0 < p.n_rowtiles) ? (p.n_rowtiles - j0 + stride - 1) / stride : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bars + 8 * s, 1);                              // full: the producer's arrive (+ tx bytes)
            mbar_init(bars + 8 * (kStages + s), G::kConsumerWarps);  // done: one arrive per consumer warp
        }
        sts_s32(abort_c, 0);  // a consumer wait expired
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == G::kConsumerWarps) {
        // ================================ producer warp ==================================
        // Walks the CTA's tiles in order.  A tile with something to read takes the next ring slot
        // (after the consumers of the slot's previous tile have arrived on done[s]) and is loaded
        // by one bulk tensor copy.  A tile in which every tap of every row is masked never enters
        // the ring: its outputs are act(bias), and this warp -- one lane per 8 bytes of the slab
        // row -- stores them itself.  After the last tile an END marker takes a slot.  The mask of
        // tile i+2 is fetched while tile i is handled, in three register buffers that rotate roles
        // (the loop is unrolled by three), so the fetched values are not touched until needed.
        using S8 = Slice<DT, 8>;
        constexpr int NE8 = S8::kElems;
        const int pd0 = slab_ch0 + lane * NE8;  // this lane's channels when it stores a masked-out tile
        const bool p_ok = lane * 8 < SLAB_BYTES && pd0 < p.D;
        uint32_t pconst[2] = {0u, 0u};
        if (p.mask != nullptr && p_ok) {
            float2 c[S8::kPairs];
#pragma unroll
            for (int q = 0; q < S8::kPairs; ++q) {
                float v[2] = {0.f, 0.f};
                if (p.bias != nullptr) {
#pragma unroll
                    for (int e = 0; e < 2; ++e)
                        v[e] = (p.wdtype == VC1D_F32)
                                   ? __ldg(reinterpret_cast<const float*>(p.bias) + pd0 + 2 * q + e)
                                   : E::to_float(__ldg(reinterpret_cast<const typename E::type*>(p.bias) + pd0 + 2 * q + e));
                }
                c[q] = make_float2(v[0], v[1]);
                if (ACT) c[q] = silu2<E::kPreciseSilu>(c[q]);
            }
            S8::pack(c, pconst);
        }
        TileIter it_fetch, it_load;  // tiles i+2 (mask fetch) and i (load)
        it_load.init(j0, p.n_ttile, stride);
        it_fetch = it_load;
        int s_ring = 0, n_ring = 0;  // next ring slot, tiles put into the ring so far
        uint32_t ph_ring = 0;        // how often the ring has wrapped, mod 2
        // claim the next slot: wait until its previous tile has been consumed
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
        auto step = [&](int i, float (&mk_use)[NMK], float (&mk_fill)[NMK]) -> bool {
            if (p.mask != nullptr && i + 2 < n_my) {
                it_fetch.next();
                fetch_mask<NMK, G::kBoxRows, H, G::kTileRows>(p, it_fetch.b, it_fetch.t0(G::kTileRows), lane, mk_fill);
            }
            const int b = it_load.b;
            const int t0 = it_load.t0(G::kTileRows);
            int cls = TILE_FULL;
            if (p.mask != nullptr) {
                bool any = false, all_one = true;
#pragma unroll
                for (int q = 0; q < NMK; ++q) {
                    const int jrow = lane + 32 * q;
                    const int t = t0 - H + jrow;
                    if (jrow < G::kBoxRows && t >= 0 && t < p.T) {
                        any |= (mk_use[q] != 0.0f);
                        all_one &= (mk_use[q] == 1.0f);
                    }
                }
                any = __any_sync(0xffffffffu, any);
                all_one = __all_sync(0xffffffffu, all_one);
                cls = all_one ? TILE_FULL : ((any || !p.skip || p.res != nullptr) ? TILE_MIXED : TILE_EMPTY);
            }
            if (cls == TILE_EMPTY) {
                if (p_ok) {
                    char* yrow = p.y + (long long)b * p.syb + (long long)t0 * p.syt + (long long)pd0 * E::kBytes;
                    const int nrows = min(G::kTileRows, p.T - t0);
                    for (int r = 0; r < nrows; ++r) S8::stg(yrow + (long long)r * p.syt, pconst);
                }
            } else {
                if (!claim()) return false;
                const int s = s_ring;
                if (cls == TILE_MIXED) {
#pragma unroll
                    for (int q = 0; q < NMK; ++q) {
                        const int jrow = lane + 32 * q;
                        if (jrow < G::kBoxRows) sts_f32(mask_base + (s * G::kMaskFloats + jrow) * 4, mk_use[q]);
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    sts_s32(flags + 12 * s, cls);
                    sts_s32(flags + 12 * s + 4, b);
                    sts_s32(flags + 12 * s + 8, t0);
                    const uint32_t full = bars + 8 * s;
                    mbar_arrive_expect_tx(full, G::kBoxRows * G::kRowBytes);
                    tma_load_3d(base + s * G::kStageBytes, &tmap_x, slab_ch0, t0 - H, b, full);
                }
                __syncwarp();
                advance();
            }
            it_load.next();
            return true;
        };
        float mk_a[NMK], mk_b[NMK], mk_c[NMK];
#pragma unroll
        for (int q = 0; q < NMK; ++q) mk_a[q] = mk_b[q] = mk_c[q] = 1.0f;
        if (p.mask != nullptr && n_my > 0)
            fetch_mask<NMK, G::kBoxRows, H, G::kTileRows>(p, it_fetch.b, it_fetch.t0(G::kTileRows), lane, mk_a);
        if (p.mask != nullptr && n_my > 1) {
            it_fetch.next();
            fetch_mask<NMK, G::kBoxRows, H, G::kTileRows>(p, it_fetch.b, it_fetch.t0(G::kTileRows), lane, mk_b);
        }
        bool live = true;
        for (int i = 0; live && i < n_my; i += 3) {
            live = step(i, mk_a, mk_c);
            if (live && i + 1 < n_my) live = step(i + 1, mk_b, mk_a);
            if (live && i + 2 < n_my) live = step(i + 2, mk_c, mk_b);
        }
        // END marker: the consumers leave when they meet it
        if (live && claim()) {
            if (lane == 0) {
                sts_s32(flags + 12 * s_ring, TILE_END);
                mbar_arrive(bars + 8 * s_ring);
            }
            __syncwarp();
        }
    } else {
        // ================================ consumer warps =================================
        const int grp = threadIdx.x / LPR;  // row group inside the tile
        const int cl = threadIdx.x % LPR;   // channel slice inside the slab
        const int d0 = slab_ch0 + cl * NE;
        const bool ch_ok = d0 < p.D;  // dim is a multiple of the 128-bit vector: a slice is in or out as a whole
        const int rbase = grp * R;

        float2 wp[W][NP];
        float2 bp[NP];
        load_weights<DT, W, VB>(p, d0, ch_ok, wp, bp);
        const bool general_kernel = (p.mask != nullptr) || (p.res != nullptr);

        int s = -1;
        uint32_t ph = 1;
        for (;;) {
            if (++s == kStages) s = 0;
            if (s == 0) ph ^= 1;
            if (!mbar_wait(bars + 8 * s, ph)) {
                if (lane == 0) atomicAdd(p.timeouts, 1u);
                break;  // no barrier is shared with the other warps: each leaves on its own
            }
            const int cls = lds_s32(flags + 12 * s);
            if (cls == TILE_END) break;
            // box row of time t is (t - t0 + H); this thread reads box rows rbase .. rbase+R+H-1
            const uint32_t trow = base + s * G::kStageBytes + rbase * G::kRowBytes + cl * VB;
            const uint32_t mk_addr = mask_base + (s * G::kMaskFloats + rbase) * 4;
            const bool mixed = (cls == TILE_MIXED);
            const int b = lds_s32(flags + 12 * s + 4);
            const int tfirst = lds_s32(flags + 12 * s + 8) + rbase;

            float2 hist[H > 0 ? H : 1][NP];
#pragma unroll
            for (int w = 0; w < H; ++w) {
                uint32_t raw[NW];
                S::lds(trow + w * G::kRowBytes, raw);
                S::unpack(raw, hist[w]);
                if (mixed) apply_mask<DT, VB>(hist[w], lds_f32(mk_addr + w * 4), p.skip);
            }
            // rows of this thread that exist in the output
            const int rows_ok = ch_ok ? min(R, max(0, p.T - tfirst)) : 0;
            char* yrow = p.y + (long long)b * p.syb + (long long)tfirst * p.syt + (long long)d0 * E::kBytes;
            const char* rb = nullptr;
            if (p.res != nullptr && !p.res_is_x && ch_ok)
                rb = p.res + (long long)b * p.srb + (long long)d0 * E::kBytes;

            if (!general_kernel || (cls == TILE_FULL && p.res == nullptr)) {
                process_rows<DT, W, VB, RPT, ACT, false, G::kRowBytes>(trow, mk_addr, p, false, nullptr, yrow, tfirst,
                                                                       rows_ok, hist, wp, bp);
            } else {
                process_rows<DT, W, VB, RPT, ACT, true, G::kRowBytes>(trow, mk_addr, p, mixed, rb, yrow, tfirst,
                                                                      rows_ok, hist, wp, bp);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + 8 * (kStages + s));  // the stage has been read
        }

        // ---- final state: right-aligned last state_len masked inputs (model/model.py:470-489) ----
        if (p.fstate != nullptr && threadIdx.x < LPR && ch_ok) {
            using T = typename E::type;
            const int L = p.state_len;
            for (int b = j0; b < p.B; b += stride) {
                const T* xb = reinterpret_cast<const T*>(p.x + (long long)b * p.sxb) + d0;
                T* out = reinterpret_cast<T*>(p.fstate) + ((long long)b * p.D + d0) * L;
                for (int jc = 0; jc < L; ++jc) {
                    const int t = p.T - L + jc;
                    float mkv = 1.0f;
                    if (t >= 0 && p.mask != nullptr)
                        mkv = load_mask(p.mask, (long long)b * p.smb + (long long)t * p.smt, p.mask_dtype);
#pragma unroll
                    for (int c = 0; c < NE; ++c) {
                        T v = E::from_float(0.f);
                        if (t >= 0) {
                            v = xb[(long long)t * (p.sxt / E::kBytes) + c];
                            if (mkv != 1.0f) v = E::from_float(E::to_float(v) * mkv);
                        }
                        out[(long long)c * L + jc] = v;
                    }
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn encode_fn();

template <int DT, int W, int SLAB_BYTES, int VB, int RPT, bool ACT>
cudaError_t launch_kernel(const vc1d_prefill_args& a, const TmaParams& base, cudaStream_t s) {
    using G = Geometry<DT, W, SLAB_BYTES, VB, RPT>;
    const int eb = Elem<DT>::kBytes;
    TmaParams p = base;
    const int slab_ch = G::kSlabElems;
    const int n_slab = (a.dim + slab_ch - 1) / slab_ch;
    p.n_ttile = (a.seqlen + G::kTileRows - 1) / G::kTileRows;
    const long long n_rowtiles = (long long)a.batch * p.n_ttile;
    if (n_rowtiles > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    p.n_rowtiles = (int)n_rowtiles;

    EncodeFn enc = encode_fn();
    if (enc == nullptr) return cudaErrorNotSupported;
    const CUtensorMapDataType dt = (DT == VC1D_F32)    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : (DT == VC1D_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                       : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    // input box: the tile's rows plus the W-1 rows above them
    CUtensorMap tmap_x;
    {
        const cuuint64_t dims[3] = {(cuuint64_t)a.dim, (cuuint64_t)a.seqlen, (cuuint64_t)a.batch};
        const cuuint32_t estr[3] = {1u, 1u, 1u};
        cuuint64_t st[2] = {(cuuint64_t)a.x_stride_t * eb, (cuuint64_t)a.x_stride_b * eb};
        // an extent of 1 makes its stride irrelevant, but the encoder still wants a legal value
        if (a.seqlen == 1) st[0] = (cuuint64_t)a.dim * eb;
        if (a.batch == 1) st[1] = st[0] * (cuuint64_t)a.seqlen;
        if (st[0] % 16 != 0 || st[1] % 16 != 0) return cudaErrorNotSupported;
        const cuuint32_t box[3] = {(cuuint32_t)slab_ch, (cuuint32_t)G::kBoxRows, 1u};
        const CUresult r = enc(&tmap_x, dt, 3, const_cast<void*>(a.x), dims, st, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorNotSupported;  // the caller falls back to the direct kernel
    }
    int stages = a.tma_stages > 0 ? a.tma_stages : 3;
    if (stages < 2) stages = 2;
    if (stages > kMaxStages) stages = kMaxStages;
    int per_sm = (a.tma_ctas_per_sm > 0 && a.tma_ctas_per_sm <= 32) ? a.tma_ctas_per_sm : 3;
    while (stages > 2 && G::smem_bytes(stages) > 200 * 1024) --stages;
    p.stages = stages;
    const int smem = G::smem_bytes(stages);
    {
        // opt in to > 48 KB of dynamic shared memory; the attribute is per device and sticky, so
        // remember the largest value set so far
        static std::atomic<int> granted[64];
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev < 0 || dev >= 64 || granted[dev].load(std::memory_order_acquire) < smem) {
            const cudaError_t e = cudaFuncSetAttribute(k_prefill_tma<DT, W, SLAB_BYTES, VB, RPT, ACT>,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 64) granted[dev].store(smem, std::memory_order_release);
        }
    }
    // persistent CTAs, split evenly over the channel slabs
    long long g = ((long long)sm_count() * per_sm) / n_slab;
    if (g < 1) g = 1;
    if (g > n_rowtiles) g = n_rowtiles;
    if (g > 65535) g = 65535;
    p.ctas_per_slab = (int)g;
    const dim3 grid((unsigned)n_slab, (unsigned)g);
    note_launch("tma");
    k_prefill_tma<DT, W, SLAB_BYTES, VB, RPT, ACT><<<grid, G::kThreads, smem, s>>>(tmap_x, p);
    return cudaGetLastError();
}

template <int DT, int W, int SLAB_BYTES>
cudaError_t launch_slab(const vc1d_prefill_args& a, const TmaParams& p, cudaStream_t s) {
    // 8 bytes of channels and 8 rows per thread; 4 rows (half-height tiles) on request
    const bool act = a.activation == VC1D_ACT_SILU;
    if (a.tma_rows_per_thread == 4)
        return act ? launch_kernel<DT, W, SLAB_BYTES, 8, 4, true>(a, p, s)
                   : launch_kernel<DT, W, SLAB_BYTES, 8, 4, false>(a, p, s);
    return act ? launch_kernel<DT, W, SLAB_BYTES, 8, 8, true>(a, p, s)
               : launch_kernel<DT, W, SLAB_BYTES, 8, 8, false>(a, p, s);
}

template <int DT, int W>
cudaError_t launch_w(const vc1d_prefill_args& a, const TmaParams& p, cudaStream_t s) {
    // 256-byte slabs when dim fills them; 128-byte slabs when that avoids idle lanes
    const int eb = Elem<DT>::kBytes;
    const int wide = 256 / eb, narrow = 128 / eb;
    bool use_wide = (a.dim % wide == 0) || (a.dim % narrow != 0);
    if (a.tma_slab_bytes == 128) use_wide = false;
    if (a.tma_slab_bytes == 256) use_wide = true;
    return use_wide ? launch_slab<DT, W, 256>(a, p, s) : launch_slab<DT, W, 128>(a, p, s);
}

template <int DT>
cudaError_t launch_dt(const vc1d_prefill_args& a, const TmaParams& p, cudaStream_t s) {
    switch (a.width) {
        case 2: return launch_w<DT, 2>(a, p, s);
        case 3: return launch_w<DT, 3>(a, p, s);
        default: return launch_w<DT, 4>(a, p, s);
    }
}

}  // namespace tma
}  // namespace vc1d
