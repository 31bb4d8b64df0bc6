// TMA-staged prefill kernel for the channel-last layout (reference call site
// model/model.py:459-466; fused mask / residual / final state: model/model.py:454-457,
// 491, 470-489).  Device code and the templated launcher; prefill_tma_<dtype>.cu instantiate it
// per element type, prefill_tma.cu holds the tensor-map encoder and the dispatch.
//
// Geometry.  A tile is kTileRows time rows x one 128- or 256-byte slab of channels of one
// sequence.  Its input box, (kTileRows + W-1) rows starting W-1 rows ABOVE the tile, arrives in
// shared memory by one cp.async.bulk.tensor.3d load issued by its own CTA; rows before t = 0 are
// out of bounds for the tensor map and are zero-filled by the hardware, which is exactly the
// causal left padding (with an initial state, the first tile of a sequence reads those rows from
// the state instead).  The grid is (channel slabs) x (persistent CTAs per slab): a CTA keeps the
// weights of its slab in registers for its whole life.
//
// Which tile a CTA takes next.  With scratch memory from the caller, the CTAs of a slab claim
// tiles from one counter per slab (atomicAdd, one tile ahead; a CTA's first tiles need no claim),
// so a CTA that met cheap tiles or runs on a faster SM takes more; the last CTA to finish resets
// the counters.  Without scratch, or when a CTA would own fewer than four tiles, CTA j of a slab
// walks tiles j, j + G, j + 2G, ...  Either way neighbouring CTAs touch neighbouring rows at
// about the same time, so the (W-1)-row halo of a tile is an L2 hit.
//
// Masks.  Every tile has a class: all of its mask rows are one (the maskless code runs), mixed, or
// every tap of every row is masked.  A tile of the last class is never loaded and never reaches
// the consumers: its rows are all act(bias), and the producer writes them with bulk tensor stores
// out of a few constant rows the CTA keeps in shared memory (when y cannot be described by a
// tensor map the tile takes a ring slot without a copy and the consumers store it).  The classes
// come from a pre-pass kernel (one byte per tile in scratch memory, copied to shared memory by
// every CTA, two bits per tile for very long batches) or, without scratch, from the CTA's own
// prologue; the main kernel is launched as a programmatic dependent of the pre-pass.  Mask values
// are looked at again only inside mixed tiles.
//
// Packed rows.  With sequence ids instead of a mask (several sequences laid end to end in one
// row) the per-row value that travels the mask's path says "a sequence starts here"; a tile
// without a start in its rows is an ordinary tile, in the others the consumers clear their
// history window at every start.
//
// Pipeline.  One producer warp and eight consumer warps share a ring of stages guarded by
// full/done mbarriers.  For every tile the producer writes a 32-byte descriptor (class, rows that
// exist, 64-bit offset of the first output row, sequence, first row) next to the stage, so the
// consumers do no index arithmetic.  Bytes in flight are set by the ring depth, not by registers.
// Each consumer thread owns 8 bytes of channels and 8 consecutive rows of the tile: a register
// window over shared memory rotated by index, packed fp32x2 FMAs, fused mask / bias / SiLU /
// residual epilogue, streaming 8-byte stores predicated inside the instruction (a warp writes 256
// contiguous bytes per row).  No consumer warp waits on HBM for its input, and none waits for
// another warp: the only synchronisation is the pair of mbarriers per stage.
//
// Every mbarrier wait is bounded; on expiry the warp records the event in a device counter
// (read by vc1d_tma_timeouts()) and leaves its loop.
#pragma once

#include <cuda.h>

#include <atomic>
#include <cstdlib>
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
    const char* init;   // initial state [B, D, init_len] (history instead of zeros left of t = 0), or NULL
    const void* weight;
    const void* bias;
    const void* mask;
    char* fstate;
    unsigned int* timeouts;  // device counter of expired waits
    unsigned int* sched;     // dynamic tile scheduler: one counter per channel slab + one CTA counter, or NULL
    const unsigned char* gtable;  // class of every (sequence, time tile), written by k_classify_tiles, or NULL
    long long sxb, sxt;  // bytes
    long long srb, srt;
    long long smb, smt;  // elements
    long long wsd, wsw;
    int wdtype;
    int B, D, T;
    int n_ttile, n_rowtiles, ctas_per_slab;
    int mask_dtype;
    int skip;
    int init_len;
    int res_is_x;
    int table_in_smem;  // every CTA copies the pre-pass class table to shared memory: 1 = a byte per tile, 2 = two bits,
                        // 3 = the pre-pass wrote an ordered tile list instead (16 bits per claim position)
    int state_len;
    int stages;      // ring depth (2..kMaxStages)
    int seg_mode;    // mask holds int32 sequence ids (packed variable-length rows), not multipliers
    int chunk;       // consecutive tiles per dynamic claim
    int empty_tma;   // tiles without any live tap are written by one bulk tensor store each
    int inline_cls;  // every CTA classifies all tiles itself (consumer warps, while the first tile is in flight)
    int table_early;  // the table or list was written by an earlier launch's pre-pass: it may be read before the
                      // grid dependency wait
    int mask_vec;    // mask rows are contiguous and 16-byte aligned: whole tiles are classified with 128-bit loads
    int static_first;  // tiles a CTA takes without a claim (j0, j0 + G, ...) before the counter hands out the rest
    unsigned spin_limit;  // polls after which a wait gives up
    int test_withhold;    // self-test of the bounded waits: every producer keeps its first tile to itself
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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned limit = kSpinLimit) {
    for (unsigned i = 0; i < limit; ++i) {
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
// One bulk tensor store of a whole tile from shared memory; rows and channels outside the tensor
// are clipped by the tensor map.  Completion is tracked by the issuing thread's bulk groups.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, int c0, int c1, int c2, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(map), "r"(c0),
                 "r"(c1), "r"(c2), "r"(src)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// until the bulk stores committed so far have read their shared-memory source (their writes to global memory
// are complete, like every other store, when the grid is)
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void prefetch_tensormap(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
// makes this thread's earlier shared-memory writes visible to bulk copies issued afterwards
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ float lds_f32(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts_f32(uint32_t a, float v) {
    asm volatile("st.volatile.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory");
}
__device__ __forceinline__ int lds_s32(uint32_t a) {
    int v;
    asm volatile("ld.volatile.shared.s32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts_s32(uint32_t a, int v) {
    asm volatile("st.volatile.shared.s32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}
// tile descriptor head: {class, rows that exist, 64-bit output offset} in one 16-byte access
__device__ __forceinline__ void sts_desc(uint32_t a, int cls, int rows, long long yoff) {
    asm volatile("st.volatile.shared.v4.s32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(cls), "r"(rows),
                 "r"((int)(unsigned)(unsigned long long)yoff), "r"((int)(unsigned)((unsigned long long)yoff >> 32))
                 : "memory");
}
__device__ __forceinline__ void lds_desc(uint32_t a, int& cls, int& rows, long long& yoff) {
    unsigned lo, hi;
    asm volatile("ld.volatile.shared.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(cls), "=r"(rows), "=r"(lo), "=r"(hi) : "r"(a));
    yoff = (long long)(((unsigned long long)hi << 32) | lo);
}
__device__ __forceinline__ int lds_u16(uint32_t a) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return (int)v;
}
__device__ __forceinline__ int lds_u8(uint32_t a) {
    int v;
    asm volatile("ld.volatile.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts_u8(uint32_t a, int v) {
    asm volatile("st.volatile.shared.u8 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}

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
    // kConstRows rows of act(bias), the source of the bulk stores of tiles without a live tap (a tile is
    // written by kTileRows / kConstRows stores: the rows are all alike, and shared memory is better spent
    // on the ring and the class table)
    static constexpr int kConstRows = 16;
    static constexpr int kConstBytes = kConstRows * kRowBytes;
    static_assert(kTileRows % kConstRows == 0 && kConstRows % RPT == 0, "whole row groups fill the constant rows");
    // layout for S stages (C = 1 with the constant tile): stages | constant tile | full[S], done[S],
    // constant-tile-ready | tile descriptor[S] | mask values[S] | class table (one byte per tile)
    // tile descriptor, 32 bytes: {class, rows of the tile that exist, byte offset of its first output
    // row (64 bits)} {sequence, first row, -, -}
    __host__ __device__ static constexpr int off_const(int S) { return S * kStageBytes; }
    __host__ __device__ static constexpr int off_bars(int S, int C) { return off_const(S) + C * kConstBytes; }
    __host__ __device__ static constexpr int off_flags(int S, int C) { return off_bars(S, C) + (2 * S + 2) * 8; }
    // mask values of a mixed tile's box rows, one float per row, written by the producer
    static constexpr int kMaskBytes = ((kBoxRows + 31) / 32) * 32 * 4;
    __host__ __device__ static constexpr int off_mvals(int S, int C) { return off_flags(S, C) + S * 32; }
    __host__ __device__ static constexpr int off_table(int S, int C) { return off_mvals(S, C) + S * kMaskBytes; }
    __host__ __device__ static constexpr int smem_bytes(int S, int C, int table_bytes) {
        return off_table(S, C) + table_bytes + 128 /* base alignment slack */;
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

// Mask multiplier of time row t of the sequence whose mask row starts at element mrow.  Rows before
// t = 0 hold zero-filled data (any multiplier works); rows past the end are never stored.
// With sequence ids instead of a mask the value is kSegStart where a new sequence begins (the taps
// of that row and of the rows after it must not reach above it) and one elsewhere.
constexpr float kSegStart = 2.0f;
__device__ __forceinline__ float tile_mask(const TmaParams& p, long long mrow, int t) {
    if (t < 0 || t >= p.T) return 1.0f;
    if (p.seg_mode) {
        if (t == 0) return 1.0f;  // rows above the tensor arrive as zeros anyway
        const int* ids = reinterpret_cast<const int*>(p.mask) + mrow + (long long)t * p.smt;
        return __ldg(ids) != __ldg(ids - p.smt) ? kSegStart : 1.0f;
    }
    return load_mask(p.mask, mrow + (long long)t * p.smt, p.mask_dtype);
}

// Address of row K of a thread's rows: one widening multiply-add.
template <int K>
__device__ __forceinline__ char* row_addr(char* yrow, unsigned pitch) {
    if constexpr (K == 0) return yrow;
    unsigned long long r;
    asm("mad.wide.u32 %0, %1, %2, %3;" : "=l"(r) : "r"(pitch), "n"(K), "l"(reinterpret_cast<unsigned long long>(yrow)));
    return reinterpret_cast<char*>(r);
}

// The R rows of one thread in one tile.  GENERAL adds the per-row mask and the residual.  Results go
// straight to global memory with streaming stores (yrow is the address of the thread's first row).
// In a mixed tile the mask value of box row j of this thread's row group sits in lane msrc + j
// (mkv), fetched with one load per lane before the rows start.
template <int DT, int W, int VB, int RPT, bool ACT, bool GENERAL, int ROW_BYTES>
__device__ __forceinline__ void process_rows(uint32_t trow, float mkv, int msrc, const TmaParams& p, bool mixed,
                                             const char* rb, char* yrow, unsigned pitch, int tfirst, int rows_ok,
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
            if (mixed) {
                const float mk = __shfl_sync(0xffffffffu, mkv, msrc + H + k);
                if (p.seg_mode) {
                    if (mk != 1.0f) {  // a sequence begins at this row: nothing above it is a tap
#pragma unroll
                        for (int w = 0; w < H; ++w)
#pragma unroll
                            for (int q = 0; q < NP; ++q) hist[w][q] = make_float2(0.f, 0.f);
                    }
                } else {
                    apply_mask<DT, VB>(cur, mk, p.skip);
                }
            }
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
        S::template stg_row<k>(row_addr<k>(yrow, pitch), outw, rows_ok);
        if constexpr (H > 0) {
#pragma unroll
            for (int q = 0; q < NP; ++q) hist[k % H][q] = cur[q];
        }
    });
}

// Class of one tile from its mask rows: all valid, mixed, or nothing to read.  One warp per tile.
__device__ __forceinline__ int classify_tile(const TmaParams& p, int b, int t0, int H, int box_rows, int lane) {
    if (p.seg_mode) {
        // a sequence starting at box row 1 or later cuts taps of this tile's rows; one starting at
        // box row 0 does not (no output of the tile reads above it)
        bool cut = false;
        for (int jrow = 1 + lane; jrow < box_rows; jrow += 32)
            cut |= tile_mask(p, (long long)b * p.smb, t0 - H + jrow) != 1.0f;
        return __any_sync(0xffffffffu, cut) ? TILE_MIXED : TILE_FULL;
    }
    bool any = false, all_one = true;
    for (int jrow = lane; jrow < box_rows; jrow += 32) {
        const int t = t0 - H + jrow;
        if (t >= 0 && t < p.T) {
            const float mk = load_mask(p.mask, (long long)b * p.smb + (long long)t * p.smt, p.mask_dtype);
            any |= (mk != 0.0f);
            all_one &= (mk == 1.0f);
        }
    }
    any = __any_sync(0xffffffffu, any);
    all_one = __all_sync(0xffffffffu, all_one);
    // (with an initial state the first rows of a sequence see history even if every input is masked)
    const bool history = p.init != nullptr && t0 == 0;
    return all_one ? TILE_FULL : ((any || !p.skip || p.res != nullptr || history) ? TILE_MIXED : TILE_EMPTY);
}

// The same classification by ONE thread (every CTA classifying all tiles of a small launch itself).
// With contiguous, aligned mask rows a whole tile's mask is read with 128-bit loads and compared as
// raw bits: FULL only if every element is exactly one, EMPTY only if every bit is zero (a negative
// zero makes the tile MIXED, where the values themselves are looked at).
__device__ __forceinline__ int classify_tile_thread(const TmaParams& p, int b, int t0, int H, int tile_rows) {
    bool any = false, all_one = true;
    const long long mrow = (long long)b * p.smb;
    for (int j = 0; j < H; ++j) {
        const int t = t0 - H + j;
        if (t >= 0 && t < p.T) {
            const float mk = load_mask(p.mask, mrow + (long long)t * p.smt, p.mask_dtype);
            any |= (mk != 0.0f);
            all_one &= (mk == 1.0f);
        }
    }
    const int rows = min(tile_rows, p.T - t0);
    if (p.mask_vec && rows == tile_rows) {
        int es = 1;
        unsigned pat0 = 0x01010101u, pat1 = 0x01010101u;
        switch (p.mask_dtype) {
            case VC1D_I32: es = 4; pat0 = pat1 = 1u; break;
            case VC1D_I64: es = 8; pat0 = 1u; pat1 = 0u; break;
            case VC1D_F32: es = 4; pat0 = pat1 = 0x3f800000u; break;
            case VC1D_BF16: es = 2; pat0 = pat1 = 0x3f803f80u; break;
            case VC1D_F16: es = 2; pat0 = pat1 = 0x3c003c00u; break;
            default: break;
        }
        const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(p.mask) + (mrow + t0) * es);
        const int n16 = tile_rows * es / 16;
#pragma unroll 4
        for (int i = 0; i < n16; ++i) {
            const uint4 v = __ldg(src + i);
            any |= (v.x | v.y | v.z | v.w) != 0u;
            all_one &= (v.x == pat0) & (v.y == pat1) & (v.z == pat0) & (v.w == pat1);
        }
    } else {
        for (int j = 0; j < rows; ++j) {
            const float mk = load_mask(p.mask, mrow + (long long)(t0 + j) * p.smt, p.mask_dtype);
            any |= (mk != 0.0f);
            all_one &= (mk == 1.0f);
        }
    }
    const bool history = p.init != nullptr && t0 == 0;
    return all_one ? TILE_FULL : ((any || !p.skip || p.res != nullptr || history) ? TILE_MIXED : TILE_EMPTY);
}

// Pre-pass of masked launches that schedule dynamically: the class of every (sequence, time tile),
// one byte each, into scratch memory.  The mask is the same for every channel slab.  A tile's class
// looks at box_rows mask rows starting H rows above the tile.
constexpr int kSchedCounterBytes = 4096;
constexpr int kSmemTableCap = 16384;  // largest pre-pass class table a CTA copies into shared memory

// (For the backward pass it can also clear the fp32 gradient accumulators, which saves a launch.)
// With `order` the pre-pass writes a list of all tiles in the order the claims hand them out instead:
// tiles with something to read from the front (ends[0] counts them), tiles without any live tap from
// the back (ends[1]).  Entry = tile number | class << 14.  The cheap tiles (a few bulk stores each) are
// then the last to be claimed, which evens out the moments at which the CTAs of a launch run dry.
// ends[] must be zero at the start; the main kernel that follows leaves them zeroed.
constexpr int kOrderedCap = 4096;         // most tiles a launch may have for the ordered list (8 KB of shared memory)
constexpr int kOrderCounters = 1016;      // ends[] = the last words of the counter region of the scratch buffer
static __global__ void __launch_bounds__(256) k_classify_tiles(const TmaParams p, unsigned char* table, int tile_rows, int H,
                                                               int box_rows, float* zero_a = nullptr, int n_a = 0,
                                                               float* zero_b = nullptr, int n_b = 0,
                                                               unsigned short* order = nullptr, unsigned int* ends = nullptr) {
    griddep_wait();  // the table may still be read by the previous launch on this stream
    griddep_launch_dependents();
    {
        const int stride = gridDim.x * blockDim.x;
        const int first = blockIdx.x * blockDim.x + threadIdx.x;
        for (int i = first; i < n_a; i += stride) zero_a[i] = 0.f;
        for (int i = first; i < n_b; i += stride) zero_b[i] = 0.f;
    }
    const int lane = threadIdx.x & 31;
    const long long tile = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (tile >= (long long)p.B * p.n_ttile) return;
    const int b = (int)(tile / p.n_ttile);
    const int tt = (int)(tile - (long long)b * p.n_ttile);
    const int cls = classify_tile(p, b, tt * tile_rows, H, box_rows, lane);
    if (lane == 0) {
        if (order != nullptr) {
            const unsigned n = (unsigned)p.n_rowtiles;
            const unsigned pos = cls == TILE_EMPTY ? n - 1u - atomicAdd(ends + 1, 1u) : atomicAdd(ends, 1u);
            if (pos < n) order[pos] = (unsigned short)((unsigned)tile | ((unsigned)cls << 14));
        } else {
            table[tile] = (unsigned char)cls;
        }
    }
}

template <int DT, int W, int SLAB_BYTES, int VB, int RPT, bool ACT>
__global__ void __launch_bounds__(Geometry<DT, W, SLAB_BYTES, VB, RPT>::kThreads)
    k_prefill_tma(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_y,
                  const TmaParams p) {
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
    const int kC = p.empty_tma;    // 1: the constant tile exists
    const uint32_t ctile = base + G::off_const(kStages);      // constant tile: act(bias) in every row
    const uint32_t bars = base + G::off_bars(kStages, kC);    // full[s] at bars + 8 s, done[s] at bars + 8 (kStages + s)
    const uint32_t cbar = bars + 8 * (2 * kStages);           // constant tile written (one arrive per consumer warp)
    const uint32_t tbar = cbar + 8;                           // class table written (one arrive per consumer warp)
    const uint32_t flags = base + G::off_flags(kStages, kC);  // per stage: 32-byte tile descriptor
    const uint32_t mvals = base + G::off_mvals(kStages, kC);  // per stage: mask value of every box row (mixed tiles)
    const uint32_t table = base + G::off_table(kStages, kC);  // class of each of this CTA's tiles (masked launches)

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int slab = blockIdx.x;
    const int j0 = blockIdx.y;
    const int stride = p.ctas_per_slab;
    const int slab_ch0 = slab * G::kSlabElems;
    const int n_my = (j0 < p.n_rowtiles) ? (p.n_rowtiles - j0 + stride - 1) / stride : 0;

    if (threadIdx.x == G::kConsumerWarps * 32) {  // the producer's first lane: the descriptors its copies will name
        prefetch_tensormap(&tmap_x);
        if (kC) prefetch_tensormap(&tmap_y);
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bars + 8 * s, 1);                              // full: the producer's arrive (+ tx bytes)
            mbar_init(bars + 8 * (kStages + s), G::kConsumerWarps);  // done: one arrive per consumer warp
        }
        mbar_init(cbar, G::kConsumerWarps);
        mbar_init(tbar, G::kConsumerWarps);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }

    // tile number -> (sequence, first row); the time position is rotated by the sequence index so
    // that tiles handled together do not all sit at the same position of their sequences (with
    // right-padded batches the late positions are the cheap, masked ones)
    auto locate = [&](int rt, int& b, int& t0) {
        b = rt / p.n_ttile;
        int tt = rt - b * p.n_ttile + b % p.n_ttile;
        if (tt >= p.n_ttile) tt -= p.n_ttile;
        t0 = tt * G::kTileRows;
    };

    // ---- prologue with a mask: the class of every tile this CTA may take is in shared memory before ----
    // the tile loop starts (the pre-pass's table or list copied from scratch memory, or, without
    // scratch, this CTA's own tiles classified here, one warp per tile), so no mask latency ever sits
    // between two bulk copies.
    // Launched with programmatic stream serialization, this grid may start while its predecessor in
    // the stream is still running: nothing above touched global memory.
    auto copy_table = [&]() {
        if (p.gtable != nullptr && p.table_in_smem == 3) {
            const int n16 = (p.n_rowtiles + 7) >> 3;  // eight entries to 16 bytes; the list is padded to that
            const uint4* src = reinterpret_cast<const uint4*>(p.gtable);
            for (int i = threadIdx.x; i < n16; i += G::kThreads) {
                const uint4 v = __ldcg(src + i);
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(table + 16 * i), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                             : "memory");
            }
        } else if (p.gtable != nullptr && p.table_in_smem == 2) {
            // large launches: two bits per tile, sixteen tiles to a word (the scratch table is padded to 16)
            const int n16 = (p.n_rowtiles + 15) >> 4;
            const uint4* src = reinterpret_cast<const uint4*>(p.gtable);
            for (int i = threadIdx.x; i < n16; i += G::kThreads) {
                const uint4 v = __ldcg(src + i);
                const unsigned wv[4] = {v.x, v.y, v.z, v.w};
                unsigned packed = 0u;
#pragma unroll
                for (int k = 0; k < 16; ++k) packed |= ((wv[k >> 2] >> (8 * (k & 3))) & 3u) << (2 * k);
                sts_s32(table + 4 * i, (int)packed);
            }
        } else if (p.gtable != nullptr && p.table_in_smem) {
            const int n16 = p.n_rowtiles >> 4;
            const uint4* src = reinterpret_cast<const uint4*>(p.gtable);
            for (int i = threadIdx.x; i < n16; i += G::kThreads) {
                const uint4 v = __ldcg(src + i);  // written by the pre-pass while this grid was already resident: no read-only path
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(table + 16 * i), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                             : "memory");
            }
            for (int i = (n16 << 4) + threadIdx.x; i < p.n_rowtiles; i += G::kThreads) sts_u8(table + i, __ldcg(p.gtable + i));
        }
    };
    // A table kept from an earlier launch is older than anything this grid could be waiting for.  With it
    // (or without a mask) the producer can work out its first tile before the wait, which it then
    // passes in its own branch; so do the consumer warps.
    const bool early = p.mask == nullptr || p.table_early;
    if (p.table_early) copy_table();
    if (!early) {
        griddep_wait();
        copy_table();
    }
    if (p.mask != nullptr && p.gtable == nullptr && !p.inline_cls) {
        for (int i = warp; i < n_my; i += G::kThreads / 32) {
            int b, t0;
            locate(j0 + i * stride, b, t0);
            const int cls = classify_tile(p, b, t0, H, G::kBoxRows, lane);
            if (lane == 0) sts_u8(table + i, cls);
        }
    }
    __syncthreads();

    if (warp == G::kConsumerWarps) {
        // ================================ producer warp ==================================
        // Walks the CTA's tiles.  Each tile takes the next ring slot (after the consumers of the
        // slot's previous tile have arrived on done[s]); a tile with something to read is loaded by
        // one bulk tensor copy, a tile in which every tap of every row is masked is only announced.
        // After the last tile an END marker takes a slot.
        int s_ring = 0, n_ring = 0;  // next ring slot, tiles put into the ring so far
        uint32_t ph_ring = 0;        // how often the ring has wrapped, mod 2
        // claim the next slot: wait until its previous tile has been consumed
        auto claim = [&]() -> bool {
            if (n_ring >= kStages) {
                const bool ok = mbar_wait(bars + 8 * (kStages + s_ring), ph_ring ^ 1, p.spin_limit);
                if (!ok && lane == 0) atomicAdd(p.timeouts, 1u);
                if (!ok) return false;
            }
            return true;
        };
        unsigned loads_issued = 0u, loads_parity = 0u;  // per stage: a copy was started, and in which ring phase
        auto advance = [&]() {
            ++n_ring;
            if (++s_ring == kStages) {
                s_ring = 0;
                ph_ring ^= 1;
            }
        };
        // Which tile comes next.  Static: this CTA's tiles are j0, j0 + G, j0 + 2G, ...  Dynamic
        // (a zeroed counter per slab in caller-provided scratch memory): the next unclaimed tile of
        // the slab, so that a CTA that met cheap (masked) tiles or runs on a faster SM takes more.
        const bool dynamic = p.sched != nullptr && (p.mask == nullptr || p.gtable != nullptr || p.inline_cls);
        int n_issued = 0;
        const unsigned chunk = (unsigned)p.chunk;  // consecutive tiles per claim
        unsigned c_next = 0u, c_left = 0u;
        auto next_tile = [&]() -> int {
            unsigned raw;
            if (dynamic && c_left > 0u) {
                raw = c_next++;  // rest of the chunk claimed last
                --c_left;
            } else if (dynamic && chunk == 1u && n_issued < p.static_first) {
                // the first tiles of a CTA need no claim: their copies start back to back
                raw = (unsigned)(j0 + n_issued * stride);
            } else if (dynamic && n_issued > 0) {
                // the counter hands out the chunks behind the unclaimed first ones of every CTA of the slab
                raw = 0u;
                if (lane == 0) raw = atomicAdd(p.sched + slab, chunk);
                raw = __shfl_sync(0xffffffffu, raw, 0) + (unsigned)stride * (chunk == 1u ? (unsigned)p.static_first : chunk);
                c_next = raw + 1u;
                c_left = chunk - 1u;
            } else if (dynamic) {
                raw = (unsigned)j0 * chunk;  // a CTA's first chunk needs no claim: the copy starts a round trip earlier
                c_next = raw + 1u;
                c_left = chunk - 1u;
            } else {
                raw = n_issued < n_my ? (unsigned)(j0 + n_issued * stride) : 0xffffffffu;
            }
            ++n_issued;
            return raw < (unsigned)p.n_rowtiles ? (int)raw : -1;
        };
        // class of a located tile: the pre-pass table (copied to shared memory when it fits), this
        // CTA's own table, or no mask at all
        auto tile_class = [&](int i, int b, int t0) -> int {
            if (p.mask == nullptr) return TILE_FULL;
            if (p.inline_cls) return lds_u8(table + (uint32_t)(b * p.n_ttile + t0 / G::kTileRows));
            if (p.gtable != nullptr) {
                const long long idx = (long long)b * p.n_ttile + t0 / G::kTileRows;
                if (p.table_in_smem == 2)
                    return (lds_s32(table + 4u * (uint32_t)(idx >> 4)) >> (2 * (int)(idx & 15))) & 3;
                return p.table_in_smem ? lds_u8(table + (uint32_t)idx) : (int)__ldcg(p.gtable + idx);
            }
            return lds_u8(table + i);
        };
        // announce a tile in the next ring slot and start its copy
        auto fetch_mask = [&](int b, int t0, float (&mv)[NMK]) {
#pragma unroll
            for (int k = 0; k < NMK; ++k) mv[k] = tile_mask(p, (long long)b * p.smb, t0 - H + lane + 32 * k);
        };
        auto put_tile = [&](int b, int t0, int cls, const float (&mv)[NMK]) {
            const int s = s_ring;
            if (p.test_withhold && n_ring == 0) return;  // self-test: the consumers' wait for this slot must expire
            // (the slot's previous tile has been consumed: claim() saw to that)
            loads_issued &= ~(1u << s);
            if (cls != TILE_EMPTY) {
                loads_issued |= 1u << s;
                loads_parity = (loads_parity & ~(1u << s)) | (ph_ring << s);
            }
            if (cls == TILE_MIXED) {
#pragma unroll
                for (int k = 0; k < NMK; ++k) sts_f32(mvals + s * G::kMaskBytes + (lane + 32 * k) * 4, mv[k]);
                __syncwarp();  // lane 0's arrive below publishes the whole warp's stores
            }
            if (lane == 0) {
                const long long yoff = (long long)b * p.syb + (long long)t0 * p.syt;
                sts_desc(flags + 32 * s, cls, p.T - t0, yoff);
                sts_s32(flags + 32 * s + 16, b);
                sts_s32(flags + 32 * s + 20, t0);
                const uint32_t full = bars + 8 * s;
                if (cls != TILE_EMPTY) {
                    mbar_arrive_expect_tx(full, G::kBoxRows * G::kRowBytes);
                    tma_load_3d(base + s * G::kStageBytes, &tmap_x, slab_ch0, t0 - H, b, full);
                } else {
                    mbar_arrive(full);  // nothing to read: the consumers store act(bias)
                }
            }
            __syncwarp();
        };
        // One claim ahead: the next tile and its class are fetched while the current tile waits for
        // its ring slot.  (Claiming further ahead was measured slower: the tiles in flight spread out
        // in memory and the tail of the launch gets longer.)  The mask rows of a mixed tile are
        // fetched at the same time and travel to the consumers with the tile.
        bool live = true;
        int rt = next_tile(), b = 0, t0 = 0, cls = TILE_FULL;
        float mv[NMK], mv_now[NMK];
#pragma unroll
        for (int k = 0; k < NMK; ++k) mv[k] = 1.0f;
        // claim position -> tile and class
        auto resolve = [&](int pos, int i, int& bb, int& tt0, int& c) {
            if (p.table_in_smem == 3) {
                const int e = lds_u16(table + 2u * (uint32_t)pos);
                const int id = e & 0x3fff;
                c = e >> 14;
                bb = id / p.n_ttile;
                tt0 = (id - bb * p.n_ttile) * G::kTileRows;
            } else {
                locate(pos, bb, tt0);
                c = tile_class(i, bb, tt0);
            }
        };
        if (rt >= 0) {
            // (classifying in the kernel: the consumer warps are still filling the table, so the
            // producer works out the class of its first tile by itself)
            if (p.inline_cls) {
                locate(rt, b, t0);
                cls = classify_tile(p, b, t0, H, G::kBoxRows, lane);
            } else {
                resolve(rt, 0, b, t0, cls);
            }
        }
        if (early) griddep_wait();  // from here on global memory is touched
        if (rt >= 0 && cls == TILE_MIXED) fetch_mask(b, t0, mv);
        bool const_ready = false;  // the consumers have written the constant tile
        bool table_ready = !p.inline_cls;  // the consumers have classified every tile
        for (int i = 0; live && rt >= 0; ++i) {
            const int b_now = b, t0_now = t0, cls_now = cls;
#pragma unroll
            for (int k = 0; k < NMK; ++k) mv_now[k] = mv[k];
            bool put_done = false;
            if (i == 0 && !(cls_now == TILE_EMPTY && kC)) {
                // a CTA's first tile: its copy starts before anything else is looked at (a CTA that
                // classifies in the kernel would otherwise wait for the table the next claim needs)
                put_tile(b_now, t0_now, cls_now, mv_now);
                advance();
                put_done = true;
            }
            rt = next_tile();
            if (rt >= 0) {
                if (!table_ready) {
                    table_ready = mbar_wait(tbar, 0, p.spin_limit);
                    if (!table_ready) {
                        if (lane == 0) atomicAdd(p.timeouts, 1u);
                        live = false;
                        break;
                    }
                }
                resolve(rt, i + 1, b, t0, cls);
                if (cls == TILE_MIXED) fetch_mask(b, t0, mv);
            }
            if (put_done) continue;
            if (cls_now == TILE_EMPTY && kC) {
                // no tap of the tile is live: every row is act(bias).  One bulk store from the
                // constant tile writes it; it takes no ring slot and no consumer sees it.
                if (!const_ready) {
                    const_ready = mbar_wait(cbar, 0, p.spin_limit);
                    if (!const_ready && lane == 0) atomicAdd(p.timeouts, 1u);
                    live = const_ready;
                    if (!live) break;
                }
                if (lane == 0) {
                    // (a store is never started past the last row; rows past it inside a box are clipped)
                    for (int r = 0; r < G::kTileRows && t0_now + r < p.T; r += G::kConstRows)
                        tma_store_3d(&tmap_y, slab_ch0, t0_now + r, b_now, ctile);
                    bulk_commit();
                }
                __syncwarp();
                continue;
            }
            live = claim();
            if (!live) break;
            put_tile(b_now, t0_now, cls_now, mv_now);
            advance();
        }
        // Every tile of this CTA is on its way: a dependent launch of the stream may now take the slots
        // that CTAs free as they finish (triggering at the top was measured slower: the early
        // CTAs of the next launch disturb the steady state of this one).
        griddep_launch_dependents();
        // END marker: the consumers leave when they meet it
        if (live && claim()) {
            loads_issued &= ~(1u << s_ring);
            if (lane == 0) {
                sts_desc(flags + 32 * s_ring, TILE_END, 0, 0);
                mbar_arrive(bars + 8 * s_ring);
            }
            __syncwarp();
        }
        // Dynamic scheduling leaves the scratch counters zeroed for the next launch: the last CTA
        // of the grid to get here (every CTA has made its last claim by then) resets them.
        if (dynamic && lane == 0) {
            const unsigned n_ctas = gridDim.x * gridDim.y;
            __threadfence();
            const unsigned done = atomicAdd(p.sched + gridDim.x, 1u);
            if (done == n_ctas - 1) {
                for (unsigned k = 0; k <= gridDim.x; ++k) p.sched[k] = 0u;
                if (p.table_in_smem == 3) p.sched[kOrderCounters] = p.sched[kOrderCounters + 1] = 0u;  // the pre-pass's
                __threadfence();
            }
        }
        // the bulk stores read the constant tile: shared memory must outlive them
        if (kC && lane == 0) bulk_wait_read();
        // No copy of this CTA may still be in flight when it ends.  Normally the consumers, who wait for
        // every copy, outlive this warp; if their waits expired they are gone already, so the copies
        // started here are waited for here as well (bounded like every wait).
        for (int s = 0; s < kStages; ++s)
            if ((loads_issued >> s) & 1u) mbar_wait(bars + 8 * s, (loads_parity >> s) & 1u, p.spin_limit);
    } else {
        // ================================ consumer warps =================================
        const int grp = threadIdx.x / LPR;  // row group inside the tile
        const int cl = threadIdx.x % LPR;   // channel slice inside the slab
        const int d0 = slab_ch0 + cl * NE;
        const bool ch_ok = d0 < p.D;  // dim is a multiple of the 128-bit vector: a slice is in or out as a whole
        const int rbase = grp * R;

        if (early) griddep_wait();
        float2 wp[W][NP];
        float2 bp[NP];
        load_weights<DT, W, VB>(p, d0, ch_ok, wp, bp);
        // value of a row whose W taps are all masked: act(bias)
        uint32_t const_row[NW];
        {
            float2 c[NP];
#pragma unroll
            for (int q = 0; q < NP; ++q) c[q] = ACT ? silu2<E::kPreciseSilu>(bp[q]) : bp[q];
            S::pack(c, const_row);
        }
        if (kC) {
            // the constant rows (the first row groups write them); the producer's bulk stores read them
            if (rbase < G::kConstRows) {
#pragma unroll
                for (int k = 0; k < R; ++k) S::sts(ctile + (rbase + k) * G::kRowBytes + cl * VB, const_row);
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(cbar);
        }
        if (p.inline_cls) {
            // class of every tile of the launch, one thread per tile; the producer meanwhile has its
            // first tile in flight and waits for this table before its second claim
            // (every CTA starts at another tile, so that the CTAs of the grid do not all ask the L2 for
            // the same mask bytes at the same moment)
            const int rot = (int)(((unsigned)(blockIdx.y * gridDim.x + blockIdx.x) * 61u) % (unsigned)p.n_rowtiles);
            for (int i = threadIdx.x; i < p.n_rowtiles; i += G::kConsumerThreads) {
                const int tile = (i + rot) % p.n_rowtiles;
                const int bb = tile / p.n_ttile;
                const int tt = tile - bb * p.n_ttile;
                sts_u8(table + tile, classify_tile_thread(p, bb, tt * G::kTileRows, H, G::kTileRows));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(tbar);
        }
        const bool general_kernel = (p.mask != nullptr) || (p.res != nullptr);
        const unsigned pitch = (unsigned)p.syt;  // output row pitch in bytes; the launcher keeps 8 rows within 32 bits

        // per-thread constants of the tile loop
        char* const ybase = p.y + (long long)rbase * p.syt + (long long)d0 * E::kBytes;
        const uint32_t tbase = base + rbase * G::kRowBytes + cl * VB;
        const int rbase_lim = ch_ok ? rbase : (1 << 28);  // makes rows_ok 0 for channel slices past dim

        int s = -1;
        uint32_t ph = 0;
        uint32_t trow = tbase - G::kStageBytes;
        for (;;) {
            trow += G::kStageBytes;
            if (++s == kStages) {
                s = 0;
                ph ^= 1;
                trow = tbase;
            }
            if (!mbar_wait(bars + 8 * s, ph, p.spin_limit)) {
                if (lane == 0) atomicAdd(p.timeouts, 1u);
                break;  // no barrier is shared with the other warps: each leaves on its own
            }
            int cls, rows_valid;
            long long yoff;
            lds_desc(flags + 32 * s, cls, rows_valid, yoff);
            if (cls == TILE_END) break;
            // box row of time t is (t - t0 + H); this thread reads box rows rbase .. rbase+R+H-1 at trow
            const int rows_ok = min(R, max(0, rows_valid - rbase_lim));  // rows of this thread that exist
            char* yrow = ybase + yoff;
            if (cls == TILE_EMPTY) {
                // every tap of every row is masked and nothing was loaded
                __syncwarp();
                if (lane == 0) mbar_arrive(bars + 8 * (kStages + s));
                static_for<0, R>([&](auto kc) {
                    constexpr int k = decltype(kc)::value;
                    S::template stg_row<k>(row_addr<k>(yrow, pitch), const_row, rows_ok);
                });
                continue;
            }
            float2 hist[H > 0 ? H : 1][NP];
#pragma unroll
            for (int w = 0; w < H; ++w) {
                uint32_t raw[NW];
                S::lds(trow + w * G::kRowBytes, raw);
                S::unpack(raw, hist[w]);
            }
            if (p.init != nullptr && rbase == 0 && ch_ok && lds_s32(flags + 32 * s + 20) == 0) {
                // first rows of a sequence: the W-1 rows above them come from the initial state
                using T = typename E::type;
                const int b = lds_s32(flags + 32 * s + 16);
                const T* in = reinterpret_cast<const T*>(p.init) + ((long long)b * p.D + d0) * p.init_len;
#pragma unroll
                for (int w = 0; w < H; ++w) {
                    T vals[NE];
#pragma unroll
                    for (int c = 0; c < NE; ++c) vals[c] = in[(long long)c * p.init_len + (p.init_len - H + w)];
                    uint32_t raw[NW];
                    const uint32_t* vw = reinterpret_cast<const uint32_t*>(vals);
#pragma unroll
                    for (int i = 0; i < NW; ++i) raw[i] = vw[i];
                    S::unpack(raw, hist[w]);
                }
            }
            if (!general_kernel || (cls == TILE_FULL && p.res == nullptr)) {
                process_rows<DT, W, VB, RPT, ACT, false, G::kRowBytes>(trow, 1.0f, 0, p, false, nullptr, yrow, pitch, 0,
                                                                       rows_ok, hist, wp, bp);
            } else {
                const bool mixed = (cls == TILE_MIXED);
                const int b = lds_s32(flags + 32 * s + 16);
                const int tfirst = lds_s32(flags + 32 * s + 20) + rbase;
                // lanes of one row group (a warp holds one or two) fetch the group's R + H mask values
                constexpr int GL = LPR < 32 ? LPR : 32;
                static_assert(R + H <= GL, "one mask value per lane of a row group");
                const int msrc = lane & ~(GL - 1);
                float mkv = 1.0f;
                if (mixed) {
                    const int j = lane & (GL - 1);
                    if (j < R + H) mkv = lds_f32(mvals + s * G::kMaskBytes + (rbase + j) * 4);  // box row rbase + j
#pragma unroll
                    for (int w = 0; w < H; ++w) {
                        const float mk = __shfl_sync(0xffffffffu, mkv, msrc + w);
                        if (p.seg_mode) {
                            if (mk != 1.0f) {  // a sequence begins at box row w: the rows above it are no taps
#pragma unroll
                                for (int v = 0; v < H; ++v) {
                                    if (v < w) {
#pragma unroll
                                        for (int q = 0; q < NP; ++q) hist[v][q] = make_float2(0.f, 0.f);
                                    }
                                }
                            }
                        } else {
                            apply_mask<DT, VB>(hist[w], mk, p.skip);
                        }
                    }
                }
                const char* rb = nullptr;
                if (p.res != nullptr && !p.res_is_x && ch_ok)
                    rb = p.res + (long long)b * p.srb + (long long)d0 * E::kBytes;
                process_rows<DT, W, VB, RPT, ACT, true, G::kRowBytes>(trow, mkv, msrc, p, mixed, rb, yrow, pitch, tfirst,
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
                        } else if (p.init != nullptr && p.init_len + t >= 0) {
                            v = reinterpret_cast<const T*>(p.init)[((long long)b * p.D + d0 + c) * p.init_len +
                                                                    (p.init_len + t)];
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
// address, on the current device, of the counter of expired bounded waits
unsigned int* timeouts_ptr();

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

    // row offsets inside a tile are computed in 32 bits
    if (a.y_stride_t < 0 || (long long)a.y_stride_t * eb >= (1LL << 28)) return cudaErrorNotSupported;

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
    // Output map for the bulk stores of tiles without a live tap (same box as a tile, no halo).  Only
    // launches that can have such tiles carry the constant tile; when y cannot be described by a
    // tensor map the consumer warps store those tiles instead.
    CUtensorMap tmap_y = tmap_x;
    p.empty_tma = 0;
    if (p.mask != nullptr && p.skip && a.residual == nullptr && !p.seg_mode && a.tma_empty_store != 1) {
        const cuuint64_t dims[3] = {(cuuint64_t)a.dim, (cuuint64_t)a.seqlen, (cuuint64_t)a.batch};
        const cuuint32_t estr[3] = {1u, 1u, 1u};
        cuuint64_t st[2] = {(cuuint64_t)a.y_stride_t * eb, (cuuint64_t)a.y_stride_b * eb};
        if (a.seqlen == 1) st[0] = (cuuint64_t)a.dim * eb;
        if (a.batch == 1) st[1] = st[0] * (cuuint64_t)a.seqlen;
        const bool addressable = a.y_stride_t > 0 && a.y_stride_b >= 0 && st[0] % 16 == 0 && st[1] % 16 == 0 &&
                                 (reinterpret_cast<uintptr_t>(a.y) & 15u) == 0;
        if (addressable) {
            const cuuint32_t box[3] = {(cuuint32_t)slab_ch, (cuuint32_t)G::kConstRows, 1u};
            const CUresult r = enc(&tmap_y, dt, 3, a.y, dims, st, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r == CUDA_SUCCESS) p.empty_tma = 1;
        }
    }
    int stages = a.tma_stages > 0 ? a.tma_stages : 3;
    if (stages < 2) stages = 2;
    if (stages > kMaxStages) stages = kMaxStages;
    int per_sm = (a.tma_ctas_per_sm > 0 && a.tma_ctas_per_sm <= 32) ? a.tma_ctas_per_sm : 3;
    p.stages = stages;
    // persistent CTAs, split evenly over the channel slabs; with a mask every CTA keeps one class
    // byte per tile in shared memory, so the grid grows before a CTA would own more than 8192 tiles
    long long g = ((long long)sm_count() * per_sm) / n_slab;
    if (g < 1) g = 1;
    if (p.mask != nullptr && n_rowtiles > g * 8192) g = (n_rowtiles + 8191) / 8192;  // only matters without scratch
    if (g > n_rowtiles) g = n_rowtiles;
    if (g > 65535) g = 65535;
    p.ctas_per_slab = (int)g;
    const long long tiles_per_cta = (n_rowtiles + g - 1) / g;

    // scratch: [4096 bytes of counters (one per slab + one), zero between launches | class byte per
    // (sequence, time tile)].  The counter region has a fixed size so that no launch's class bytes
    // can land where a later launch with more slabs keeps its counters.
    p.sched = nullptr;
    p.gtable = nullptr;
    p.table_in_smem = 0;
    // Class tables of the three tile heights (64, 128, 32 rows) have places of their own behind the
    // counters, each as long as this batch and seqlen need, so that launches of different geometry that
    // share a mask (the Canon layers of one block differ in width) can each keep theirs.  A scratch
    // buffer with room for one table only has it at the front.
    constexpr int kRegion = G::kTileRows == 64 ? 0 : (G::kTileRows == 128 ? 1 : 2);
    // (a place holds two bytes per tile: a class byte each, or the ordered list of a launch of up to kOrderedCap tiles)
    auto table_len = [&](int rows) { return ((long long)a.batch * ((a.seqlen + rows - 1) / rows) + 15) / 16 * 32; };
    long long tab_off = kRegion == 0 ? 0 : (kRegion == 1 ? table_len(64) : table_len(64) + table_len(128));
    bool own_region = true;
    if (p.mask != nullptr && a.scratch_bytes < kSchedCounterBytes + tab_off + table_len(G::kTileRows)) {
        tab_off = 0;
        own_region = false;
    }
    const bool ordered = p.mask != nullptr && a.tma_classify == 0 && n_rowtiles <= kOrderedCap &&
                         a.scratch_bytes >= kSchedCounterBytes + tab_off + table_len(G::kTileRows);
    const long long table_need = p.mask != nullptr ? tab_off + n_rowtiles : 0;
    // dynamic claims pay off once a CTA has several tiles; with two or three the claim round trips
    // (and, with a mask, the pre-pass) cost more than the balance gains
    p.spin_limit = a.tma_test_expire ? (1u << 12) : kSpinLimit;
    p.test_withhold = a.tma_test_expire ? 1 : 0;
    p.chunk = (a.tma_claim_chunk == 2 || a.tma_claim_chunk == 4) ? a.tma_claim_chunk : 1;
    if (tiles_per_cta < 4LL * p.chunk) p.chunk = 1;
    // two unclaimed tiles per CTA: both copies start back to back at the top of the kernel
    p.static_first = (a.tma_static_first >= 1 && a.tma_static_first <= 1024) ? a.tma_static_first : 2;
    {
        // every unclaimed tile j0 + k * g must exist: k < n_rowtiles / g; leave a few tiles to the counters
        const long long whole = n_rowtiles / g;
        if (p.static_first > whole - 2) p.static_first = (int)(whole - 2 > 1 ? whole - 2 : 1);
    }
    const bool use_scratch = tiles_per_cta >= 4 && a.scratch != nullptr && n_slab + 1 <= kOrderCounters &&
                             a.scratch_bytes >= kSchedCounterBytes + table_need &&
                             (reinterpret_cast<uintptr_t>(a.scratch) & 15u) == 0;
    unsigned char* tab = nullptr;
    int table_bytes = 0;  // class bytes in shared memory
    // Tile classes of a masked launch with dynamic claims.  A small mask whose rows can be read with
    // 128-bit loads is classified by every CTA itself (its consumer warps do it while the first tile
    // is in flight: no pre-pass launch, nothing on the critical path); otherwise a pre-pass kernel
    // writes the classes to scratch memory once for all CTAs.
    p.inline_cls = 0;
    p.mask_vec = 0;
    if (p.mask != nullptr && !p.seg_mode) {
        const int es = elem_bytes(p.mask_dtype);
        const bool vec = es > 0 && p.smt == 1 && (p.smb * es) % 16 == 0 &&
                         (reinterpret_cast<uintptr_t>(p.mask) & 15u) == 0;
        p.mask_vec = vec ? 1 : 0;
        const long long loads = n_rowtiles * G::kTileRows * es / 16;  // 128-bit loads for the whole mask
        if (use_scratch && vec && n_rowtiles <= kSmemTableCap && loads <= 32LL * G::kConsumerThreads &&
            a.tma_classify == 2)
            p.inline_cls = 1;
    }
    if (use_scratch) {
        p.sched = reinterpret_cast<unsigned int*>(a.scratch);
        if (p.inline_cls) {
            table_bytes = (int)((n_rowtiles + 15) / 16 * 16);
        } else if (p.mask != nullptr) {
            tab = reinterpret_cast<unsigned char*>(a.scratch) + kSchedCounterBytes + tab_off;
            if (ordered) {
                p.table_in_smem = 3;
                table_bytes = (int)((n_rowtiles + 7) / 8 * 16);
            } else if (n_rowtiles <= kSmemTableCap) {
                p.table_in_smem = 1;
                table_bytes = (int)((n_rowtiles + 15) / 16 * 16);
            } else if (n_rowtiles <= 4LL * kSmemTableCap &&
                       a.scratch_bytes >= kSchedCounterBytes + tab_off + (n_rowtiles + 15) / 16 * 16) {
                p.table_in_smem = 2;
                table_bytes = (int)((n_rowtiles + 15) / 16 * 4);
            }
        }
    } else if (p.mask != nullptr) {
        // static assignment: every CTA classifies its own tiles into shared memory
        if (tiles_per_cta > 8192) return cudaErrorNotSupported;  // the direct kernel takes it
        table_bytes = (int)((tiles_per_cta + 15) / 16 * 16);
    }
    const int smem = G::smem_bytes(stages, p.empty_tma, table_bytes);
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
    // Both kernels are launched with programmatic stream serialization: each may start while its
    // predecessor in the stream drains, and waits (griddep_wait) before it touches global memory, which
    // hides the launch latencies and the part of the prologue that needs no global memory.
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed =
        (pdl_enabled() && (tab != nullptr || a.tma_pdl != 1)) ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // tma_kept_tables: the caller vouches that the table at this geometry's place is the one the pre-pass would write
    const bool keep_table = tab != nullptr && own_region && a.tma_classify != 2 && ((a.tma_kept_tables >> kRegion) & 1) != 0;
    p.table_early = keep_table ? 1 : 0;
    note_class_table(tab == nullptr ? 0 : ((keep_table ? 2 : (own_region ? 1 : 3)) | (kRegion << 8)));
    if (keep_table) {
        p.gtable = tab;
    } else if (tab != nullptr) {
        const long long threads = n_rowtiles * 32;
        cfg.gridDim = dim3((unsigned)((threads + 255) / 256));
        cfg.blockDim = dim3(256);
        cfg.dynamicSmemBytes = 0;
        const cudaError_t e = cudaLaunchKernelEx(
            &cfg, k_classify_tiles, p, tab, (int)G::kTileRows, (int)G::kH, (int)G::kBoxRows, (float*)nullptr, 0, (float*)nullptr,
            0, ordered ? reinterpret_cast<unsigned short*>(tab) : (unsigned short*)nullptr,
            ordered ? p.sched + kOrderCounters : (unsigned int*)nullptr);
        if (e != cudaSuccess) return e;
        note_launch("classify");
        p.gtable = tab;
    }
    cfg.gridDim = dim3((unsigned)n_slab, (unsigned)g);
    cfg.blockDim = dim3(G::kThreads);
    cfg.dynamicSmemBytes = (size_t)smem;
    note_launch("tma");
    return cudaLaunchKernelEx(&cfg, k_prefill_tma<DT, W, SLAB_BYTES, VB, RPT, ACT>, tmap_x, tmap_y, p);
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
