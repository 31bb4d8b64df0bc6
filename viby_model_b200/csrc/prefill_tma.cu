// TMA-staged prefill kernel for the channel-last layout (reference call site
// model/model.py:459-466; fused mask / residual / final state: model/model.py:454-457,
// 491, 470-489).
//
// Geometry.  A tile is T_TILE time rows x one 128- or 256-byte slab of channels of one
// sequence.  Its input box, (T_TILE + W-1) rows starting W-1 rows ABOVE the tile, arrives in
// shared memory by one cp.async.bulk.tensor.3d load (no multicast); rows before t = 0 are
// out of bounds for the tensor map and are zero-filled by the hardware, which is exactly the
// causal left padding.  The grid is (channel slabs) x (persistent CTAs per slab): a CTA keeps
// the weights of its slab in registers for its whole life and walks row tiles
// j, j + G, j + 2G, ... of that slab, so neighbouring CTAs touch neighbouring rows and the
// (W-1)-row halo of a tile is an L2 hit.
//
// Pipeline.  One producer warp and kConsumerWarps consumer warps share a ring of kStages
// buffers guarded by full/empty mbarriers.  The producer scans the tile's mask rows (32 lanes,
// a few loads each), stores them as floats beside the data and classifies the tile: all rows
// valid, mixed, or nothing to read -- in the last case no bytes are requested from HBM at all.
// Bytes in flight are set by the ring depth (kStages x 17 KB per CTA, three CTAs per SM), not
// by registers.  Each consumer thread owns one 128-bit channel vector and kRowsPerThread
// consecutive rows: a register sliding window over shared memory, fp32x2 FMAs, fused
// mask / bias / SiLU / residual epilogue.  Results overwrite the input rows in place and leave
// by one cp.async.bulk.tensor store per tile, issued by the producer warp, so no consumer warp
// ever waits on HBM in either direction; the store also clips the ragged last tile in time and
// in channels.
//
// Every mbarrier wait is bounded; on expiry the CTA records the event in a device counter
// (read by vc1d_tma_timeouts()) and leaves its loops.
#include <cuda.h>

#include <atomic>
#include <mutex>

#include "vc1d_common.cuh"
#include "vc1d_internal.h"

namespace vc1d {
namespace {

constexpr int kStages = 4;
constexpr int kConsumerWarps = 4;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;  // + producer warp
constexpr int kRowsPerThread = 8;
constexpr unsigned kSpinLimit = 1u << 24;

__device__ unsigned int g_tma_timeouts = 0;

enum : int { TILE_EMPTY = 0, TILE_MIXED = 1, TILE_FULL = 2 };

struct TmaParams {
    char* y;
    const char* x;  // for the final-state pass
    const char* res;
    const void* weight;
    const void* bias;
    const void* mask;
    char* fstate;
    long long syb, syt;  // bytes
    long long sxb, sxt;
    long long srb, srt;
    long long smb, smt;  // elements
    long long wsd, wsw;
    int wdtype;
    int B, D, T;
    int n_ttile, n_rowtiles, ctas_per_slab;
    int act;
    int mask_dtype;
    int skip;
    int res_is_x;
    int state_len;
    int w_fast;
};

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

__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, int c0, int c1, int c2, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
                 ::"l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(src)
                 : "memory");
}

template <int DT, int W>
__device__ __forceinline__ void load_weights_tma(const TmaParams& p, int d0, bool in_range,
                                                 float2 (&wp)[W][Pack<DT>::kPairs],
                                                 float2 (&bp)[Pack<DT>::kPairs]) {
    using E = Elem<DT>;
    using T = typename E::type;
    constexpr int VEC = E::kVec;
    constexpr int PAIRS = Pack<DT>::kPairs;
    float wf[VEC * W];
    float bf[VEC];
#pragma unroll
    for (int i = 0; i < VEC * W; ++i) wf[i] = 0.f;
#pragma unroll
    for (int c = 0; c < VEC; ++c) bf[c] = 0.f;
    if (in_range) {
        if (p.w_fast) {
            const char* base = reinterpret_cast<const char*>(p.weight) + (long long)d0 * W * E::kBytes;
#pragma unroll
            for (int j = 0; j < W; ++j) {
                float2 f[PAIRS];
                Pack<DT>::unpack(ld_vec(base + j * 16), f);
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
        if (p.bias != nullptr) {
#pragma unroll
            for (int c = 0; c < VEC; ++c) {
                bf[c] = (p.wdtype == VC1D_F32)
                            ? __ldg(reinterpret_cast<const float*>(p.bias) + d0 + c)
                            : E::to_float(__ldg(reinterpret_cast<const T*>(p.bias) + d0 + c));
            }
        }
    }
#pragma unroll
    for (int w = 0; w < W; ++w) {
#pragma unroll
        for (int q = 0; q < PAIRS; ++q) wp[w][q] = make_float2(wf[(2 * q) * W + w], wf[(2 * q + 1) * W + w]);
    }
#pragma unroll
    for (int q = 0; q < PAIRS; ++q) bp[q] = make_float2(bf[2 * q], bf[2 * q + 1]);
}

// one staged row -> fp32 pairs, with the reference's multiplicative mask (x * mask rounded to
// the I/O dtype); with skip_masked_loads a zero mask makes the row +0 whatever it holds
template <int DT>
__device__ __forceinline__ void decode_smem_row(const uint4& raw, bool mixed, float mk, int skip,
                                                float2 (&f)[Pack<DT>::kPairs]) {
    using PK = Pack<DT>;
    PK::unpack(raw, f);
    if (mixed && mk != 1.0f) {
        if (mk == 0.0f && skip) {
#pragma unroll
            for (int q = 0; q < PK::kPairs; ++q) f[q] = make_float2(0.f, 0.f);
        } else {
            const float2 m2 = make_float2(mk, mk);
#pragma unroll
            for (int q = 0; q < PK::kPairs; ++q) f[q] = PK::round_trip(mul2(f[q], m2));
        }
    }
}
template <int DT>
__device__ __forceinline__ void load_row(const unsigned char* src, bool mixed, float mk, int skip,
                                         float2 (&f)[Pack<DT>::kPairs]) {
    decode_smem_row<DT>(*reinterpret_cast<const uint4*>(src), mixed, mk, skip, f);
}

template <int DT, int W, int LPR>
struct Geometry {
    static constexpr int kH = W - 1;
    static constexpr int kGroups = kConsumerThreads / LPR;          // row groups per tile
    static constexpr int kTileRows = kGroups * kRowsPerThread;      // T_TILE
    static constexpr int kBoxRows = kTileRows + kH;
    static constexpr int kRowBytes = LPR * 16;
    static constexpr int kStageBytes = ((kBoxRows * kRowBytes + 127) / 128) * 128;
    static constexpr int kMaskFloats = ((kBoxRows + 31) / 32) * 32;
    static constexpr int kSmemBytes = kStages * kStageBytes + kStages * kMaskFloats * 4 + 128 /*barriers, flags*/ +
                                      128 /*alignment slack*/;
};

template <int DT, int W, int LPR>
__global__ void __launch_bounds__(kThreads) k_prefill_tma(const __grid_constant__ CUtensorMap tmap_x,
                                                          const __grid_constant__ CUtensorMap tmap_y,
                                                          const TmaParams p) {
    using E = Elem<DT>;
    using PK = Pack<DT>;
    using G = Geometry<DT, W, LPR>;
    constexpr int VEC = E::kVec;
    constexpr int PAIRS = PK::kPairs;
    constexpr int H = G::kH;
    constexpr int R = kRowsPerThread;

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    unsigned char* data = smem;                                                  // kStages * kStageBytes
    float* mask_s = reinterpret_cast<float*>(smem + kStages * G::kStageBytes);   // kStages * kMaskFloats
    uint64_t* bars = reinterpret_cast<uint64_t*>(mask_s + kStages * G::kMaskFloats);  // full[kStages], done[kStages]
    int* flags = reinterpret_cast<int*>(bars + 2 * kStages);                      // tile class per stage, abort

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int slab = blockIdx.x;        // channel slab
    const int j0 = blockIdx.y;          // first row tile of this CTA
    const int stride = p.ctas_per_slab;
    const int slab_ch0 = slab * (LPR * VEC);
    const int n_my = (j0 < p.n_rowtiles) ? (p.n_rowtiles - j0 + stride - 1) / stride : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);                         // full: the producer's arrive (+ tx bytes)
            mbar_init(smem_u32(&bars[kStages + s]), kConsumerWarps);  // done: one arrive per consumer warp
        }
        flags[kStages] = 0;      // a consumer wait expired
        flags[kStages + 1] = 0;  // a producer wait expired
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == kConsumerWarps) {
        // ================================ producer warp ==================================
        // Iteration i issues the load of tile i, then waits for the consumers of tile i-(S-1) and
        // issues its store.  The stage of tile i held tile i-S, whose store was issued in the
        // previous iteration: it is the newest bulk group, so wait_group.read 0 frees the stage.
        bool live = true;
        for (int i = 0; live && i < n_my + kStages - 1; ++i) {
            if (i < n_my) {
                const int s = i % kStages;
                if (i >= kStages && lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                __syncwarp();
                const int rt = j0 + i * stride;
                const int b = rt / p.n_ttile;
                const int t0 = (rt - b * p.n_ttile) * G::kTileRows;
                int cls = TILE_FULL;
                if (p.mask != nullptr) {
                    bool any = false, all_one = true;
                    for (int jrow = lane; jrow < G::kBoxRows; jrow += 32) {
                        const int t = t0 - H + jrow;
                        float mk = 1.0f;          // rows before t = 0 are zero-filled data: any multiplier works
                        if (t >= p.T) mk = 0.0f;  // rows past the end are never stored
                        else if (t >= 0)
                            mk = load_mask(p.mask, (long long)b * p.smb + (long long)t * p.smt, p.mask_dtype);
                        mask_s[s * G::kMaskFloats + jrow] = mk;
                        if (t >= 0 && t < p.T) {
                            any |= (mk != 0.0f);
                            all_one &= (mk == 1.0f);
                        }
                    }
                    any = __any_sync(0xffffffffu, any);
                    all_one = __all_sync(0xffffffffu, all_one);
                    cls = all_one ? TILE_FULL : ((any || !p.skip || p.res != nullptr) ? TILE_MIXED : TILE_EMPTY);
                    __syncwarp();
                }
                if (lane == 0) {
                    flags[s] = cls;
                    const uint32_t full = smem_u32(&bars[s]);
                    if (cls != TILE_EMPTY) {
                        mbar_arrive_expect_tx(full, G::kBoxRows * G::kRowBytes);
                        tma_load_3d(smem_u32(data + s * G::kStageBytes), &tmap_x, slab_ch0, t0 - H, b, full);
                    } else {
                        mbar_arrive(full);
                    }
                }
                __syncwarp();
            }
            const int j = i - (kStages - 1);
            if (j >= 0 && j < n_my) {
                const int s = j % kStages;
                if (!mbar_wait(smem_u32(&bars[kStages + s]), (j / kStages) & 1)) {
                    // recorded only: the consumers decide among themselves when to stop (they share a barrier)
                    if (lane == 0) { atomicAdd(&g_tma_timeouts, 1u); atomicExch(&flags[kStages + 1], 1); }
                    live = false;
                } else if (*reinterpret_cast<volatile int*>(&flags[kStages])) {
                    live = false;
                } else if (lane == 0) {
                    const int rt = j0 + j * stride;
                    const int b = rt / p.n_ttile;
                    const int t0 = (rt - b * p.n_ttile) * G::kTileRows;
                    // output row t sits in box row t - t0 + H: the store starts H rows into the stage
                    tma_store_3d(&tmap_y, slab_ch0, t0, b, smem_u32(data + s * G::kStageBytes + H * G::kRowBytes));
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
                __syncwarp();
            }
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    } else {
        // ================================ consumer warps =================================
        const int grp = threadIdx.x / LPR;   // row group inside the tile
        const int cl = threadIdx.x % LPR;    // channel vector inside the slab
        const int d0 = slab_ch0 + cl * VEC;
        const bool ch_ok = d0 < p.D;         // dim is a multiple of VEC: a vector is in or out as a whole
        const int rbase = grp * R;

        float2 wp[W][PAIRS];
        float2 bp[PAIRS];
        load_weights_tma<DT, W>(p, d0, ch_ok, wp, bp);
        // value of a row whose W taps are all masked: act(bias)
        uint4 const_row;
        {
            float2 c[PAIRS];
#pragma unroll
            for (int q = 0; q < PAIRS; ++q) c[q] = p.act ? silu2<E::kPreciseSilu>(bp[q]) : bp[q];
            const_row = PK::pack(c);
        }

        for (int i = 0; i < n_my; ++i) {
            const int s = i % kStages;
            const bool ok = mbar_wait(smem_u32(&bars[s]), (i / kStages) & 1);
            if (!ok && lane == 0) { atomicAdd(&g_tma_timeouts, 1u); atomicExch(&flags[kStages], 1); }
            const int cls = flags[s];
            const int rt = j0 + i * stride;
            const int b = rt / p.n_ttile;
            const int t0 = (rt - b * p.n_ttile) * G::kTileRows;
            // box row of time t is (t - t0 + H); this thread reads box rows rbase .. rbase+R+H-1 and
            // writes its R results over box rows rbase+H .. rbase+R+H-1 (the rows it has just consumed)
            unsigned char* trow = data + s * G::kStageBytes + cl * 16 + rbase * G::kRowBytes;
            const float* mk = mask_s + s * G::kMaskFloats + rbase;
            const bool mixed = (cls == TILE_MIXED);
            const int tfirst = t0 + rbase;

            float2 hist[H > 0 ? H : 1][PAIRS];
            if (cls != TILE_EMPTY) {
#pragma unroll
                for (int w = 0; w < H; ++w)
                    load_row<DT>(trow + w * G::kRowBytes, mixed, mixed ? mk[w] : 1.0f, p.skip, hist[w]);
            }
            // The first H rows a group reads are the last rows the group above it overwrites: nobody
            // writes until everybody holds its history.  The same barrier makes an expired wait a
            // collective decision, so no warp is left alone at it.
            asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
            if (*reinterpret_cast<volatile int*>(&flags[kStages])) break;

            if (cls == TILE_EMPTY) {
#pragma unroll
                for (int k = 0; k < R; ++k) *reinterpret_cast<uint4*>(trow + (H + k) * G::kRowBytes) = const_row;
            } else {
                const char* rb = (p.res != nullptr && !p.res_is_x && ch_ok)
                                     ? p.res + (long long)b * p.srb + (long long)d0 * E::kBytes
                                     : nullptr;
#pragma unroll
                for (int k = 0; k < R; ++k) {
                    const int t = tfirst + k;
                    uint4* slot = reinterpret_cast<uint4*>(trow + (H + k) * G::kRowBytes);
                    const uint4 rawk = *slot;
                    float2 cur[PAIRS];
                    decode_smem_row<DT>(rawk, mixed, mixed ? mk[H + k] : 1.0f, p.skip, cur);
                    float2 acc[PAIRS];
#pragma unroll
                    for (int q = 0; q < PAIRS; ++q) {
                        acc[q] = bp[q];
#pragma unroll
                        for (int w = 0; w < H; ++w) acc[q] = fma2(wp[w][q], hist[w][q], acc[q]);
                        acc[q] = fma2(wp[H][q], cur[q], acc[q]);
                        if (p.act) acc[q] = silu2<E::kPreciseSilu>(acc[q]);
                    }
                    if (p.res != nullptr) {
                        float2 rr[PAIRS];
                        if (p.res_is_x) {
                            PK::unpack(rawk, rr);  // the unmasked input, already on chip
                        } else {
                            uint4 rv = make_uint4(0u, 0u, 0u, 0u);
                            if (rb != nullptr && t < p.T) rv = ld_vec(rb + (long long)t * p.srt);
                            PK::unpack(rv, rr);
                        }
#pragma unroll
                        for (int q = 0; q < PAIRS; ++q) acc[q] = add2(PK::round_trip(acc[q]), rr[q]);
                    }
                    *slot = PK::pack(acc);
#pragma unroll
                    for (int w = 0; w + 1 < H; ++w) {
#pragma unroll
                        for (int q = 0; q < PAIRS; ++q) hist[w][q] = hist[w + 1][q];
                    }
                    if (H > 0) {
#pragma unroll
                        for (int q = 0; q < PAIRS; ++q) hist[H - 1][q] = cur[q];
                    }
                }
            }
            // results were written through the generic proxy; the bulk store reads through the async proxy
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars[kStages + s]));
        }

        // ---- final state: right-aligned last state_len masked inputs (model/model.py:470-489) ----
        if (p.fstate != nullptr && threadIdx.x < LPR && ch_ok) {
            using T = typename E::type;
            const int L = p.state_len;
            for (int b = j0; b < p.B; b += stride) {
                const char* xb = p.x + (long long)b * p.sxb + (long long)d0 * E::kBytes;
                const long long row0 = (long long)b * p.D + d0;
                for (int jc = 0; jc < L; ++jc) {
                    const int t = p.T - L + jc;
                    uint4 rawv = make_uint4(0u, 0u, 0u, 0u);
                    if (t >= 0) {
                        rawv = ld_vec(xb + (long long)t * p.sxt);
                        if (p.mask != nullptr) {
                            const float mkv = load_mask(p.mask, (long long)b * p.smb + (long long)t * p.smt, p.mask_dtype);
                            if (mkv != 1.0f) {
                                float2 f[PAIRS];
                                PK::unpack(rawv, f);
                                const float2 m2 = make_float2(mkv, mkv);
#pragma unroll
                                for (int q = 0; q < PAIRS; ++q) f[q] = mul2(f[q], m2);
                                rawv = PK::pack(f);
                            }
                        }
                    }
                    T vals[VEC];
                    *reinterpret_cast<uint4*>(vals) = rawv;
                    T* out = reinterpret_cast<T*>(p.fstate);
#pragma unroll
                    for (int c = 0; c < VEC; ++c) out[(row0 + c) * L + jc] = vals[c];
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

EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(sym);
    });
    return fn;
}

template <int DT, int W, int LPR>
cudaError_t launch_geom(const vc1d_prefill_args& a, const TmaParams& base, cudaStream_t s) {
    using G = Geometry<DT, W, LPR>;
    constexpr int VEC = Elem<DT>::kVec;
    const int eb = Elem<DT>::kBytes;
    TmaParams p = base;
    const int slab_ch = LPR * VEC;
    const int n_slab = (a.dim + slab_ch - 1) / slab_ch;
    p.n_ttile = (a.seqlen + G::kTileRows - 1) / G::kTileRows;
    const long long n_rowtiles = (long long)a.batch * p.n_ttile;
    if (n_rowtiles > 0x7fffffffLL || n_slab > 0x7fffffff) return cudaErrorInvalidConfiguration;
    p.n_rowtiles = (int)n_rowtiles;

    EncodeFn enc = encode_fn();
    if (enc == nullptr) return cudaErrorNotSupported;
    const CUtensorMapDataType dt = (DT == VC1D_F32)    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : (DT == VC1D_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                       : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const cuuint64_t dims[3] = {(cuuint64_t)a.dim, (cuuint64_t)a.seqlen, (cuuint64_t)a.batch};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    // input box: tile rows plus the W-1 rows above; output box: the tile rows
    CUtensorMap tmap_x, tmap_y;
    {
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
    {
        cuuint64_t st[2] = {(cuuint64_t)a.y_stride_t * eb, (cuuint64_t)a.y_stride_b * eb};
        if (a.seqlen == 1) st[0] = (cuuint64_t)a.dim * eb;
        if (a.batch == 1) st[1] = st[0] * (cuuint64_t)a.seqlen;
        if (st[0] % 16 != 0 || st[1] % 16 != 0) return cudaErrorNotSupported;
        const cuuint32_t box[3] = {(cuuint32_t)slab_ch, (cuuint32_t)G::kTileRows, 1u};
        const CUresult r = enc(&tmap_y, dt, 3, a.y, dims, st, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorNotSupported;
    }

    {
        // opt in to > 48 KB of dynamic shared memory, once per device
        static std::atomic<bool> done[64];
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev < 0 || dev >= 64 || !done[dev].load(std::memory_order_acquire)) {
            const cudaError_t e = cudaFuncSetAttribute(k_prefill_tma<DT, W, LPR>,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, G::kSmemBytes);
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 64) done[dev].store(true, std::memory_order_release);
        }
    }

    // persistent CTAs: three per SM, split evenly over the channel slabs
    int per_sm = a.block_threads > 0 ? a.block_threads : 3;  // block_threads doubles as CTAs/SM override here
    if (per_sm > 8) per_sm = 3;
    long long g = ((long long)sm_count() * per_sm) / n_slab;
    if (g < 1) g = 1;
    if (g > n_rowtiles) g = n_rowtiles;
    if (g > 65535) g = 65535;
    p.ctas_per_slab = (int)g;
    const dim3 grid((unsigned)n_slab, (unsigned)g);
    note_launch("tma");
    k_prefill_tma<DT, W, LPR><<<grid, kThreads, G::kSmemBytes, s>>>(tmap_x, tmap_y, p);
    return cudaGetLastError();
}

template <int DT, int W>
cudaError_t launch_w(const vc1d_prefill_args& a, const TmaParams& p, cudaStream_t s) {
    // 256-byte slabs when dim fills them; 128-byte slabs when that avoids idle lanes
    const int vec = Elem<DT>::kVec;
    const int wide = 16 * vec, narrow = 8 * vec;
    const bool use_wide = (a.dim % wide == 0) || (a.dim % narrow != 0);
    if (a.rows_per_thread == 8) return launch_geom<DT, W, 8>(a, p, s);    // tuning override: narrow slabs
    if (a.rows_per_thread == 16) return launch_geom<DT, W, 16>(a, p, s);  // tuning override: wide slabs
    return use_wide ? launch_geom<DT, W, 16>(a, p, s) : launch_geom<DT, W, 8>(a, p, s);
}

template <int DT>
cudaError_t launch_dt(const vc1d_prefill_args& a, const TmaParams& p, cudaStream_t s) {
    switch (a.width) {
        case 2: return launch_w<DT, 2>(a, p, s);
        case 3: return launch_w<DT, 3>(a, p, s);
        default: return launch_w<DT, 4>(a, p, s);
    }
}

}  // namespace

bool tma_available() { return encode_fn() != nullptr; }

unsigned int tma_timeouts() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tma_timeouts, sizeof(v)) != cudaSuccess) return 0xffffffffu;
    return v;
}

cudaError_t launch_prefill_tma(const vc1d_prefill_args& a, cudaStream_t s) {
    const int eb = elem_bytes(a.dtype);
    TmaParams p;
    p.y = reinterpret_cast<char*>(a.y);
    p.x = reinterpret_cast<const char*>(a.x);
    p.res = reinterpret_cast<const char*>(a.residual);
    p.weight = a.weight;
    p.bias = a.bias;
    p.mask = a.mask;
    p.fstate = reinterpret_cast<char*>(a.final_state);
    p.syb = a.y_stride_b * eb;
    p.syt = a.y_stride_t * eb;
    p.sxb = a.x_stride_b * eb;
    p.sxt = a.x_stride_t * eb;
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
    p.n_ttile = p.n_rowtiles = p.ctas_per_slab = 0;
    p.act = a.activation;
    p.mask_dtype = a.mask_dtype;
    p.skip = (a.mask != nullptr && a.skip_masked_loads) ? 1 : 0;
    p.res_is_x = (a.residual != nullptr && a.residual == a.x && a.r_stride_b == a.x_stride_b &&
                  a.r_stride_t == a.x_stride_t)
                     ? 1
                     : 0;
    p.state_len = a.state_len;
    p.w_fast = (a.wdtype == a.dtype && a.w_stride_w == 1 && a.w_stride_d == a.width &&
                (reinterpret_cast<uintptr_t>(a.weight) & 15u) == 0)
                   ? 1
                   : 0;
    switch (a.dtype) {
        case VC1D_F32: return launch_dt<VC1D_F32>(a, p, s);
        case VC1D_BF16: return launch_dt<VC1D_BF16>(a, p, s);
        default: return launch_dt<VC1D_F16>(a, p, s);
    }
}

}  // namespace vc1d
