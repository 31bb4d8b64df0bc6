// Device-side helpers shared by every kernel of the library: 128-bit vector access,
// element <-> fp32 conversion, packed fp32x2 arithmetic and the SiLU epilogue.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "../../include/vc1d.h"

namespace vc1d {

// ---------------------------------------------------------------------------------------
// Element traits.  VEC = elements in one 128-bit access.
// ---------------------------------------------------------------------------------------
template <int DT>
struct Elem;

template <>
struct Elem<VC1D_F32> {
    using type = float;
    static constexpr int kBytes = 4;
    static constexpr int kVec = 4;
    static constexpr bool kPreciseSilu = true;
    __device__ __forceinline__ static float to_float(float v) { return v; }
    __device__ __forceinline__ static float from_float(float v) { return v; }
};

template <>
struct Elem<VC1D_BF16> {
    using type = __nv_bfloat16;
    static constexpr int kBytes = 2;
    static constexpr int kVec = 8;
    static constexpr bool kPreciseSilu = false;
    __device__ __forceinline__ static float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ __forceinline__ static __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
};

template <>
struct Elem<VC1D_F16> {
    using type = __half;
    static constexpr int kBytes = 2;
    static constexpr int kVec = 8;
    static constexpr bool kPreciseSilu = false;
    __device__ __forceinline__ static float to_float(__half v) { return __half2float(v); }
    __device__ __forceinline__ static __half from_float(float v) { return __float2half_rn(v); }
};

// ---------------------------------------------------------------------------------------
// 128-bit global accesses.  Inputs are read once per CTA neighbourhood (halo rows are the
// only reuse), outputs are never read back: stream the stores past L1/L2 residency.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ld_vec(const void* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ uint4 ld_vec_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void st_vec_stream(void* p, const uint4& v) {
    __stcs(reinterpret_cast<uint4*>(p), v);
}
__device__ __forceinline__ void st_vec(void* p, const uint4& v) {
    *reinterpret_cast<uint4*>(p) = v;
}

// ---------------------------------------------------------------------------------------
// Programmatic dependent launch.  A kernel launched with the programmatic-stream-serialization
// attribute may begin before its predecessor in the stream has finished; griddep_wait() returns
// once the predecessor has completed and its writes are visible (at once when the attribute is
// absent), so every thread calls it before its first global access.  griddep_launch_dependents()
// lets the next such kernel of the stream start its own prologue.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------------------
// Packed fp32x2 arithmetic (sm_100 issues one instruction for two fp32 lanes).
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long f2_bits(float2 v) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(v.x), "f"(v.y));
    return r;
}
__device__ __forceinline__ float2 bits_f2(unsigned long long r) {
    float2 v;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(v.x), "=f"(v.y) : "l"(r));
    return v;
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ >= 1000)
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(f2_bits(a)), "l"(f2_bits(b)), "l"(f2_bits(c)));
    return bits_f2(d);
#else
    return make_float2(fmaf(a.x, b.x, c.x), fmaf(a.y, b.y, c.y));
#endif
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ >= 1000)
    unsigned long long d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(f2_bits(a)), "l"(f2_bits(b)));
    return bits_f2(d);
#else
    return make_float2(a.x * b.x, a.y * b.y);
#endif
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ >= 1000)
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(f2_bits(a)), "l"(f2_bits(b)));
    return bits_f2(d);
#else
    return make_float2(a.x + b.x, a.y + b.y);
#endif
}

// ---------------------------------------------------------------------------------------
// Unpack one 128-bit vector into kVec/2 fp32 pairs and back.
// ---------------------------------------------------------------------------------------
template <int DT>
struct Pack;

template <>
struct Pack<VC1D_F32> {
    static constexpr int kPairs = 2;
    __device__ __forceinline__ static void unpack(const uint4& v, float2 (&f)[2]) {
        f[0] = make_float2(__uint_as_float(v.x), __uint_as_float(v.y));
        f[1] = make_float2(__uint_as_float(v.z), __uint_as_float(v.w));
    }
    __device__ __forceinline__ static uint4 pack(const float2 (&f)[2]) {
        return make_uint4(__float_as_uint(f[0].x), __float_as_uint(f[0].y), __float_as_uint(f[1].x),
                          __float_as_uint(f[1].y));
    }
    // round an fp32 pair to the element type and back (used by the multiplicative mask)
    __device__ __forceinline__ static float2 round_trip(float2 f) { return f; }
};

template <>
struct Pack<VC1D_BF16> {
    static constexpr int kPairs = 4;
    __device__ __forceinline__ static float2 up(uint32_t u) {
        // bf16 -> fp32 is a 16-bit left shift: low half by shifting, high half by masking
        return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
    }
    __device__ __forceinline__ static uint32_t down(float2 f) {
        __nv_bfloat162 h = __float22bfloat162_rn(f);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    __device__ __forceinline__ static void unpack(const uint4& v, float2 (&f)[4]) {
        f[0] = up(v.x);
        f[1] = up(v.y);
        f[2] = up(v.z);
        f[3] = up(v.w);
    }
    __device__ __forceinline__ static uint4 pack(const float2 (&f)[4]) {
        return make_uint4(down(f[0]), down(f[1]), down(f[2]), down(f[3]));
    }
    __device__ __forceinline__ static float2 round_trip(float2 f) { return up(down(f)); }
};

template <>
struct Pack<VC1D_F16> {
    static constexpr int kPairs = 4;
    __device__ __forceinline__ static float2 up(uint32_t u) {
        return __half22float2(*reinterpret_cast<const __half2*>(&u));
    }
    __device__ __forceinline__ static uint32_t down(float2 f) {
        __half2 h = __float22half2_rn(f);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    __device__ __forceinline__ static void unpack(const uint4& v, float2 (&f)[4]) {
        f[0] = up(v.x);
        f[1] = up(v.y);
        f[2] = up(v.z);
        f[3] = up(v.w);
    }
    __device__ __forceinline__ static uint4 pack(const float2 (&f)[4]) {
        return make_uint4(down(f[0]), down(f[1]), down(f[2]), down(f[3]));
    }
    __device__ __forceinline__ static float2 round_trip(float2 f) { return up(down(f)); }
};

// ---------------------------------------------------------------------------------------
// SiLU, x / (1 + exp(-x)) (reference: causal_conv1d.metal:95-97, model/model.py:669-670).
// fp32 I/O uses the accurate expf and an IEEE division (1e-5 relative budget); 16-bit I/O
// uses ex2.approx + rcp.approx, whose ~2^-22 relative error vanishes under the final
// rounding to 8 or 11 mantissa bits.  Two special-function ops per element is the scarce
// resource of this kernel at HBM speed, so everything around them is packed fp32x2.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float silu_precise(float v) { return v / (1.0f + expf(-v)); }

__device__ __forceinline__ float ex2_approx(float v) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ float rcp_approx(float v) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}

template <bool PRECISE>
__device__ __forceinline__ float2 silu2(float2 v) {
    if (PRECISE) {
        return make_float2(silu_precise(v.x), silu_precise(v.y));
    } else {
        const float2 t = mul2(v, make_float2(-1.4426950408889634f, -1.4426950408889634f));
        float2 e = make_float2(ex2_approx(t.x), ex2_approx(t.y));
        e = add2(e, make_float2(1.0f, 1.0f));
        const float2 r = make_float2(rcp_approx(e.x), rcp_approx(e.y));
        return mul2(v, r);
    }
}

template <bool PRECISE>
__device__ __forceinline__ float silu1(float v) {
    if (PRECISE) return silu_precise(v);
    return v * rcp_approx(1.0f + ex2_approx(v * -1.4426950408889634f));
}

// ---------------------------------------------------------------------------------------
// Mask element of any supported type as a float multiplier.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float load_mask(const void* base, int64_t idx, int mask_dtype) {
    switch (mask_dtype) {
        case VC1D_U8:
            return (float)__ldg(reinterpret_cast<const uint8_t*>(base) + idx);
        case VC1D_I32:
            return (float)__ldg(reinterpret_cast<const int32_t*>(base) + idx);
        case VC1D_I64:
            return (float)__ldg(reinterpret_cast<const long long*>(base) + idx);
        case VC1D_F32:
            return __ldg(reinterpret_cast<const float*>(base) + idx);
        case VC1D_BF16:
            return __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16*>(base) + idx));
        case VC1D_F16:
            return __half2float(__ldg(reinterpret_cast<const __half*>(base) + idx));
        default:
            return 1.0f;
    }
}

// Compile-time loop: f is called with std::integral_constant<int, K> for K = first .. last-1.
template <int K, int N, class F>
__device__ __forceinline__ void static_for(F&& f) {
    if constexpr (K < N) {
        f(std::integral_constant<int, K>{});
        static_for<K + 1, N>(f);
    }
}

// ---- a thread's slice of one row: VB bytes = NP fp32 pairs ----------------------------------------
template <int DT, int VB>
struct Slice {
    static constexpr int kElems = VB / Elem<DT>::kBytes;
    static constexpr int kPairs = kElems / 2;
    static constexpr int kWords = VB / 4;

    __device__ __forceinline__ static void lds(uint32_t a, uint32_t (&r)[kWords]) {
        if constexpr (VB == 16)
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(r[0]), "=r"(r[1]), "=r"(r[kWords > 2 ? 2 : 0]), "=r"(r[kWords > 3 ? 3 : 0])
                         : "r"(a));
        else if constexpr (VB == 8)
            asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[kWords > 1 ? 1 : 0]) : "r"(a));
        else
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(r[0]) : "r"(a));
    }
    __device__ __forceinline__ static void sts(uint32_t a, const uint32_t (&r)[kWords]) {
        if constexpr (VB == 16)
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(r[0]), "r"(r[1]),
                         "r"(r[kWords > 2 ? 2 : 0]), "r"(r[kWords > 3 ? 3 : 0])
                         : "memory");
        else if constexpr (VB == 8)
            asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(a), "r"(r[0]), "r"(r[kWords > 1 ? 1 : 0]) : "memory");
        else
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(r[0]) : "memory");
    }
    __device__ __forceinline__ static void ldg(const void* g, uint32_t (&r)[kWords]) {
        if constexpr (VB == 16)
            asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(r[0]), "=r"(r[1]), "=r"(r[kWords > 2 ? 2 : 0]), "=r"(r[kWords > 3 ? 3 : 0])
                         : "l"(g));
        else if constexpr (VB == 8)
            asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[kWords > 1 ? 1 : 0]) : "l"(g));
        else
            asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(r[0]) : "l"(g));
    }
    __device__ __forceinline__ static void stg(void* g, const uint32_t (&r)[kWords]) {
        if constexpr (VB == 16)
            asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(g), "r"(r[0]), "r"(r[1]),
                         "r"(r[kWords > 2 ? 2 : 0]), "r"(r[kWords > 3 ? 3 : 0])
                         : "memory");
        else if constexpr (VB == 8)
            asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(g), "r"(r[0]), "r"(r[kWords > 1 ? 1 : 0]) : "memory");
        else
            asm volatile("st.global.cs.u32 [%0], %1;" ::"l"(g), "r"(r[0]) : "memory");
    }
    // Streaming store of row K of a thread's rows, predicated on K < rows_ok inside the instruction
    // (a guarded store written in C++ around inline assembly becomes a branch per row instead).
    template <int K>
    __device__ __forceinline__ static void stg_row(void* g, const uint32_t (&r)[kWords], int rows_ok) {
        if constexpr (VB == 16)
            asm volatile(
                "{\n .reg .pred p;\n setp.gt.s32 p, %5, %6;\n @p st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};\n}" ::"l"(g),
                "r"(r[0]), "r"(r[1]), "r"(r[kWords > 2 ? 2 : 0]), "r"(r[kWords > 3 ? 3 : 0]), "r"(rows_ok), "n"(K)
                : "memory");
        else if constexpr (VB == 8)
            asm volatile("{\n .reg .pred p;\n setp.gt.s32 p, %3, %4;\n @p st.global.cs.v2.u32 [%0], {%1,%2};\n}" ::"l"(g),
                         "r"(r[0]), "r"(r[kWords > 1 ? 1 : 0]), "r"(rows_ok), "n"(K)
                         : "memory");
        else
            asm volatile("{\n .reg .pred p;\n setp.gt.s32 p, %2, %3;\n @p st.global.cs.u32 [%0], %1;\n}" ::"l"(g),
                         "r"(r[0]), "r"(rows_ok), "n"(K)
                         : "memory");
    }
    __device__ __forceinline__ static void unpack(const uint32_t (&r)[kWords], float2 (&f)[kPairs]) {
        if constexpr (DT == VC1D_F32) {
#pragma unroll
            for (int q = 0; q < kPairs; ++q) f[q] = make_float2(__uint_as_float(r[2 * q]), __uint_as_float(r[2 * q + 1]));
        } else if constexpr (DT == VC1D_BF16) {
#pragma unroll
            for (int q = 0; q < kPairs; ++q) f[q] = Pack<VC1D_BF16>::up(r[q]);
        } else {
#pragma unroll
            for (int q = 0; q < kPairs; ++q) f[q] = Pack<VC1D_F16>::up(r[q]);
        }
    }
    __device__ __forceinline__ static void pack(const float2 (&f)[kPairs], uint32_t (&r)[kWords]) {
        if constexpr (DT == VC1D_F32) {
#pragma unroll
            for (int q = 0; q < kPairs; ++q) {
                r[2 * q] = __float_as_uint(f[q].x);
                r[2 * q + 1] = __float_as_uint(f[q].y);
            }
        } else if constexpr (DT == VC1D_BF16) {
#pragma unroll
            for (int q = 0; q < kPairs; ++q) r[q] = Pack<VC1D_BF16>::down(f[q]);
        } else {
#pragma unroll
            for (int q = 0; q < kPairs; ++q) r[q] = Pack<VC1D_F16>::down(f[q]);
        }
    }
    __device__ __forceinline__ static float2 round_trip(float2 f) { return Pack<DT>::round_trip(f); }
};

}  // namespace vc1d
