// C-ABI layer: argument validation, kernel selection, bookkeeping.  No kernel lives here.
#include <atomic>
#include <cstdlib>
#include <cstdio>
#include <cstring>

#include "vc1d_internal.h"

namespace vc1d {

namespace {
std::atomic<uint64_t> g_launches{0};
thread_local const char* t_last_kernel = "none";
thread_local int t_class_table = 0;
std::atomic<int> g_sm_count[64];
}  // namespace

int sm_count() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = g_sm_count[dev].load(std::memory_order_relaxed);
    if (n > 0) return n;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sm_count[dev].store(n, std::memory_order_relaxed);
    return n;
}

namespace {
std::atomic<int> g_pdl_override{-1};  // -1: follow the environment; 0 / 1: set by vc1d_set_pdl
}

bool pdl_enabled() {
    static const bool env_on = [] {
        const char* v = std::getenv("VC1D_NO_PDL");
        return !(v != nullptr && v[0] == '1');
    }();
    const int o = g_pdl_override.load(std::memory_order_relaxed);
    return o < 0 ? env_on : (o != 0);
}

void note_class_table(int state) { t_class_table = state; }

void note_launch(const char* kernel_name) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    t_last_kernel = kernel_name;
}

namespace {

inline bool is_io_dtype(int dt) { return dt == VC1D_F32 || dt == VC1D_BF16 || dt == VC1D_F16; }
inline bool is_mask_dtype(int dt) {
    return dt == VC1D_U8 || dt == VC1D_I32 || dt == VC1D_I64 || dt == VC1D_F32 || dt == VC1D_BF16 ||
           dt == VC1D_F16;
}
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// byte range [lo, hi) touched by a strided 3-d tensor
struct Range {
    const char* lo;
    const char* hi;
};
Range extent3(const void* base, int eb, long long n0, long long s0, long long n1, long long s1, long long n2,
              long long s2) {
    long long lo = 0, hi = 0;
    const long long n[3] = {n0, n1, n2};
    const long long s[3] = {s0, s1, s2};
    for (int i = 0; i < 3; ++i) {
        const long long span = (n[i] - 1) * s[i];
        if (span < 0)
            lo += span;
        else
            hi += span;
    }
    const char* b = reinterpret_cast<const char*>(base);
    return {b + lo * eb, b + (hi + 1) * eb};
}
inline bool overlaps(const Range& a, const Range& b) { return a.lo < b.hi && b.lo < a.hi; }

int check_prefill(const vc1d_prefill_args* a) {
    if (a == nullptr) return VC1D_E_NULL;
    if (a->struct_size != sizeof(vc1d_prefill_args)) return VC1D_E_STRUCT;
    if (!is_io_dtype(a->dtype)) return VC1D_E_DTYPE;
    if (a->wdtype != a->dtype && a->wdtype != VC1D_F32) return VC1D_E_DTYPE;
    if (a->activation != VC1D_ACT_NONE && a->activation != VC1D_ACT_SILU) return VC1D_E_ACTIVATION;
    if (a->width < 2 || a->width > 4) return VC1D_E_WIDTH;
    if (a->batch < 0 || a->dim < 0 || a->seqlen < 0) return VC1D_E_SHAPE;
    if (a->mask != nullptr && !is_mask_dtype(a->mask_dtype)) return VC1D_E_DTYPE;
    if (a->initial_state != nullptr && a->init_len < a->width - 1) return VC1D_E_SHAPE;
    if (a->final_state != nullptr && a->state_len < 1) return VC1D_E_SHAPE;
    if (a->kernel < VC1D_KERNEL_AUTO || a->kernel > VC1D_KERNEL_TMA) return VC1D_E_SHAPE;
    if (a->seq_idx != nullptr && (a->mask != nullptr || a->initial_state != nullptr || a->final_state != nullptr))
        return VC1D_E_SHAPE;
    const long long n = (long long)a->batch * a->dim * a->seqlen;
    if (n == 0) return VC1D_OK;
    if (a->x == nullptr || a->y == nullptr || a->weight == nullptr) return VC1D_E_NULL;
    // y must not overlap x (halo rows of x are re-read after neighbouring outputs are written)
    const int eb = elem_bytes(a->dtype);
    const Range rx = extent3(a->x, eb, a->batch, a->x_stride_b, a->dim, a->x_stride_d, a->seqlen, a->x_stride_t);
    const Range ry = extent3(a->y, eb, a->batch, a->y_stride_b, a->dim, a->y_stride_d, a->seqlen, a->y_stride_t);
    if (overlaps(rx, ry)) return VC1D_E_ALIAS;
    if (a->residual != nullptr) {
        const Range rr = extent3(a->residual, eb, a->batch, a->r_stride_b, a->dim, a->r_stride_d, a->seqlen,
                                 a->r_stride_t);
        if (overlaps(rr, ry) && !(a->residual == a->y && a->r_stride_b == a->y_stride_b &&
                                  a->r_stride_d == a->y_stride_d && a->r_stride_t == a->y_stride_t))
            return VC1D_E_ALIAS;
    }
    return VC1D_OK;
}

bool channel_last_ok(const vc1d_prefill_args* a) {
    const int eb = elem_bytes(a->dtype);
    const int vec = 16 / eb;
    if (a->dim % vec != 0) return false;
    if (a->x_stride_d != 1 || a->y_stride_d != 1) return false;
    if (!aligned16(a->x) || !aligned16(a->y)) return false;
    if (a->x_stride_b % vec || a->x_stride_t % vec || a->y_stride_b % vec || a->y_stride_t % vec) return false;
    if (a->residual != nullptr) {
        if (a->r_stride_d != 1 || !aligned16(a->residual) || a->r_stride_b % vec || a->r_stride_t % vec)
            return false;
    }
    return true;
}

bool time_major_ok(const vc1d_prefill_args* a) {
    const int eb = elem_bytes(a->dtype);
    const int vec = 16 / eb;
    if (a->mask || a->residual || a->initial_state || a->final_state) return false;
    if (a->seqlen % vec != 0) return false;
    if (a->x_stride_t != 1 || a->y_stride_t != 1) return false;
    if (!aligned16(a->x) || !aligned16(a->y)) return false;
    if (a->x_stride_b % vec || a->x_stride_d % vec || a->y_stride_b % vec || a->y_stride_d % vec) return false;
    return true;
}

int check_prefill_bwd(const vc1d_prefill_bwd_args* a) {
    if (a == nullptr) return VC1D_E_NULL;
    if (a->struct_size != sizeof(vc1d_prefill_bwd_args)) return VC1D_E_STRUCT;
    if (!is_io_dtype(a->dtype)) return VC1D_E_DTYPE;
    if (a->wdtype != a->dtype && a->wdtype != VC1D_F32) return VC1D_E_DTYPE;
    if (a->activation != VC1D_ACT_NONE && a->activation != VC1D_ACT_SILU) return VC1D_E_ACTIVATION;
    if (a->width < 2 || a->width > 4) return VC1D_E_WIDTH;
    if (a->batch < 0 || a->dim < 0 || a->seqlen < 0) return VC1D_E_SHAPE;
    if (a->mask != nullptr && !is_mask_dtype(a->mask_dtype)) return VC1D_E_DTYPE;
    if (a->kernel != VC1D_KERNEL_AUTO && a->kernel != VC1D_KERNEL_GENERIC && a->kernel != VC1D_KERNEL_TMA)
        return VC1D_E_SHAPE;
    if (a->initial_state != nullptr && a->init_len < a->width - 1) return VC1D_E_SHAPE;
    if (a->initial_state == nullptr && a->dinitial_state != nullptr) return VC1D_E_NULL;
    if (a->seq_idx != nullptr && (a->mask != nullptr || a->initial_state != nullptr)) return VC1D_E_SHAPE;
    if ((long long)a->batch * a->dim * a->seqlen == 0) return VC1D_OK;
    if (a->x == nullptr || a->dy == nullptr || a->dx == nullptr || a->weight == nullptr) return VC1D_E_NULL;
    const int eb = elem_bytes(a->dtype);
    const Range rx = extent3(a->x, eb, a->batch, a->x_stride_b, a->dim, a->x_stride_d, a->seqlen, a->x_stride_t);
    const Range rg = extent3(a->dy, eb, a->batch, a->dy_stride_b, a->dim, a->dy_stride_d, a->seqlen, a->dy_stride_t);
    const Range rd = extent3(a->dx, eb, a->batch, a->dx_stride_b, a->dim, a->dx_stride_d, a->seqlen, a->dx_stride_t);
    if (overlaps(rx, rd) || overlaps(rg, rd)) return VC1D_E_ALIAS;  // neighbours' rows are read after dx rows are written
    return VC1D_OK;
}

bool bwd_channel_last_ok(const vc1d_prefill_bwd_args* a) {
    const int eb = elem_bytes(a->dtype);
    const int vec = 16 / eb;
    if (a->dim % vec != 0) return false;
    if (a->x_stride_d != 1 || a->dy_stride_d != 1 || a->dx_stride_d != 1) return false;
    if (!aligned16(a->x) || !aligned16(a->dy) || !aligned16(a->dx)) return false;
    if (a->x_stride_b % vec || a->x_stride_t % vec || a->dy_stride_b % vec || a->dy_stride_t % vec ||
        a->dx_stride_b % vec || a->dx_stride_t % vec)
        return false;
    return true;
}

int check_update(const vc1d_update_args* a) {
    if (a == nullptr) return VC1D_E_NULL;
    if (a->struct_size != sizeof(vc1d_update_args)) return VC1D_E_STRUCT;
    if (!is_io_dtype(a->dtype)) return VC1D_E_DTYPE;
    if (a->wdtype != a->dtype && a->wdtype != VC1D_F32) return VC1D_E_DTYPE;
    if (a->activation != VC1D_ACT_NONE && a->activation != VC1D_ACT_SILU) return VC1D_E_ACTIVATION;
    if (a->width < 2 || a->width > 4) return VC1D_E_WIDTH;
    if (a->batch < 0 || a->dim < 0) return VC1D_E_SHAPE;
    if (a->state_len < a->width - 1 || a->state_len < 1) return VC1D_E_SHAPE;
    if (a->kernel != VC1D_KERNEL_AUTO && a->kernel != VC1D_KERNEL_GENERIC) return VC1D_E_SHAPE;
    if ((long long)a->batch * a->dim == 0) return VC1D_OK;
    if (a->x == nullptr || a->y == nullptr || a->weight == nullptr || a->conv_state == nullptr) return VC1D_E_NULL;
    return VC1D_OK;
}

bool update_vec_ok(const vc1d_update_args* a) {
    const int eb = elem_bytes(a->dtype);
    const int vec = 16 / eb;
    if (a->cache_seqlens != nullptr) return false;
    if (!update_vec_supports(a->state_len, a->width)) return false;
    if (a->dim % vec != 0) return false;
    if (a->x_stride_d != 1 || a->y_stride_d != 1) return false;
    if (a->s_stride_l != 1 || a->s_stride_d != a->state_len) return false;
    if (!aligned16(a->x) || !aligned16(a->y) || !aligned16(a->conv_state)) return false;
    if (a->x_stride_b % vec || a->y_stride_b % vec || a->s_stride_b % vec) return false;
    return true;
}

// one channel per lane: state rows of 16 or 32 bytes; takes the circular state and the 8-column states
bool update_lane_ok(const vc1d_update_args* a) {
    const int eb = elem_bytes(a->dtype);
    if (!update_lane_supports(a->dtype, a->state_len, a->width)) return false;
    if (a->x_stride_d != 1 || a->y_stride_d != 1) return false;
    if (a->s_stride_l != 1 || a->s_stride_d != a->state_len) return false;
    if (!aligned16(a->conv_state) || (a->s_stride_b * eb) % 16 != 0) return false;
    // the 128-bit-per-8-channels kernel keeps the short shifting states
    if (a->cache_seqlens == nullptr && a->state_len * eb == 16 && eb == 4 && update_vec_ok(a)) return false;
    return true;
}

}  // namespace
}  // namespace vc1d

extern "C" {

VC1D_API int vc1d_prefill(const vc1d_prefill_args* a, void* stream) {
    using namespace vc1d;
    note_class_table(0);
    const int st = check_prefill(a);
    if (st != VC1D_OK) return st;
    if ((long long)a->batch * a->dim * a->seqlen == 0) return VC1D_OK;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const bool cl = channel_last_ok(a);
    const bool tm = time_major_ok(a);
    cudaError_t err;
    if (a->seq_idx != nullptr) {
        // packed rows: the TMA-staged kernel when it applies, else the scalar kernel
        if (a->kernel == VC1D_KERNEL_CHANNEL_LAST || a->kernel == VC1D_KERNEL_TIME_MAJOR) return VC1D_E_STRIDE;
        if (a->kernel == VC1D_KERNEL_TMA && (!cl || !tma_available())) return VC1D_E_STRIDE;
        const long long elems = (long long)a->batch * a->dim * a->seqlen;
        err = cudaErrorNotSupported;
        if (a->kernel != VC1D_KERNEL_GENERIC && cl && tma_available() &&
            (a->kernel == VC1D_KERNEL_TMA || (a->seqlen >= 16 && elems >= (1LL << 20))))
            err = launch_prefill_tma(*a, s);
        if (err == cudaErrorNotSupported && a->kernel != VC1D_KERNEL_TMA) err = launch_prefill_generic(*a, s);
        return (int)err;
    }
    switch (a->kernel) {
        case VC1D_KERNEL_CHANNEL_LAST:
            if (!cl) return VC1D_E_STRIDE;
            err = launch_prefill_channel_last(*a, s);
            break;
        case VC1D_KERNEL_TMA:
            if (!cl || !tma_available()) return VC1D_E_STRIDE;
            err = launch_prefill_tma(*a, s);
            break;
        case VC1D_KERNEL_TIME_MAJOR:
            if (!tm) return VC1D_E_STRIDE;
            err = launch_prefill_time_major(*a, s);
            break;
        case VC1D_KERNEL_GENERIC:
            err = launch_prefill_generic(*a, s);
            break;
        default:
            // a dim-1 or seqlen-1 tensor can satisfy both layouts; channel-last carries the fused options
            if (cl && (a->dim > 1 || !tm)) {
                // large problems stream through the TMA pipeline; small ones are launch-bound and
                // take the direct kernel, as does anything the tensor map cannot describe
                const long long elems = (long long)a->batch * a->dim * a->seqlen;
                err = cudaErrorNotSupported;
                if (a->seqlen >= 16 && elems >= (1LL << 20) && tma_available())
                    err = launch_prefill_tma(*a, s);
                if (err == cudaErrorNotSupported) err = launch_prefill_channel_last(*a, s);
            } else if (tm) {
                err = launch_prefill_time_major(*a, s);
            } else {
                err = launch_prefill_generic(*a, s);
            }
            break;
    }
    return (int)err;
}

VC1D_API int vc1d_prefill_bwd(const vc1d_prefill_bwd_args* a, void* stream) {
    using namespace vc1d;
    const int st = check_prefill_bwd(a);
    if (st != VC1D_OK) return st;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if ((long long)a->batch * a->dim * a->seqlen == 0) {
        // nothing to sum: the gradients of the parameters are zero
        if (a->zero_grads && a->dim > 0) {
            cudaError_t e = a->dweight != nullptr
                                ? cudaMemsetAsync(a->dweight, 0, sizeof(float) * (size_t)a->dim * a->width, s)
                                : cudaSuccess;
            if (e == cudaSuccess && a->dbias != nullptr) e = cudaMemsetAsync(a->dbias, 0, sizeof(float) * (size_t)a->dim, s);
            return (int)e;
        }
        return VC1D_OK;
    }
    const bool cl = bwd_channel_last_ok(a);
    cudaError_t err;
    switch (a->kernel) {
        case VC1D_KERNEL_GENERIC:
            err = launch_prefill_bwd_generic(*a, s);
            break;
        case VC1D_KERNEL_TMA:
            if (!cl || !tma_available() || a->initial_state != nullptr) return VC1D_E_STRIDE;
            err = launch_prefill_bwd_tma(*a, s);
            break;
        default: {
            const long long elems = (long long)a->batch * a->dim * a->seqlen;
            err = cudaErrorNotSupported;
            if (cl && a->initial_state == nullptr && a->seqlen >= 16 && elems >= (1LL << 18) && tma_available())
                err = launch_prefill_bwd_tma(*a, s);
            if (err == cudaErrorNotSupported) err = launch_prefill_bwd_generic(*a, s);
            break;
        }
    }
    return (int)err;
}

VC1D_API uint32_t vc1d_sizeof_prefill_bwd_args(void) { return (uint32_t)sizeof(vc1d_prefill_bwd_args); }

VC1D_API int vc1d_update(const vc1d_update_args* a, void* stream) {
    using namespace vc1d;
    const int st = check_update(a);
    if (st != VC1D_OK) return st;
    if ((long long)a->batch * a->dim == 0) return VC1D_OK;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    cudaError_t err;
    if (a->kernel == VC1D_KERNEL_AUTO && update_lane_ok(a))
        err = launch_update_lane(*a, s);
    else if (a->kernel == VC1D_KERNEL_AUTO && update_vec_ok(a))
        err = launch_update_vec(*a, s);
    else
        err = launch_update_generic(*a, s);
    return (int)err;
}

VC1D_API int vc1d_update_multi(const vc1d_update_args* calls, int32_t n_calls, void* stream) {
    using namespace vc1d;
    if (n_calls == 0) return VC1D_OK;
    if (calls == nullptr) return VC1D_E_NULL;
    if (n_calls < 0 || n_calls > VC1D_UPDATE_MULTI_MAX) return VC1D_E_SHAPE;
    // problems with nothing to do are left out; the rest must share the I/O dtype (one kernel instantiation)
    static thread_local vc1d_update_args live[VC1D_UPDATE_MULTI_MAX];
    unsigned char vec_ok[VC1D_UPDATE_MULTI_MAX];
    int n = 0;
    for (int i = 0; i < n_calls; ++i) {
        const int st = check_update(&calls[i]);
        if (st != VC1D_OK) return st;
        if ((long long)calls[i].batch * calls[i].dim == 0) continue;
        if (n > 0 && calls[i].dtype != live[0].dtype) return VC1D_E_DTYPE;
        live[n] = calls[i];
        vec_ok[n] = (calls[i].kernel == VC1D_KERNEL_AUTO && update_vec_ok(&calls[i])) ? 1 : 0;
        ++n;
    }
    if (n == 0) return VC1D_OK;
    return (int)launch_update_multi(live, n, vec_ok, reinterpret_cast<cudaStream_t>(stream));
}

VC1D_API int vc1d_update_bwd(const vc1d_update_bwd_args* a, void* stream) {
    using namespace vc1d;
    if (a == nullptr) return VC1D_E_NULL;
    if (a->struct_size != sizeof(vc1d_update_bwd_args)) return VC1D_E_STRUCT;
    if (!is_io_dtype(a->dtype)) return VC1D_E_DTYPE;
    if (a->wdtype != a->dtype && a->wdtype != VC1D_F32) return VC1D_E_DTYPE;
    if (a->activation != VC1D_ACT_NONE && a->activation != VC1D_ACT_SILU) return VC1D_E_ACTIVATION;
    if (a->width < 2 || a->width > 4) return VC1D_E_WIDTH;
    if (a->batch < 0 || a->dim < 0 || a->state_len < a->width - 1) return VC1D_E_SHAPE;
    if ((long long)a->batch * a->dim == 0) return VC1D_OK;
    if (a->x == nullptr || a->conv_state == nullptr || a->dy == nullptr || a->dx == nullptr || a->weight == nullptr)
        return VC1D_E_NULL;
    return (int)launch_update_bwd(*a, reinterpret_cast<cudaStream_t>(stream));
}

VC1D_API uint32_t vc1d_sizeof_update_bwd_args(void) { return (uint32_t)sizeof(vc1d_update_bwd_args); }

VC1D_API int vc1d_abi_version(void) { return VC1D_ABI_VERSION; }
VC1D_API uint32_t vc1d_sizeof_prefill_args(void) { return (uint32_t)sizeof(vc1d_prefill_args); }
VC1D_API uint32_t vc1d_sizeof_update_args(void) { return (uint32_t)sizeof(vc1d_update_args); }

VC1D_API const char* vc1d_status_string(int status) {
    switch (status) {
        case VC1D_OK: return "ok";
        case VC1D_E_NULL: return "VC1D_E_NULL: a required pointer is NULL";
        case VC1D_E_DTYPE: return "VC1D_E_DTYPE: unsupported element type";
        case VC1D_E_WIDTH: return "VC1D_E_WIDTH: width must be 2, 3 or 4";
        case VC1D_E_SHAPE: return "VC1D_E_SHAPE: invalid size";
        case VC1D_E_STRIDE: return "VC1D_E_STRIDE: layout not addressable by the requested kernel";
        case VC1D_E_STRUCT: return "VC1D_E_STRUCT: argument struct size mismatch";
        case VC1D_E_ACTIVATION: return "VC1D_E_ACTIVATION: unknown activation";
        case VC1D_E_ALIAS: return "VC1D_E_ALIAS: output overlaps an input";
        case VC1D_E_TOO_LARGE: return "VC1D_E_TOO_LARGE: size beyond the entry point's limit";
        default: break;
    }
    if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
    return "unknown vc1d status";
}

VC1D_API uint64_t vc1d_launch_count(void) { return vc1d::g_launches.load(std::memory_order_relaxed); }

VC1D_API const char* vc1d_last_kernel(void) { return vc1d::t_last_kernel; }

VC1D_API int vc1d_last_class_table(void) { return vc1d::t_class_table; }

VC1D_API unsigned int vc1d_tma_timeouts(void) { return vc1d::tma_timeouts(); }

VC1D_API int vc1d_set_pdl(int enabled) {
    const int before = vc1d::pdl_enabled() ? 1 : 0;
    vc1d::g_pdl_override.store(enabled < 0 ? -1 : (enabled != 0 ? 1 : 0), std::memory_order_relaxed);
    return before;
}

}  // extern "C"
