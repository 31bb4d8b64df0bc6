"""ctypes binding of libvc1d.so (declarations: include/vc1d.h).

The shared library is the product; there is no fallback.  Importing this module raises
ImportError when the library has not been built (``python viby_model_b200/build.py``).
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

# ---- constants mirrored from include/vc1d.h -------------------------------------------------
VC1D_ABI_VERSION = 1
UPDATE_MULTI_MAX = 80  # VC1D_UPDATE_MULTI_MAX

VC1D_F32, VC1D_BF16, VC1D_F16 = 0, 1, 2
VC1D_U8, VC1D_I32, VC1D_I64 = 8, 9, 10

VC1D_ACT_NONE, VC1D_ACT_SILU = 0, 1

VC1D_OK = 0
VC1D_E_NULL, VC1D_E_DTYPE, VC1D_E_WIDTH, VC1D_E_SHAPE = -1, -2, -3, -4
VC1D_E_STRIDE, VC1D_E_STRUCT, VC1D_E_ACTIVATION, VC1D_E_ALIAS, VC1D_E_TOO_LARGE = -5, -6, -7, -8, -9

KERNEL_AUTO, KERNEL_CHANNEL_LAST, KERNEL_TIME_MAJOR, KERNEL_GENERIC, KERNEL_TMA = 0, 1, 2, 3, 4
KERNEL_BY_NAME = {
    None: KERNEL_AUTO,
    "auto": KERNEL_AUTO,
    "channel_last": KERNEL_CHANNEL_LAST,
    "time_major": KERNEL_TIME_MAJOR,
    "generic": KERNEL_GENERIC,
    "tma": KERNEL_TMA,
}


class PrefillArgs(C.Structure):
    """struct vc1d_prefill_args"""

    _fields_ = [
        ("struct_size", C.c_uint32),
        ("dtype", C.c_int32),
        ("wdtype", C.c_int32),
        ("activation", C.c_int32),
        ("batch", C.c_int32),
        ("dim", C.c_int32),
        ("seqlen", C.c_int32),
        ("width", C.c_int32),
        ("x", C.c_void_p),
        ("y", C.c_void_p),
        ("weight", C.c_void_p),
        ("bias", C.c_void_p),
        ("x_stride_b", C.c_int64),
        ("x_stride_d", C.c_int64),
        ("x_stride_t", C.c_int64),
        ("y_stride_b", C.c_int64),
        ("y_stride_d", C.c_int64),
        ("y_stride_t", C.c_int64),
        ("w_stride_d", C.c_int64),
        ("w_stride_w", C.c_int64),
        ("mask", C.c_void_p),
        ("mask_dtype", C.c_int32),
        ("skip_masked_loads", C.c_int32),
        ("mask_stride_b", C.c_int64),
        ("mask_stride_t", C.c_int64),
        ("residual", C.c_void_p),
        ("r_stride_b", C.c_int64),
        ("r_stride_d", C.c_int64),
        ("r_stride_t", C.c_int64),
        ("initial_state", C.c_void_p),
        ("init_len", C.c_int32),
        ("state_len", C.c_int32),
        ("final_state", C.c_void_p),
        ("kernel", C.c_int32),
        ("rows_per_thread", C.c_int32),
        ("block_threads", C.c_int32),
        ("unroll", C.c_int32),
        ("tma_stages", C.c_int32),
        ("tma_ctas_per_sm", C.c_int32),
        ("tma_slab_bytes", C.c_int32),
        ("tma_rows_per_thread", C.c_int32),
        ("scratch", C.c_void_p),
        ("scratch_bytes", C.c_int64),
        ("seq_idx", C.c_void_p),
        ("seq_stride_b", C.c_int64),
        ("seq_stride_t", C.c_int64),
        ("tma_claim_chunk", C.c_int32),
        ("tma_empty_store", C.c_int32),
        ("tma_classify", C.c_int32),
        ("tma_pdl", C.c_int32),
        ("tma_static_first", C.c_int32),
        ("tma_test_expire", C.c_int32),
        ("tma_kept_tables", C.c_int32),
        ("tma_reserved", C.c_int32),
    ]


class PrefillBwdArgs(C.Structure):
    """struct vc1d_prefill_bwd_args"""

    _fields_ = [
        ("struct_size", C.c_uint32),
        ("dtype", C.c_int32),
        ("wdtype", C.c_int32),
        ("activation", C.c_int32),
        ("batch", C.c_int32),
        ("dim", C.c_int32),
        ("seqlen", C.c_int32),
        ("width", C.c_int32),
        ("x", C.c_void_p),
        ("dy", C.c_void_p),
        ("dx", C.c_void_p),
        ("weight", C.c_void_p),
        ("bias", C.c_void_p),
        ("x_stride_b", C.c_int64),
        ("x_stride_d", C.c_int64),
        ("x_stride_t", C.c_int64),
        ("dy_stride_b", C.c_int64),
        ("dy_stride_d", C.c_int64),
        ("dy_stride_t", C.c_int64),
        ("dx_stride_b", C.c_int64),
        ("dx_stride_d", C.c_int64),
        ("dx_stride_t", C.c_int64),
        ("w_stride_d", C.c_int64),
        ("w_stride_w", C.c_int64),
        ("mask", C.c_void_p),
        ("mask_dtype", C.c_int32),
        ("residual", C.c_int32),
        ("mask_stride_b", C.c_int64),
        ("mask_stride_t", C.c_int64),
        ("dweight", C.c_void_p),
        ("dbias", C.c_void_p),
        ("kernel", C.c_int32),
        ("tma_stages", C.c_int32),
        ("tma_ctas_per_sm", C.c_int32),
        ("tma_variant", C.c_int32),
        ("scratch", C.c_void_p),
        ("scratch_bytes", C.c_int64),
        ("initial_state", C.c_void_p),
        ("dinitial_state", C.c_void_p),
        ("init_len", C.c_int32),
        ("zero_grads", C.c_int32),
        ("seq_idx", C.c_void_p),
        ("seq_stride_b", C.c_int64),
        ("seq_stride_t", C.c_int64),
    ]


class UpdateArgs(C.Structure):
    """struct vc1d_update_args"""

    _fields_ = [
        ("struct_size", C.c_uint32),
        ("dtype", C.c_int32),
        ("wdtype", C.c_int32),
        ("activation", C.c_int32),
        ("batch", C.c_int32),
        ("dim", C.c_int32),
        ("width", C.c_int32),
        ("state_len", C.c_int32),
        ("x", C.c_void_p),
        ("y", C.c_void_p),
        ("conv_state", C.c_void_p),
        ("weight", C.c_void_p),
        ("bias", C.c_void_p),
        ("x_stride_b", C.c_int64),
        ("x_stride_d", C.c_int64),
        ("y_stride_b", C.c_int64),
        ("y_stride_d", C.c_int64),
        ("s_stride_b", C.c_int64),
        ("s_stride_d", C.c_int64),
        ("s_stride_l", C.c_int64),
        ("w_stride_d", C.c_int64),
        ("w_stride_w", C.c_int64),
        ("cache_seqlens", C.c_void_p),
        ("residual", C.c_int32),
        ("kernel", C.c_int32),
        ("block_threads", C.c_int32),
        ("reserved", C.c_int32),
    ]


class UpdateBwdArgs(C.Structure):
    """struct vc1d_update_bwd_args"""

    _fields_ = [
        ("struct_size", C.c_uint32),
        ("dtype", C.c_int32),
        ("wdtype", C.c_int32),
        ("activation", C.c_int32),
        ("batch", C.c_int32),
        ("dim", C.c_int32),
        ("width", C.c_int32),
        ("state_len", C.c_int32),
        ("x", C.c_void_p),
        ("conv_state", C.c_void_p),
        ("dy", C.c_void_p),
        ("dx", C.c_void_p),
        ("dstate", C.c_void_p),
        ("weight", C.c_void_p),
        ("bias", C.c_void_p),
        ("x_stride_b", C.c_int64),
        ("x_stride_d", C.c_int64),
        ("dy_stride_b", C.c_int64),
        ("dy_stride_d", C.c_int64),
        ("dx_stride_b", C.c_int64),
        ("dx_stride_d", C.c_int64),
        ("s_stride_b", C.c_int64),
        ("s_stride_d", C.c_int64),
        ("s_stride_l", C.c_int64),
        ("w_stride_d", C.c_int64),
        ("w_stride_w", C.c_int64),
        ("cache_seqlens", C.c_void_p),
        ("residual", C.c_int32),
        ("reserved", C.c_int32),
        ("dweight", C.c_void_p),
        ("dbias", C.c_void_p),
    ]


# every symbol include/vc1d.h declares: name -> (restype, argtypes)
EXPORTS = {
    "vc1d_prefill": (C.c_int, [C.POINTER(PrefillArgs), C.c_void_p]),
    "vc1d_prefill_noalloc": (C.c_int, [C.POINTER(PrefillArgs), C.c_void_p]),
    "vc1d_prefill_bwd": (C.c_int, [C.POINTER(PrefillBwdArgs), C.c_void_p]),
    "vc1d_sizeof_prefill_bwd_args": (C.c_uint32, []),
    "vc1d_update": (C.c_int, [C.POINTER(UpdateArgs), C.c_void_p]),
    "vc1d_update_multi": (C.c_int, [C.POINTER(UpdateArgs), C.c_int32, C.c_void_p]),
    "vc1d_update_bwd": (C.c_int, [C.POINTER(UpdateBwdArgs), C.c_void_p]),
    "vc1d_sizeof_update_bwd_args": (C.c_uint32, []),
    "vc1d_abi_version": (C.c_int, []),
    "vc1d_sizeof_prefill_args": (C.c_uint32, []),
    "vc1d_sizeof_update_args": (C.c_uint32, []),
    "vc1d_status_string": (C.c_char_p, [C.c_int]),
    "vc1d_launch_count": (C.c_uint64, []),
    "vc1d_last_kernel": (C.c_char_p, []),
    "vc1d_last_class_table": (C.c_int, []),
    "vc1d_tma_timeouts": (C.c_uint, []),
    "vc1d_set_pdl": (C.c_int, [C.c_int]),
}


def library_path() -> Path:
    env = os.environ.get("VC1D_LIBRARY")
    if env:
        return Path(env)
    return Path(__file__).resolve().parent / "libvc1d.so"


def _load() -> C.CDLL:
    path = library_path()
    if not path.exists():
        raise ImportError(
            f"{path} not found: the CUDA library has not been built. "
            "Run `python viby_model_b200/build.py` (needs nvcc 12.9, targets sm_100a). "
            "There is no CPU or PyTorch fallback."
        )
    lib = C.CDLL(str(path))
    for name, (restype, argtypes) in EXPORTS.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:  # pragma: no cover - a stale library
            raise ImportError(f"{path} does not export {name}; rebuild it") from e
        fn.restype = restype
        fn.argtypes = argtypes
    if lib.vc1d_abi_version() != VC1D_ABI_VERSION:
        raise ImportError(f"{path}: ABI version {lib.vc1d_abi_version()} != binding {VC1D_ABI_VERSION}")
    if (
        lib.vc1d_sizeof_prefill_args() != C.sizeof(PrefillArgs)
        or lib.vc1d_sizeof_update_args() != C.sizeof(UpdateArgs)
        or lib.vc1d_sizeof_prefill_bwd_args() != C.sizeof(PrefillBwdArgs)
        or lib.vc1d_sizeof_update_bwd_args() != C.sizeof(UpdateBwdArgs)
    ):
        raise ImportError(f"{path}: argument struct layout differs from the binding; rebuild it")
    return lib


lib = _load()


def status_string(status: int) -> str:
    return lib.vc1d_status_string(int(status)).decode()


def launch_count() -> int:
    return int(lib.vc1d_launch_count())


def last_kernel() -> str:
    return lib.vc1d_last_kernel().decode()


def set_pdl(enabled) -> bool:
    """Programmatic dependent launch between the library's kernels: True / False, or None to follow the
    environment (VC1D_NO_PDL).  Returns the previous setting."""
    return bool(lib.vc1d_set_pdl(-1 if enabled is None else int(bool(enabled))))


def tma_timeouts() -> int:
    """Expired mbarrier waits in the TMA kernel so far (synchronising read; 0 when healthy)."""
    return int(lib.vc1d_tma_timeouts())


_VALUE_ERRORS = {
    VC1D_E_NULL,
    VC1D_E_DTYPE,
    VC1D_E_WIDTH,
    VC1D_E_SHAPE,
    VC1D_E_STRIDE,
    VC1D_E_ACTIVATION,
    VC1D_E_ALIAS,
    VC1D_E_TOO_LARGE,
}


def check(status: int, what: str) -> None:
    """Raise for a non-zero launcher status: ValueError for argument errors, RuntimeError for CUDA errors."""
    if status == VC1D_OK:
        return
    msg = f"{what}: {status_string(status)} (status {status})"
    if status in _VALUE_ERRORS:
        raise ValueError(msg)
    raise RuntimeError(msg)
