"""The C-ABI shared library: loads, exports every symbol include/vc1d.h declares, agrees on the
struct layouts and rejects bad arguments before touching CUDA.  No compute; runs without a GPU."""
import ctypes as C
import re
from pathlib import Path

import pytest
import torch

from viby_model_b200 import _cabi

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "vc1d.h").read_text()


def declared_symbols():
    return re.findall(r"VC1D_API\s+[\w\s\*]+?\b(vc1d_\w+)\s*\(", HEADER)


def test_header_symbols_are_exported_and_bound():
    names = declared_symbols()
    assert len(names) >= 8
    raw = C.CDLL(str(_cabi.library_path()))
    for n in names:
        assert hasattr(raw, n), f"{n} declared in include/vc1d.h but not exported"
        assert n in _cabi.EXPORTS, f"{n} has no ctypes binding"
    assert set(_cabi.EXPORTS) == set(names)


def test_abi_version_and_struct_sizes():
    assert _cabi.lib.vc1d_abi_version() == int(re.search(r"#define VC1D_ABI_VERSION (\d+)", HEADER).group(1))
    assert _cabi.lib.vc1d_sizeof_prefill_args() == C.sizeof(_cabi.PrefillArgs)
    assert _cabi.lib.vc1d_sizeof_update_args() == C.sizeof(_cabi.UpdateArgs)


def test_enum_values_match_header():
    for name in ("VC1D_F32", "VC1D_BF16", "VC1D_F16", "VC1D_U8", "VC1D_I32", "VC1D_I64", "VC1D_E_NULL",
                 "VC1D_E_DTYPE", "VC1D_E_WIDTH", "VC1D_E_SHAPE", "VC1D_E_STRIDE", "VC1D_E_STRUCT",
                 "VC1D_E_ACTIVATION", "VC1D_E_ALIAS", "VC1D_E_TOO_LARGE"):
        m = re.search(rf"\b{name}\s*=\s*(-?\d+)", HEADER)
        assert m, name
        assert getattr(_cabi, name) == int(m.group(1)), name


def _prefill_args(**kw):
    a = _cabi.PrefillArgs()
    a.struct_size = C.sizeof(_cabi.PrefillArgs)
    a.dtype = _cabi.VC1D_BF16
    a.wdtype = _cabi.VC1D_BF16
    a.batch, a.dim, a.seqlen, a.width = 1, 8, 8, 4
    for k, v in kw.items():
        setattr(a, k, v)
    return a


def _update_args(**kw):
    a = _cabi.UpdateArgs()
    a.struct_size = C.sizeof(_cabi.UpdateArgs)
    a.dtype = _cabi.VC1D_BF16
    a.wdtype = _cabi.VC1D_BF16
    a.batch, a.dim, a.width, a.state_len = 1, 8, 4, 3
    for k, v in kw.items():
        setattr(a, k, v)
    return a


@pytest.mark.parametrize(
    "kw,code",
    [
        (dict(struct_size=4), _cabi.VC1D_E_STRUCT),
        (dict(dtype=7), _cabi.VC1D_E_DTYPE),
        (dict(wdtype=_cabi.VC1D_F16), _cabi.VC1D_E_DTYPE),
        (dict(activation=5), _cabi.VC1D_E_ACTIVATION),
        (dict(width=5), _cabi.VC1D_E_WIDTH),
        (dict(width=1), _cabi.VC1D_E_WIDTH),
        (dict(batch=-1), _cabi.VC1D_E_SHAPE),
        (dict(kernel=9), _cabi.VC1D_E_SHAPE),
        (dict(), _cabi.VC1D_E_NULL),  # x, y, weight are NULL
        (dict(x=4096, y=4096, weight=64, x_stride_b=64, x_stride_d=1, x_stride_t=8, y_stride_b=64, y_stride_d=1,
              y_stride_t=8), _cabi.VC1D_E_ALIAS),
    ],
)
def test_prefill_rejects_bad_arguments_without_launching(kw, code):
    before = _cabi.launch_count()
    assert _cabi.lib.vc1d_prefill(C.byref(_prefill_args(**kw)), None) == code
    assert _cabi.launch_count() == before


@pytest.mark.parametrize(
    "kw,code",
    [
        (dict(struct_size=4), _cabi.VC1D_E_STRUCT),
        (dict(dtype=3), _cabi.VC1D_E_DTYPE),
        (dict(width=7), _cabi.VC1D_E_WIDTH),
        (dict(state_len=2), _cabi.VC1D_E_SHAPE),  # shorter than width-1
        (dict(kernel=_cabi.KERNEL_TMA), _cabi.VC1D_E_SHAPE),
        (dict(), _cabi.VC1D_E_NULL),
    ],
)
def test_update_rejects_bad_arguments_without_launching(kw, code):
    before = _cabi.launch_count()
    assert _cabi.lib.vc1d_update(C.byref(_update_args(**kw)), None) == code
    assert _cabi.launch_count() == before


def test_null_struct_and_empty_inputs():
    assert _cabi.lib.vc1d_prefill(None, None) == _cabi.VC1D_E_NULL
    assert _cabi.lib.vc1d_update(None, None) == _cabi.VC1D_E_NULL
    # empty tensors are a successful no-op: nothing is dereferenced or launched
    assert _cabi.lib.vc1d_prefill(C.byref(_prefill_args(seqlen=0)), None) == _cabi.VC1D_OK
    assert _cabi.lib.vc1d_prefill(C.byref(_prefill_args(batch=0)), None) == _cabi.VC1D_OK
    assert _cabi.lib.vc1d_update(C.byref(_update_args(batch=0)), None) == _cabi.VC1D_OK


def test_status_strings():
    assert _cabi.status_string(0) == "ok"
    for code in range(-9, 0):
        assert _cabi.status_string(code).startswith("VC1D_E_")
    assert "unknown" in _cabi.status_string(-100)
    with pytest.raises(ValueError, match="VC1D_E_WIDTH"):
        _cabi.check(_cabi.VC1D_E_WIDTH, "x")
    with pytest.raises(RuntimeError):
        _cabi.check(1, "x")  # cudaErrorInvalidValue


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    monkeypatch.setenv("VC1D_LIBRARY", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        _cabi._load()


def test_header_is_plain_c(tmp_path):
    """include/vc1d.h is the boundary for C, cgo, JNI or FFI callers: it must compile as C99 on its own,
    and the struct sizes a C compiler computes must be the ones the library was built with."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    src = tmp_path / "probe.c"
    src.write_text(
        '#include <stdio.h>\n#include "vc1d.h"\n'
        "int main(void) {\n"
        "  vc1d_prefill_args a = {0}; vc1d_update_args u = {0}; vc1d_prefill_bwd_args g = {0}; vc1d_update_bwd_args h = {0};\n"
        "  a.struct_size = sizeof a; u.struct_size = sizeof u; g.struct_size = sizeof g; h.struct_size = sizeof h;\n"
        '  printf("%u %u %u %u %d\\n", a.struct_size, u.struct_size, g.struct_size, h.struct_size, VC1D_NOALLOC_MAX_TILES);\n'
        "  return 0;\n}\n"
    )
    exe = tmp_path / "probe"
    subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-pedantic", "-I", str(ROOT / "include"), str(src), "-o", str(exe)],
                   check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    sizes = [int(v) for v in out[:4]]
    assert sizes == [_cabi.lib.vc1d_sizeof_prefill_args(), _cabi.lib.vc1d_sizeof_update_args(),
                     _cabi.lib.vc1d_sizeof_prefill_bwd_args(), _cabi.lib.vc1d_sizeof_update_bwd_args()]
    assert int(out[4]) == 61440


def test_update_multi_rejects_bad_tables_without_launching():
    """vc1d_update_multi validates every problem of its table like vc1d_update, wants one I/O dtype and at
    most VC1D_UPDATE_MULTI_MAX problems; empty tables and empty problems are a successful no-op."""
    limit = int(re.search(r"#define VC1D_UPDATE_MULTI_MAX (\d+)", HEADER).group(1))
    assert limit == _cabi.UPDATE_MULTI_MAX
    before = _cabi.launch_count()
    table = (_cabi.UpdateArgs * 3)()
    for i in range(3):
        table[i] = _update_args(batch=0)  # nothing to do
    assert _cabi.lib.vc1d_update_multi(table, 3, None) == _cabi.VC1D_OK
    assert _cabi.lib.vc1d_update_multi(None, 0, None) == _cabi.VC1D_OK
    assert _cabi.lib.vc1d_update_multi(None, 2, None) == _cabi.VC1D_E_NULL
    assert _cabi.lib.vc1d_update_multi(table, limit + 1, None) == _cabi.VC1D_E_SHAPE
    assert _cabi.lib.vc1d_update_multi(table, -1, None) == _cabi.VC1D_E_SHAPE
    table[1] = _update_args(width=7)
    assert _cabi.lib.vc1d_update_multi(table, 3, None) == _cabi.VC1D_E_WIDTH
    table[1] = _update_args()  # pointers are NULL
    assert _cabi.lib.vc1d_update_multi(table, 3, None) == _cabi.VC1D_E_NULL
    # two problems that look valid (the addresses are never dereferenced: the table is refused first)
    fake = dict(x=1 << 20, y=2 << 20, conv_state=3 << 20, weight=4 << 20, x_stride_b=8, x_stride_d=1, y_stride_b=8,
                y_stride_d=1, s_stride_b=24, s_stride_d=3, s_stride_l=1, w_stride_d=4, w_stride_w=1)
    table[0] = _update_args(**fake)
    table[1] = _update_args(dtype=_cabi.VC1D_F32, wdtype=_cabi.VC1D_F32, **fake)
    assert _cabi.lib.vc1d_update_multi(table, 2, None) == _cabi.VC1D_E_DTYPE
    assert _cabi.launch_count() == before
