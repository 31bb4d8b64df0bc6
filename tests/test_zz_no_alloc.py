"""vc1d_prefill_noalloc: the prefill entry point whose scheduler scratch is a fixed array inside
the library, called through the C ABI and compared with vc1d_prefill.  The file name sorts last so
that it also runs after every other GPU test has used the library in the same process."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from viby_model_b200 import _cabi  # noqa: E402

DEV = torch.device("cuda", 0)
DTYPES = {torch.float32: _cabi.VC1D_F32, torch.bfloat16: _cabi.VC1D_BF16, torch.float16: _cabi.VC1D_F16}


def prefill_args(x, y, w, b, mask):
    """x, y: [B, T, D] contiguous device tensors (the channel-last layout of the operator)."""
    B, T, D = x.shape
    a = _cabi.PrefillArgs()
    a.struct_size = C.sizeof(_cabi.PrefillArgs)
    a.dtype = a.wdtype = DTYPES[x.dtype]
    a.activation = _cabi.VC1D_ACT_SILU
    a.batch, a.dim, a.seqlen, a.width = B, D, T, w.shape[1]
    a.x, a.y, a.weight, a.bias = x.data_ptr(), y.data_ptr(), w.data_ptr(), b.data_ptr()
    a.x_stride_b, a.x_stride_d, a.x_stride_t = T * D, 1, D
    a.y_stride_b, a.y_stride_d, a.y_stride_t = T * D, 1, D
    a.w_stride_d, a.w_stride_w = w.shape[1], 1
    if mask is not None:
        a.mask = mask.data_ptr()
        a.mask_dtype = _cabi.VC1D_U8
        a.mask_stride_b, a.mask_stride_t = T, 1
        a.skip_masked_loads = 1
    return a


def make(B, T, D, W, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, T, D, generator=g).to(dtype).to(DEV)
    w = torch.randn(D, W, generator=g).to(dtype).to(DEV)
    b = torch.randn(D, generator=g).to(dtype).to(DEV)
    lens = torch.randint(T // 3, T + 1, (B,), generator=g)
    mask = (torch.arange(T)[None, :] < lens[:, None]).to(torch.uint8).to(DEV)
    return x, w, b, mask


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("masked", [True, False])
def test_noalloc_matches_prefill_twice_in_a_row(dtype, masked):
    from oracle import canon_oracle as O
    from parity import assert_close_to_oracle

    stream = torch.cuda.current_stream(DEV).cuda_stream
    # Shapes that give every CTA of the kernel several tiles, so that it claims them from the counters
    # in the library's array (and, with a mask, reads the class bytes a pre-pass kernel wrote there):
    # different slab counts share the one array.  The last shape is too small for that and runs with
    # static assignment, the array untouched.
    shapes = [(32, 1024, 3456, 4), (16, 2048, 1152, 3), (6, 777, 1152, 4)]
    for rep in range(2):
        for i, (B, T, D, W) in enumerate(shapes):
            x, w, b, mask = make(B, T, D, W, dtype, seed=17 * rep + i)
            m = mask if masked else None
            y_ref = torch.full_like(x, float("nan"))
            y_new = torch.full_like(x, float("nan"))
            a_ref = prefill_args(x, y_ref, w, b, m)
            a_ref.kernel = _cabi.KERNEL_TMA
            assert _cabi.lib.vc1d_prefill(C.byref(a_ref), stream) == 0
            a_new = prefill_args(x, y_new, w, b, m)
            torch.cuda.synchronize()
            free_before, _ = torch.cuda.mem_get_info(DEV)
            # two calls in a row: the second finds the array as the first left it
            launches = _cabi.launch_count()
            assert _cabi.lib.vc1d_prefill_noalloc(C.byref(a_new), stream) == 0
            if i < 2:
                # the tile-classification pre-pass ran before the main kernel: its class bytes, and the claim
                # counters beside them, live in the library's array
                assert _cabi.launch_count() - launches == (2 if masked else 1)
            y_first = y_new.clone()
            y_new.fill_(float("nan"))
            assert _cabi.lib.vc1d_prefill_noalloc(C.byref(a_new), stream) == 0
            torch.cuda.synchronize()
            assert torch.equal(y_first, y_ref)
            assert torch.equal(y_new, y_ref)
            assert not torch.isnan(y_ref).any()
            if rep == 0:
                # and against the CPU oracle directly, on the first two sequences
                ref = O.causal_conv1d_ref(x[:2].cpu().transpose(1, 2), w.cpu(), b.cpu(), "silu",
                                          attention_mask=None if m is None else m[:2].cpu())
                assert_close_to_oracle(y_new[:2].transpose(1, 2), ref, f"noalloc {B}x{T}x{D}")
            if rep == 1:
                # set-up happened in the first round; y_first's clone is the only allocation since
                free_after, _ = torch.cuda.mem_get_info(DEV)
                assert free_before - free_after <= y_first.numel() * y_first.element_size() + (2 << 20)
    assert _cabi.tma_timeouts() == 0


def test_noalloc_rejects_sizes_beyond_its_array():
    stream = torch.cuda.current_stream(DEV).cuda_stream
    x, w, b, _ = make(1, 64, 64, 4, torch.bfloat16, seed=1)
    y = torch.empty_like(x)
    a = prefill_args(x, y, w, b, None)
    # claim a problem with more tiles than the array has class bytes; nothing may be launched
    a.batch, a.seqlen = 4096, 32 * 16
    before = _cabi.launch_count()
    st = _cabi.lib.vc1d_prefill_noalloc(C.byref(a), stream)
    assert st == _cabi.VC1D_E_TOO_LARGE
    assert "limit" in _cabi.status_string(st)
    assert _cabi.launch_count() == before
    # a layout the TMA-staged kernel cannot take is refused like vc1d_prefill refuses it
    a = prefill_args(x, y, w, b, None)
    a.x_stride_d, a.x_stride_t = 64, 1
    assert _cabi.lib.vc1d_prefill_noalloc(C.byref(a), stream) == _cabi.VC1D_E_STRIDE
    a = prefill_args(x, y, w, b, None)
    a.struct_size = 8
    assert _cabi.lib.vc1d_prefill_noalloc(C.byref(a), stream) == _cabi.VC1D_E_STRUCT
