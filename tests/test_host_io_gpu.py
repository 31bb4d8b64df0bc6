"""HostPrefill: pinned host tensors in, pinned host tensors out, chunked over three streams.
Results must equal the device-resident operator bit for bit, with rows behind the last valid
position left out of the copy-in and with consecutive batches pipelined into each other."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

import viby_model_b200 as V  # noqa: E402
from viby_model_b200.host_io import HostPrefill  # noqa: E402

DEV = torch.device("cuda", 0)


def make(B, T, D, W, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, T, D, generator=g).to(dtype).pin_memory()
    w = torch.randn(D, W, generator=g).to(dtype).to(DEV)
    b = torch.randn(D, generator=g).to(dtype).to(DEV)
    lens = torch.randint(1, T + 1, (B,), generator=g)
    m = torch.arange(T)[None, :] < lens[:, None]
    m[0, :] = False       # a sequence with nothing valid
    m[1, T // 3] = False  # a hole inside a sequence
    if B > 2:
        m[2, :] = True
    return x, w, b, m.pin_memory()


def direct(x, w, b, m):
    xd = x.to(DEV)
    md = m.to(DEV) if m is not None else None
    return V.causal_conv1d_fn(xd.transpose(1, 2), w, b, activation="silu", attention_mask=md).transpose(1, 2)


@pytest.mark.parametrize("masked", [True, False])
@pytest.mark.parametrize("B,T,D,chunk", [(7, 300, 1152, 2), (5, 1024, 256, 4), (3, 64, 64, 8)])
def test_host_prefill_matches_device_operator(B, T, D, chunk, masked):
    dtype = torch.bfloat16
    x, w, b, m = make(B, T, D, 4, dtype, seed=B + T)
    pipe = HostPrefill(B, T, D, dtype, device=DEV, chunk_batch=chunk, masked=masked, mask_dtype=torch.bool)
    # poison the device input buffer: rows that are not sent must never be used
    pipe.x_dev.fill_(float("nan"))
    y_host = torch.empty_like(x).pin_memory()
    pipe.run(x, w, b, "silu", m if masked else None, y_host)
    torch.cuda.synchronize()
    ref = direct(x, w, b, m if masked else None)
    assert torch.equal(y_host.to(DEV), ref)
    if masked:
        lens = HostPrefill.valid_prefix_lengths(m)
        assert lens[0] == 0 and pipe.h2d_bytes == sum(lens) * D * 2 + B * T
    else:
        assert pipe.h2d_bytes == B * T * D * 2


def test_host_prefill_pipelines_consecutive_batches():
    B, T, D = 6, 512, 1152
    dtype = torch.bfloat16
    pipe = HostPrefill(B, T, D, dtype, device=DEV, chunk_batch=2, masked=True, mask_dtype=torch.bool)
    batches = [make(B, T, D, 4, dtype, seed=100 + i) for i in range(4)]
    w, b = batches[0][1], batches[0][2]
    outs = [torch.empty(B, T, D, dtype=dtype).pin_memory() for _ in batches]
    for (x, _, _, m), y in zip(batches, outs):
        pipe.run(x, w, b, "silu", m, y, join=False)
    pipe.join()
    torch.cuda.synchronize()
    for (x, _, _, m), y in zip(batches, outs):
        assert torch.equal(y.to(DEV), direct(x, w, b, m))


def test_host_prefill_sending_all_rows_gives_the_same_result():
    B, T, D = 4, 256, 512
    x, w, b, m = make(B, T, D, 4, torch.bfloat16, seed=9)
    outs = []
    for send_all in (False, True):
        pipe = HostPrefill(B, T, D, torch.bfloat16, device=DEV, chunk_batch=2, mask_dtype=torch.bool,
                           send_masked_rows=send_all)
        y = torch.empty_like(x).pin_memory()
        pipe.run(x, w, b, "silu", m, y)
        torch.cuda.synchronize()
        outs.append(y.clone())
        assert pipe.h2d_bytes == ((B * T * D * 2 + B * T) if send_all else
                                  (sum(HostPrefill.valid_prefix_lengths(m)) * D * 2 + B * T))
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("has_bias", [True, False])
@pytest.mark.parametrize("act", ["silu", None])
def test_host_prefill_filling_constant_rows_on_the_host_gives_the_same_bytes(act, has_bias):
    """Rows width-1 or more steps behind a sequence's last valid position are act(bias) in every
    sequence: with skip_constant_rows they are not copied back but written by the host, and y_host
    must still equal the full copy bit for bit (pipelined batches included)."""
    B, T, D, W = 7, 300, 1152, 4
    x, w, b, m = make(B, T, D, W, torch.bfloat16, seed=21)
    if not has_bias:
        b = None
    full = HostPrefill(B, T, D, torch.bfloat16, device=DEV, chunk_batch=2, mask_dtype=torch.bool)
    lean = HostPrefill(B, T, D, torch.bfloat16, device=DEV, chunk_batch=2, mask_dtype=torch.bool,
                       skip_constant_rows=True)
    y_full = torch.empty_like(x).pin_memory()
    y_lean = torch.full_like(x, float("nan")).pin_memory()
    full.run(x, w, b, act, m, y_full)
    for _ in range(3):
        lean.run(x, w, b, act, m, y_lean, join=False)
    lean.join()
    torch.cuda.synchronize()
    assert torch.equal(y_full.view(torch.int16), y_lean.view(torch.int16))
    lens = HostPrefill.valid_prefix_lengths(m)
    expect = sum(min(T, n + W - 1) for n in lens) * D * 2 + D * 2
    assert lean.d2h_bytes == expect and expect < full.d2h_bytes
