"""The [B,T,D] operators of causal-conv1d-mps on the CUDA kernels, with the reference's own test
recipes (causal-conv1d-mps/test.py:149-197 for short_conv_fused, :200-252 for edge and error
cases) plus the forward of short_conv_update, which the reference only grad-checks."""
import pytest
import torch

import viby_model_b200 as V
from oracle import canon_oracle as O
from parity import assert_close_to_oracle

DEV = "cuda"


@pytest.mark.gpu
@pytest.mark.parametrize("itype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("silu_activation", [False, True])
@pytest.mark.parametrize("has_bias", [False, True])
@pytest.mark.parametrize("seqlen", [8, 16, 32, 64])
@pytest.mark.parametrize("dim", [64, 128])
def test_short_conv_fused(dim, seqlen, has_bias, silu_activation, itype):
    torch.random.manual_seed(42)
    batch = 2
    x = torch.randn(batch, seqlen, dim).to(itype)
    weight = torch.randn(dim, 4)
    bias = torch.randn(dim) if has_bias else None
    mask = torch.ones(batch, seqlen)
    for b in range(batch):
        mask[b, int(torch.randint(seqlen // 2, seqlen, (1,))):] = 0
    out = V.short_conv_fused(x.to(DEV), weight.to(DEV), bias.to(DEV) if has_bias else None, mask.to(DEV),
                             activation=silu_activation, residual=True)
    assert out.shape == x.shape and out.is_contiguous()
    conv = O.causal_conv1d_ref(x.transpose(1, 2), weight, bias, "silu" if silu_activation else None,
                               attention_mask=mask)
    # the reference's own tolerance for this test (test.py:162-167)
    rtol, atol = (3e-4, 1e-3) if itype == torch.float32 else (5e-3, 2e-2)
    ref = x + conv.transpose(1, 2)
    assert torch.allclose(out.cpu().float(), ref.float(), rtol=rtol, atol=atol)
    no_res = V.short_conv_fused(x.to(DEV), weight.to(DEV), bias.to(DEV) if has_bias else None, mask.to(DEV),
                                activation=silu_activation, residual=False)
    assert_close_to_oracle(no_res.transpose(1, 2), conv, "short_conv_fused without residual")


@pytest.mark.gpu
def test_causal_conv1d_fwd_edge_cases_and_dtype():
    x = torch.randn(1, 1, 1, device=DEV)
    assert V.causal_conv1d_fwd(x, torch.randn(1, 4, device=DEV), torch.randn(1, device=DEV), False).shape == (1, 1, 1)
    x = torch.randn(2, 3, 5, device=DEV)
    assert V.causal_conv1d_fwd(x, torch.randn(3, 4, device=DEV), None, False).shape == (2, 3, 5)
    x = torch.randn(2, 64, 32, device=DEV)
    w = torch.randn(64, 4, device=DEV)
    b = torch.randn(64, device=DEV)
    y = V.causal_conv1d_fwd(x, w, b, True)
    assert y.dtype == torch.float32 and y.shape == (2, 64, 32)
    assert_close_to_oracle(y, O.causal_conv1d_ref(x.cpu(), w.cpu(), b.cpu(), "silu"))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_short_conv_update_forward(dtype):
    B, D, S = 3, 64, 8
    g = torch.Generator().manual_seed(3)
    w = (torch.rand(D, 4, generator=g) - 0.5).to(dtype)
    b = (torch.rand(D, generator=g) - 0.5).to(dtype)
    state = torch.randn(B, D, S, generator=g).to(dtype)
    seqlens = torch.tensor([5, 0, 11], dtype=torch.int32)
    sd = state.to(DEV)
    for step in range(12):
        xt = torch.randn(B, D, generator=g).to(dtype)
        y = V.short_conv_update(xt.to(DEV), sd, w.to(DEV), b.to(DEV), seqlens.to(DEV), activation=True, residual=True)
        ref = O.causal_conv1d_update_ref(xt, state, w, b, "silu", cache_seqlens=seqlens, residual=True)
        assert_close_to_oracle(y, ref, f"step {step}")
        assert torch.equal(sd.cpu(), state)
        seqlens = seqlens + 1
    # default cache_seqlens is arange(batch), as in the reference
    xt = torch.randn(B, D, generator=g).to(dtype)
    y = V.short_conv_update(xt.to(DEV), sd, w.to(DEV), None, None, activation=False, residual=False)
    ref = O.causal_conv1d_update_ref(xt, state, w, None, None, cache_seqlens=torch.arange(B, dtype=torch.int32))
    assert_close_to_oracle(y, ref)
    assert torch.equal(sd.cpu(), state)


def test_error_messages_follow_the_reference():
    # test.py:226-236 -- these checks come before any device check, so they run without a GPU
    with pytest.raises(ValueError, match="does not match"):
        V.causal_conv1d_fwd(torch.randn(2, 4, 8), torch.randn(5, 4), None, False)
    with pytest.raises(ValueError, match="Expected 3D input tensor"):
        V.causal_conv1d_fwd(torch.randn(4, 8), torch.randn(4, 4), None, False)
    with pytest.raises(ValueError, match="Expected 3D input tensor"):
        V.short_conv_fused(torch.randn(4, 8), torch.randn(8, 4))
    with pytest.raises(ValueError, match="Attention mask shape"):
        V.short_conv_fused(torch.randn(2, 4, 8), torch.randn(8, 4), None, torch.ones(2, 5))
    with pytest.raises(ValueError, match="doesn't match conv_state"):
        V.short_conv_update(torch.randn(2, 8), torch.randn(3, 8, 8), torch.randn(8, 4))
    with pytest.raises(ValueError, match="must be on CUDA device"):
        V.short_conv_fused(torch.randn(2, 4, 8), torch.randn(8, 4))
