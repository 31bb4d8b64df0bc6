"""The backward oracle against gradients of the reference's own CanonLayer (torch.autograd through
its PyTorch branch) and against torch.autograd through the forward oracle.  CPU only."""
import pytest
import torch

from conftest import GOLDEN_BWD_CASES
from oracle import canon_oracle as O

IDS = [repr(c) for c in GOLDEN_BWD_CASES]


def _inputs(c):
    b = c.get("bias") if c.has("bias") else None
    m = c.get("mask") if c.has("mask") else None
    return c.get("x"), c.get("weight"), b, m, c.get("dy")


@pytest.mark.parametrize("c", GOLDEN_BWD_CASES, ids=IDS)
def test_backward_oracle_matches_reference_gradients(c):
    x, w, b, m, dy = _inputs(c)
    # the reference's branch computes in the model dtype, transposed: the oracle gets [B,D,T] views
    dx, dw, db = O.causal_conv1d_bwd_ref(x.transpose(1, 2), w, b, dy.transpose(1, 2), c.activation,
                                         attention_mask=m, residual_masked=True)
    gdx, gdw = c.get("dx").float(), c.get("dweight").float()
    if c.dtype == torch.float32:
        tol = dict(rtol=2e-5, atol=2e-5)
    else:
        # the reference differentiates bf16 ops (every intermediate rounded to 8 bits); the oracle
        # rounds once, so agreement is to a few bf16 steps of the largest term
        tol = dict(rtol=4e-2, atol=4e-2 * float(gdx.abs().max()))
    assert torch.allclose(dx.transpose(1, 2).float(), gdx, **tol)
    wtol = tol if c.dtype == torch.float32 else dict(rtol=4e-2, atol=4e-2 * float(gdw.abs().max()) + 1e-3)
    assert torch.allclose(dw.float(), gdw, **wtol)
    if b is not None:
        gdb = c.get("dbias").float()
        btol = tol if c.dtype == torch.float32 else dict(rtol=4e-2, atol=4e-2 * float(gdb.abs().max()) + 1e-3)
        assert torch.allclose(db.float(), gdb, **btol)


@pytest.mark.parametrize("W", [2, 3, 4])
@pytest.mark.parametrize("act", [None, "silu"])
@pytest.mark.parametrize("masked", [False, True])
@pytest.mark.parametrize("residual", [False, True])
def test_backward_oracle_matches_autograd_of_forward_oracle(W, act, masked, residual):
    g = torch.Generator().manual_seed(10 * W + masked)
    B, D, T = 3, 10, 13
    x = torch.randn(B, D, T, generator=g, dtype=torch.float64).requires_grad_(True)
    w = torch.randn(D, W, generator=g, dtype=torch.float64).requires_grad_(True)
    b = torch.randn(D, generator=g, dtype=torch.float64).requires_grad_(True)
    dy = torch.randn(B, D, T, generator=g, dtype=torch.float64)
    m = (torch.rand(B, T, generator=g) > 0.3).to(torch.float64) if masked else None
    xm = x * m.unsqueeze(1) if masked else x
    y = torch.nn.functional.conv1d(torch.nn.functional.pad(xm, (W - 1, 0)), w.unsqueeze(1), b, groups=D)
    if act:
        y = torch.nn.functional.silu(y)
    if residual:
        y = y + x
    (y * dy).sum().backward()
    dx, dw, db = O.causal_conv1d_bwd_ref(x.detach(), w.detach(), b.detach(), dy, act, attention_mask=m, residual=residual)
    assert torch.allclose(dx, x.grad, rtol=1e-10, atol=1e-10)
    assert torch.allclose(dw, w.grad, rtol=1e-10, atol=1e-10)
    assert torch.allclose(db, b.grad, rtol=1e-10, atol=1e-10)


@pytest.mark.parametrize("L", [3, 4, 8])
@pytest.mark.parametrize("act", [None, "silu"])
def test_update_backward_oracle_matches_autograd(L, act):
    g = torch.Generator().manual_seed(L)
    B, D, W = 3, 6, 4
    x = torch.randn(B, D, generator=g, dtype=torch.float64).requires_grad_(True)
    st = torch.randn(B, D, L, generator=g, dtype=torch.float64).requires_grad_(True)
    w = torch.randn(D, W, generator=g, dtype=torch.float64).requires_grad_(True)
    b = torch.randn(D, generator=g, dtype=torch.float64).requires_grad_(True)
    dy = torch.randn(B, D, generator=g, dtype=torch.float64)
    cat = torch.cat([st, x.unsqueeze(-1)], -1)
    y = (cat[..., -W:] * w).sum(-1) + b
    if act:
        y = torch.nn.functional.silu(y)
    y = y + x
    (y * dy).sum().backward()
    dx, dst, dw, db = O.causal_conv1d_update_bwd_ref(x.detach(), st.detach(), w.detach(), b.detach(), dy, act, residual=True)
    for a, r in ((dx, x.grad), (dst, st.grad), (dw, w.grad), (db, b.grad)):
        assert torch.allclose(a, r, rtol=1e-10, atol=1e-10)


RIGHT_PADDED_BWD = [c for c in GOLDEN_BWD_CASES if c.has("mask") and c.mask == "right"]


@pytest.mark.parametrize("c", RIGHT_PADDED_BWD, ids=[repr(c) for c in RIGHT_PADDED_BWD])
def test_packed_backward_oracle_equals_padded_backward_on_valid_positions(c):
    """Gradients on packed rows (seq_idx) against the padded backward oracle, which is pinned to the
    gradients of the reference's CanonLayer above: with the upstream gradient of the padded steps set to
    zero, dx at the valid positions, dweight and dbias must be the same numbers.  (Without that, the
    padded steps right behind a sequence send gradient into its last inputs and into the parameters.)"""
    x, w, b, m, dy = _inputs(c)
    lens = [int(v) for v in (m != 0).sum(1)]
    if sum(lens) == 0:
        pytest.skip("no valid position")
    dy = dy * m.unsqueeze(-1).to(dy.dtype)
    pdx, pdw, pdb = O.causal_conv1d_bwd_ref(x.transpose(1, 2), w, b, dy.transpose(1, 2), c.activation, attention_mask=m)
    xp = torch.cat([x[i, :n] for i, n in enumerate(lens)], 0).unsqueeze(0)
    dyp = torch.cat([dy[i, :n] for i, n in enumerate(lens)], 0).unsqueeze(0)
    ids = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(lens)]).unsqueeze(0)
    kdx, kdw, kdb = O.causal_conv1d_packed_bwd_ref(xp.transpose(1, 2), w, b, dyp.transpose(1, 2), c.activation,
                                                   seq_idx=ids)
    at = 0
    for i, n in enumerate(lens):
        assert torch.equal(kdx[0, :, at:at + n], pdx[i, :, :n]), f"sequence {i}"
        at += n
    assert torch.allclose(kdw, pdw, rtol=1e-9, atol=1e-9)
    if b is not None:
        # padded steps contribute silu'(bias) * 0 to dbias once their upstream gradient is zero
        assert torch.allclose(kdb, pdb, rtol=1e-9, atol=1e-9)
