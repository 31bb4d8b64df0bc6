"""Backward pass of causal_conv1d_fn on the GPU: both kernels against the float64 oracle, the
autograd wiring against finite differences (the reference's own gradient-test design,
causal-conv1d-mps/test.py:8-80, 259-321), and size-independent properties at the bench shape."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

import viby_model_b200 as V  # noqa: E402
from oracle import canon_oracle as O  # noqa: E402

DEV = torch.device("cuda", 0)
ULP = {torch.float32: 2.0 ** -23, torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10}  # relative spacing


def make(B, T, D, W, dtype, seed, channel_last=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, T, D, generator=g).to(dtype)
    dy = torch.randn(B, T, D, generator=g).to(dtype)
    w = (torch.rand(D, W, generator=g) - 0.5).to(dtype)
    b = (torch.rand(D, generator=g) - 0.5).to(dtype)
    if channel_last:
        x, dy = x.transpose(1, 2), dy.transpose(1, 2)
    else:
        x, dy = x.transpose(1, 2).contiguous(), dy.transpose(1, 2).contiguous()
    return x, dy, w, b


def mask_for(kind, B, T, seed):
    g = torch.Generator().manual_seed(seed)
    if kind == "none":
        return None
    if kind == "right":
        lens = torch.randint(max(T // 3, 1), T + 1, (B,), generator=g)
        m = (torch.arange(T)[None, :] < lens[:, None]).to(torch.int64)
        m[0, :] = 1
        if B > 1:
            m[1, 2:] = 0
        return m
    return (torch.rand(B, T, generator=g) > 0.3).to(torch.int64)  # holes


def magnitude(x, w, b, dy, act, m, residual):
    """Per-element sum of |terms| of dx: the scale rounding errors are measured against."""
    B, D, T = x.shape
    W = w.shape[1]
    _, dwa, _ = O.causal_conv1d_bwd_ref(x, w, b, dy, act, attention_mask=m)
    dxa, _, _ = O.causal_conv1d_bwd_ref(x.abs(), w.abs(), None, dy.abs(), None, attention_mask=m, residual=residual)
    return dxa.double(), dwa


def check(x, dy, w, b, act, m, residual, kernel):
    dev = lambda t: None if t is None else t.to(DEV)  # noqa: E731
    before = V.launch_count()
    dx, dw, db = V.causal_conv1d_bwd(dev(x), dev(w), dev(b), dev(dy), act, attention_mask=dev(m), residual=residual,
                                     kernel=kernel)
    assert V.launch_count() - before in (1, 2)  # two with the tile-classification pre-pass of masked launches
    if kernel is not None:
        assert V.last_kernel() == "bwd_" + kernel
    rdx, rdw, rdb = O.causal_conv1d_bwd_ref(x, w, b, dy, act, attention_mask=m, residual=residual)
    # dx: an fp32 sum rounded once; kernel and oracle may round a borderline value to neighbouring
    # numbers, so the bound is one step of the output type at the scale of the summed |terms|
    # (SiLU' scales each term by at most 1.1)
    scale, _ = magnitude(x, w, b, dy, act, m, residual)
    err = (dx.cpu().double() - rdx.double()).abs()
    bound = 1.1 * scale * (ULP[x.dtype] * 1.01 + 4e-6) + 1e-7
    assert bool((err <= bound).all()), f"dx: max err/bound {(err / bound).max().item():.2f}"
    assert dx.stride() == x.stride() and dx.dtype == x.dtype
    # parameter gradients: fp32 sums of exact products
    n = x.shape[0] * x.shape[2]
    wscale = rdw.abs().max().item() + 1e-3
    assert torch.allclose(dw.cpu().double(), rdw, rtol=2e-4, atol=2e-5 * wscale * n ** 0.5)
    if b is not None:
        bscale = rdb.abs().max().item() + 1e-3
        assert torch.allclose(db.cpu().double(), rdb, rtol=2e-4, atol=2e-5 * bscale * n ** 0.5)
    else:
        assert db is None
    return dx, dw, db


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("W", [2, 3, 4])
@pytest.mark.parametrize("act", [None, "silu"])
@pytest.mark.parametrize("mask_kind", ["none", "right", "holes"])
@pytest.mark.parametrize("kernel", ["generic", "tma"])
def test_backward_kernels_match_oracle(dtype, W, act, mask_kind, kernel):
    for (B, T, D) in ((2, 37, 64), (3, 200, 192), (1, 130, 1000 if dtype != torch.float32 else 500)):
        x, dy, w, b = make(B, T, D, W, dtype, seed=B * T + W)
        m = mask_for(mask_kind, B, T, seed=T)
        for residual in (False, True):
            check(x, dy, w, b, act, m, residual, kernel)
    torch.cuda.synchronize()
    assert V.tma_timeouts() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_backward_without_bias_and_time_major_layout(dtype):
    x, dy, w, _ = make(2, 96, 128, 4, dtype, seed=3)
    check(x, dy, w, None, "silu", mask_for("right", 2, 96, 1), True, None)
    x, dy, w, b = make(2, 96, 40, 4, dtype, seed=4, channel_last=False)  # contiguous [B,D,T]: generic kernel
    check(x, dy, w, b, "silu", None, False, None)
    assert V.last_kernel() == "bwd_generic"


def test_backward_kernels_agree_and_repeat():
    """Both kernels produce the same dx bits; launches back to back reuse the scheduler scratch."""
    x, dy, w, b = make(4, 700, 960, 4, torch.bfloat16, seed=9)
    m = mask_for("right", 4, 700, 5)
    dev = lambda t: t.to(DEV)  # noqa: E731
    ref = None
    for _ in range(3):
        dx, dw, db = V.causal_conv1d_bwd(dev(x), dev(w), dev(b), dev(dy), "silu", attention_mask=dev(m), residual=True,
                                         kernel="tma")
        if ref is None:
            ref = dx.clone()
        assert torch.equal(dx, ref)
    dxg, dwg, dbg = V.causal_conv1d_bwd(dev(x), dev(w), dev(b), dev(dy), "silu", attention_mask=dev(m), residual=True,
                                        kernel="generic")
    assert torch.equal(dxg, ref)
    assert torch.allclose(dwg, dw, rtol=1e-4, atol=1e-3)
    assert torch.allclose(dbg, db, rtol=1e-4, atol=1e-3)
    torch.cuda.synchronize()
    assert V.tma_timeouts() == 0


def numerical_grads(f, inputs, eps=1e-3):
    grads = []
    for inp in inputs:
        g = torch.zeros_like(inp)
        flat, gflat = inp.data.view(-1), g.view(-1)
        for j in range(flat.numel()):
            keep = flat[j].item()
            flat[j] = keep + eps
            lp = f().sum().item()
            flat[j] = keep - eps
            lm = f().sum().item()
            flat[j] = keep
            gflat[j] = (lp - lm) / (2 * eps)
        grads.append(g)
    return grads


@pytest.mark.parametrize("api", ["fn", "fused", "fwd"])
def test_autograd_matches_finite_differences(api):
    g = torch.Generator().manual_seed(11)
    B, T, D, W = 2, 12, 8, 4
    x = torch.randn(B, T, D, generator=g, dtype=torch.float32).to(DEV).requires_grad_(True)
    w = torch.randn(D, W, generator=g).to(DEV).requires_grad_(True)
    b = torch.randn(D, generator=g).to(DEV).requires_grad_(True)
    mask = torch.ones(B, T, device=DEV)
    mask[1, 9:] = 0
    weights = torch.randn(B, T, D, generator=g).to(DEV)  # so that the loss is not a plain sum

    def f():
        if api == "fn":
            y = V.causal_conv1d_fn(x.transpose(1, 2), w, b, activation="silu", attention_mask=mask,
                                   residual=True).transpose(1, 2)
        elif api == "fused":
            y = V.short_conv_fused(x, w, b, attention_mask=mask, activation=True, residual=True)
        else:
            y = V.causal_conv1d_fwd(x.transpose(1, 2).contiguous(), w, b, True).transpose(1, 2)
        return y * weights

    for t in (x, w, b):
        t.grad = None
    f().sum().backward()
    analytical = [x.grad.clone(), w.grad.clone(), b.grad.clone()]
    with torch.no_grad():
        numerical = numerical_grads(f, [x, w, b])
    for a, n in zip(analytical, numerical):
        assert torch.allclose(a, n, atol=2e-2, rtol=2e-2), (a - n).abs().max().item()


def test_autograd_residual_tensor_and_no_grad_path():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(2, 64, 128, generator=g).to(torch.bfloat16).to(DEV)
    r = torch.randn(2, 64, 128, generator=g).to(torch.bfloat16).to(DEV).requires_grad_(True)
    w = torch.randn(128, 4, generator=g).to(torch.bfloat16).to(DEV).requires_grad_(True)
    y = V.causal_conv1d_fn(x.transpose(1, 2), w, None, activation="silu", residual=r.transpose(1, 2))
    dy = torch.randn_like(y)
    y.backward(dy)
    assert torch.equal(r.grad, dy.transpose(1, 2))
    assert w.grad is not None and w.grad.dtype == torch.bfloat16
    before = V.launch_count()
    with torch.no_grad():
        V.causal_conv1d_fn(x.transpose(1, 2), w, None, activation="silu")
    assert V.launch_count() == before + 1


def test_backward_bench_shape_properties():
    """Bench shape (32 x 1024 x 3456 bf16, masked): linearity in dy, no gradient into masked inputs
    (residual aside), and dbias equal to the sum of g over rows, checked on a channel sample."""
    from viby_model_b200 import workloads as WL

    cfg = WL.CANON_D_PREFILL
    w, b = WL.weights(cfg.cfg, cfg.dim, cfg.width, cfg.dtype, device=DEV)
    x = WL.prefill_inputs(cfg, list(range(cfg.batch))).to(DEV)
    m = WL.attention_mask(cfg, device=DEV, dtype=torch.bool)
    g = torch.Generator(device=DEV).manual_seed(3)
    dy = torch.randn(x.shape, generator=g, device=DEV).to(cfg.dtype)
    xv, dyv = x.transpose(1, 2), dy.transpose(1, 2)
    dx1, dw1, db1 = V.causal_conv1d_bwd(xv, w, b, dyv, "silu", attention_mask=m)
    assert V.last_kernel() == "bwd_tma"
    dx2, dw2, db2 = V.causal_conv1d_bwd(xv, w, b, (2 * dy).transpose(1, 2), "silu", attention_mask=m)
    assert torch.equal(dx2, 2 * dx1)  # scaling by two is exact in binary floating point
    assert torch.allclose(dw2, 2 * dw1, rtol=1e-4, atol=1e-2)
    assert bool((dx1.transpose(1, 2)[~m] == 0).all())
    # oracle on a slice of channels and sequences
    ch = slice(1000, 1064)
    rdx, rdw, rdb = O.causal_conv1d_bwd_ref(xv[:4, ch].cpu(), w[ch].cpu(), b[ch].cpu(), dyv[:4, ch].cpu(), "silu",
                                            attention_mask=m[:4].cpu())
    err = (dx1[:4, ch].cpu().double() - rdx.double()).abs().max().item()
    assert err < 0.05
    torch.cuda.synchronize()
    assert V.tma_timeouts() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("L", [3, 4, 8])
@pytest.mark.parametrize("act", [None, "silu"])
@pytest.mark.parametrize("W", [2, 4])
def test_update_backward_matches_oracle(dtype, L, act, W):
    g = torch.Generator().manual_seed(L * 10 + W)
    B, D = 37, 200
    x = torch.randn(B, D, generator=g).to(dtype)
    st = torch.randn(B, D, L, generator=g).to(dtype)
    dy = torch.randn(B, D, generator=g).to(dtype)
    w = (torch.rand(D, W, generator=g) - 0.5).to(dtype)
    b = (torch.rand(D, generator=g) - 0.5).to(dtype)
    dev = lambda t: t.to(DEV)  # noqa: E731
    for residual in (False, True):
        dx, dst, dw, db = V.causal_conv1d_update_bwd(dev(x), dev(st), dev(w), dev(b), dev(dy), act, residual=residual)
        assert V.last_kernel() == "update_bwd"
        rdx, rdst, rdw, rdb = O.causal_conv1d_update_bwd_ref(x, st, w, b, dy, act, residual=residual)
        tol = dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
        assert torch.allclose(dx.cpu().float(), rdx.float(), **tol)
        assert torch.allclose(dst.cpu().float(), rdst.float(), **tol)
        assert torch.allclose(dw.cpu().double(), rdw, rtol=1e-3, atol=1e-3)
        assert torch.allclose(db.cpu().double(), rdb, rtol=1e-3, atol=1e-3)


def test_update_autograd_matches_finite_differences():
    """The reference's own test design for the decode step (causal-conv1d-mps/test.py:296-321):
    circular state with cache_seqlens, activation and residual on."""
    g = torch.Generator().manual_seed(2)
    B, D, W, L = 2, 8, 4, 8
    x = torch.randn(B, D, generator=g).to(DEV).requires_grad_(True)
    st = torch.randn(B, D, L, generator=g).to(DEV).requires_grad_(True)
    w = torch.randn(D, W, generator=g).to(DEV).requires_grad_(True)
    b = torch.randn(D, generator=g).to(DEV).requires_grad_(True)
    seqlens = torch.tensor([5, 11], dtype=torch.int32, device=DEV)
    coef = torch.randn(B, D, generator=g).to(DEV)

    def f():
        return V.short_conv_update(x, st.clone(), w, b, seqlens, activation=True, residual=True) * coef

    f().sum().backward()
    analytical = [x.grad.clone(), st.grad.clone(), w.grad.clone(), b.grad.clone()]
    with torch.no_grad():
        numerical = numerical_grads(f, [x, st, w, b])
    for a, n in zip(analytical, numerical):
        assert torch.allclose(a, n, atol=2e-2, rtol=2e-2), (a - n).abs().max().item()


def test_gradient_flows_through_two_decode_steps():
    """Back-propagation through time over two steps: the second step reads what the first wrote."""
    g = torch.Generator().manual_seed(8)
    B, D, W, L = 2, 6, 4, 4
    x1 = torch.randn(B, D, generator=g).to(DEV).requires_grad_(True)
    x2 = torch.randn(B, D, generator=g).to(DEV).requires_grad_(True)
    st0 = torch.randn(B, D, L, generator=g).to(DEV).requires_grad_(True)
    w = torch.randn(D, W, generator=g).to(DEV).requires_grad_(True)

    def f():
        st = st0.clone()
        y1 = V.causal_conv1d_update(x1, st, w, None, activation="silu")
        y2 = V.causal_conv1d_update(x2, st, w, None, activation="silu")
        return y1 * 0.5 + y2

    f().sum().backward()
    analytical = [x1.grad.clone(), x2.grad.clone(), st0.grad.clone(), w.grad.clone()]
    with torch.no_grad():
        numerical = numerical_grads(f, [x1, x2, st0, w])
    for a, n in zip(analytical, numerical):
        assert torch.allclose(a, n, atol=2e-2, rtol=2e-2), (a - n).abs().max().item()


@pytest.mark.parametrize("W", [2, 4])
def test_gradients_of_a_chunked_continuation(W):
    """Two chunks handing a state over: gradients of the second chunk, including the one with
    respect to the state it started from, against autograd over the whole sequence."""
    g = torch.Generator().manual_seed(13)
    B, D, T1, T2 = 2, 12, 9, 11
    x = torch.randn(B, T1 + T2, D, generator=g, dtype=torch.float64)
    w = torch.randn(D, W, generator=g, dtype=torch.float64)
    b = torch.randn(D, generator=g, dtype=torch.float64)
    coef = torch.randn(B, T2, D, generator=g, dtype=torch.float64)
    # float64 reference: the second chunk's outputs as a function of the first chunk's inputs
    xr = x.clone().requires_grad_(True)
    wr, br = w.clone().requires_grad_(True), b.clone().requires_grad_(True)
    yr = torch.nn.functional.silu(torch.nn.functional.conv1d(
        torch.nn.functional.pad(xr.transpose(1, 2), (W - 1, 0)), wr.unsqueeze(1), br, groups=D))
    (yr[..., T1:].transpose(1, 2) * coef).sum().backward()
    # kernels: state = last L columns of chunk 1, chunk 2 continues from it
    L = W + 1
    x2 = x[:, T1:].float().to(DEV).requires_grad_(True)
    st = x[:, T1 - L:T1].transpose(1, 2).contiguous().float().to(DEV).requires_grad_(True)
    wd, bd = w.float().to(DEV).requires_grad_(True), b.float().to(DEV).requires_grad_(True)
    y2 = V.causal_conv1d_fn(x2.transpose(1, 2), wd, bd, activation="silu", initial_states=st)
    assert V.last_kernel() in ("channel_last", "tma", "generic")
    before = V.launch_count()
    (y2.transpose(1, 2) * coef.float().to(DEV)).sum().backward()
    assert V.launch_count() == before + 1  # (the backward runs on an autograd thread: last_kernel() is per thread)
    assert torch.allclose(x2.grad.cpu().double(), xr.grad[:, T1:], rtol=1e-4, atol=1e-4)
    ref_dst = xr.grad[:, T1 - L:T1].transpose(1, 2)
    assert torch.allclose(st.grad.cpu().double(), ref_dst, rtol=1e-4, atol=1e-4)
    assert bool((st.grad[..., : L - (W - 1)] == 0).all())
    # parameter gradients of chunk 2 alone equal the whole-sequence ones because the loss only
    # looks at chunk 2
    assert torch.allclose(wd.grad.cpu().double(), wr.grad, rtol=1e-4, atol=1e-4)
    assert torch.allclose(bd.grad.cpu().double(), br.grad, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("masked", [False, True])
@pytest.mark.parametrize("T1,L", [(9, 3), (9, 6), (2, 5)])
def test_gradient_flows_through_the_returned_final_state(T1, L, masked):
    """Chunked training as the documentation describes it: ``y1, s = fn(x1, return_final_states=True)``
    then ``y2 = fn(x2, initial_states=s)``.  The gradient the second chunk sends into its initial state
    must reach the last inputs of the first chunk (and, when the first chunk is shorter than the state,
    the first chunk's own initial state): compared with float64 autograd over the whole sequence."""
    W = 4
    g = torch.Generator().manual_seed(31 + T1 + L)
    B, D, T0, T2 = 2, 16, 4, 11
    x = torch.randn(B, T0 + T1 + T2, D, generator=g, dtype=torch.float64)
    w = torch.randn(D, W, generator=g, dtype=torch.float64)
    b = torch.randn(D, generator=g, dtype=torch.float64)
    coef = torch.randn(B, T0 + T1 + T2, D, generator=g, dtype=torch.float64)
    mask = torch.ones(B, T0 + T1 + T2, dtype=torch.float64)
    if masked:
        mask[0, T0 + T1 - 1] = 0  # the last step of chunk 1 of one sequence is padding
        mask[1, T0 + 1] = 0
    xr = x.clone().requires_grad_(True)
    wr, br = w.clone().requires_grad_(True), b.clone().requires_grad_(True)
    xm = xr * mask.unsqueeze(-1)
    yr = torch.nn.functional.silu(torch.nn.functional.conv1d(
        torch.nn.functional.pad(xm.transpose(1, 2), (W - 1, 0)), wr.unsqueeze(1), br, groups=D))
    (yr[..., T0:].transpose(1, 2) * coef[:, T0:]).sum().backward()

    dev = lambda t: t.float().to(DEV)  # noqa: E731
    s0 = x[:, :T0].transpose(1, 2).contiguous().float().to(DEV).requires_grad_(True)  # history before chunk 1
    x1 = dev(x[:, T0:T0 + T1]).requires_grad_(True)
    x2 = dev(x[:, T0 + T1:]).requires_grad_(True)
    wd, bd = dev(w).requires_grad_(True), dev(b).requires_grad_(True)
    m1 = dev(mask[:, T0:T0 + T1]) if masked else None
    m2 = dev(mask[:, T0 + T1:]) if masked else None
    y1, s1 = V.causal_conv1d_fn(x1.transpose(1, 2), wd, bd, activation="silu", initial_states=s0, attention_mask=m1,
                                return_final_states=True, state_len=L)
    assert s1.requires_grad
    y2 = V.causal_conv1d_fn(x2.transpose(1, 2), wd, bd, activation="silu", initial_states=s1, attention_mask=m2)
    loss = (y1.transpose(1, 2) * dev(coef[:, T0:T0 + T1])).sum() + (y2.transpose(1, 2) * dev(coef[:, T0 + T1:])).sum()
    loss.backward()
    tol = dict(rtol=1e-4, atol=1e-4)
    assert torch.allclose(x1.grad.cpu().double(), xr.grad[:, T0:T0 + T1], **tol)
    assert torch.allclose(x2.grad.cpu().double(), xr.grad[:, T0 + T1:], **tol)
    assert torch.allclose(s0.grad.cpu().double(), xr.grad[:, :T0].transpose(1, 2), **tol)
    assert torch.allclose(wd.grad.cpu().double(), wr.grad, **tol)
    assert torch.allclose(bd.grad.cpu().double(), br.grad, **tol)


def test_backward_of_the_whole_ragged_configuration():
    """512 x 4096 x 3456 bf16: x, dy and dx are 14.5 GB each, byte offsets pass 2^32.  dx of sequences from the
    start, the middle and the end of the batch must equal the same sequences differentiated on their own;
    dweight / dbias of the first 8 sequences launched together must equal the sum of their single launches."""
    from viby_model_b200 import workloads as WL

    free, _ = torch.cuda.mem_get_info()
    if free < 60 * 2 ** 30:
        pytest.skip("needs 60 GB of free device memory")
    cfg = WL.RAGGED_SWEEP
    x = WL.prefill_inputs(cfg, device=DEV, generate_on="cuda")
    m = WL.attention_mask(cfg, device=DEV, dtype=torch.bool)
    w, b = WL.weights(cfg.cfg, cfg.dim, cfg.width, cfg.dtype, device=DEV)
    dy = torch.empty_like(x)
    g = torch.Generator(device=DEV).manual_seed(5)
    for i in range(0, cfg.batch, 64):
        dy[i:i + 64] = torch.randn(dy[i:i + 64].shape, generator=g, device=DEV).to(cfg.dtype)
    xv, dyv = x.transpose(1, 2), dy.transpose(1, 2)
    dx, dw, db = V.causal_conv1d_bwd(xv, w, b, dyv, "silu", attention_mask=m)
    assert V.last_kernel() == "bwd_tma"
    for i in (0, 1, 255, 256, 511):
        dxi, _, _ = V.causal_conv1d_bwd(xv[i:i + 1], w, b, dyv[i:i + 1], "silu", attention_mask=m[i:i + 1])
        assert torch.equal(dxi, dx[i:i + 1]), f"sequence {i}"
    _, dw8, db8 = V.causal_conv1d_bwd(xv[:8], w, b, dyv[:8], "silu", attention_mask=m[:8])
    dws, dbs = torch.zeros_like(dw8), torch.zeros_like(db8)
    for i in range(8):
        _, dwi, dbi = V.causal_conv1d_bwd(xv[i:i + 1], w, b, dyv[i:i + 1], "silu", attention_mask=m[i:i + 1])
        dws += dwi
        dbs += dbi
    assert torch.allclose(dw8, dws, rtol=1e-4, atol=1e-2) and torch.allclose(db8, dbs, rtol=1e-4, atol=1e-2)
    assert bool(torch.isfinite(dw).all()) and bool(torch.isfinite(db).all())
    torch.cuda.synchronize()
    assert V.tma_timeouts() == 0
