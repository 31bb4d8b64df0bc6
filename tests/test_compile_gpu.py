"""torch.compile(fullgraph=True) over code that calls the operators (the reference compiles its
model this way for evaluation, eval_model.py:157): the operators must trace as single graph nodes
and give the eager results, forward and backward."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

import viby_model_b200 as V  # noqa: E402

DEV = torch.device("cuda", 0)


def canon_like(x, w, b, mask):
    """The fused CanonLayer body: mask, conv, SiLU, residual, final state; then a scaling to have
    ordinary torch ops on both sides of the operator."""
    y, state = V.causal_conv1d_fn((x * 1.0).transpose(1, 2), w, b, activation="silu", attention_mask=mask,
                                  residual=True, return_final_states=True, state_len=4)
    return y.transpose(1, 2) * 2.0, state


def decode_like(xt, state, w, b):
    y = V.causal_conv1d_update(xt, state, w, b, activation="silu")
    return y + 1.0


@pytest.mark.parametrize("backend", ["aot_eager", "inductor"])
def test_compiled_prefill_and_decode_match_eager(backend):
    g = torch.Generator().manual_seed(0)
    B, T, D = 3, 96, 256
    x = torch.randn(B, T, D, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(D, 4, generator=g).to(torch.bfloat16).to(DEV)
    b = torch.randn(D, generator=g).to(torch.bfloat16).to(DEV)
    mask = (torch.arange(T, device=DEV)[None, :] < torch.tensor([96, 40, 7], device=DEV)[:, None])
    y_ref, st_ref = canon_like(x, w, b, mask)
    before = V.launch_count()
    compiled = torch.compile(canon_like, backend=backend, fullgraph=True)
    y, st = compiled(x, w, b, mask)
    assert V.launch_count() > before, "the compiled graph did not reach the CUDA kernels"
    assert torch.equal(y, y_ref) and torch.equal(st, st_ref)

    xt = torch.randn(B, D, generator=g).to(torch.bfloat16).to(DEV)
    s_eager, s_comp = st_ref.clone(), st_ref.clone()
    y1 = decode_like(xt, s_eager, w, b)
    y2 = torch.compile(decode_like, backend=backend, fullgraph=True)(xt, s_comp, w, b)
    assert torch.equal(y1, y2)
    assert torch.equal(s_eager, s_comp), "the in-place state update was lost in the compiled graph"


@pytest.mark.parametrize("backend", ["aot_eager", "inductor"])
def test_compiled_backward_matches_eager(backend):
    g = torch.Generator().manual_seed(1)
    B, T, D = 2, 64, 128
    w0 = torch.randn(D, 4, generator=g).to(DEV)
    b0 = torch.randn(D, generator=g).to(DEV)
    x0 = torch.randn(B, T, D, generator=g).to(DEV)
    mask = torch.ones(B, T, device=DEV, dtype=torch.bool)
    mask[1, 50:] = False

    def loss_fn(x, w, b):
        y, _ = canon_like(x, w, b, mask)
        return (y * y).sum()

    grads = []
    for fn in (loss_fn, torch.compile(loss_fn, backend=backend, fullgraph=True)):
        x, w, b = (t.clone().requires_grad_(True) for t in (x0, w0, b0))
        fn(x, w, b).backward()
        grads.append((x.grad, w.grad, b.grad))
    for a, c in zip(*grads):
        assert torch.allclose(a, c, rtol=1e-4, atol=1e-3)


def test_compiled_multi_tensor_call_on_slices_of_one_projection():
    """q | k | v as column slices of one fused projection (non-dense inputs): the shape function of the
    custom op must describe the tensor the launch wrapper really allocates, or the compiled graph
    asserts on strides (or indexes the result wrongly)."""
    g = torch.Generator().manual_seed(4)
    B, T = 2, 80
    dims = (128, 32, 32)
    qkv = torch.randn(B, T, sum(dims), generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(sum(dims), 4, generator=g).to(torch.bfloat16).to(DEV)
    b = torch.randn(sum(dims), generator=g).to(torch.bfloat16).to(DEV)

    def fn(qkv, w, b):
        parts = [p.transpose(1, 2) for p in (qkv * 1.0).split(dims, dim=-1)]
        outs = V.causal_conv1d_fn_multi(parts, w, b, activation="silu", residual=True)
        return torch.cat([o.transpose(1, 2) for o in outs], dim=-1) + 1.0

    ref = fn(qkv, w, b)
    whole = V.causal_conv1d_fn(qkv.transpose(1, 2), w, b, activation="silu", residual=True).transpose(1, 2) + 1.0
    assert torch.equal(ref, whole)
    for backend in ("aot_eager", "inductor"):
        out = torch.compile(fn, backend=backend, fullgraph=True)(qkv, w, b)
        assert torch.equal(out, ref), backend


def test_compiled_as_the_reference_compiles_its_model():
    """eval_model.py:157 of the reference: torch.compile(model, mode="reduce-overhead", fullgraph=True),
    i.e. inductor with CUDA graphs.  Prefill and a few decode steps, replayed several times."""
    g = torch.Generator().manual_seed(6)
    B, T, D = 2, 128, 640
    w = torch.randn(D, 4, generator=g).to(torch.bfloat16).to(DEV)
    b = torch.randn(D, generator=g).to(torch.bfloat16).to(DEV)
    mask = (torch.arange(T, device=DEV)[None, :] < torch.tensor([128, 50], device=DEV)[:, None])
    prefill = torch.compile(canon_like, mode="reduce-overhead", fullgraph=True)
    decode = torch.compile(decode_like, mode="reduce-overhead", fullgraph=True)
    for rep in range(4):  # warm-up runs, graph capture, replays
        x = torch.randn(B, T, D, generator=g).to(torch.bfloat16).to(DEV)
        y_ref, st_ref = canon_like(x, w, b, mask)
        before = V.launch_count()
        y, st = prefill(x, w, b, mask)
        y, st = y.clone(), st.clone()  # outputs of a replayed graph live in its pool
        if rep < 2:
            assert V.launch_count() > before
        assert torch.equal(y, y_ref) and torch.equal(st, st_ref), rep
        s_eager, s_comp = st_ref.clone(), st_ref.clone()
        for _ in range(3):
            xt = torch.randn(B, D, generator=g).to(torch.bfloat16).to(DEV)
            y1 = decode_like(xt, s_eager, w, b)
            y2 = decode(xt, s_comp, w, b).clone()
            assert torch.equal(y1, y2)
            assert torch.equal(s_eager, s_comp)
    torch.cuda.synchronize()
    assert V.tma_timeouts() == 0


@pytest.mark.parametrize("backend", ["aot_eager", "inductor"])
def test_compiled_backward_of_a_chunked_continuation_and_of_a_decode_step(backend):
    g = torch.Generator().manual_seed(9)
    B, T, D, L = 2, 24, 64, 4
    x0 = torch.randn(B, T, D, generator=g).to(DEV)
    s0 = torch.randn(B, D, L, generator=g).to(DEV)
    w0 = torch.randn(D, 4, generator=g).to(DEV)
    b0 = torch.randn(D, generator=g).to(DEV)
    xt0 = torch.randn(B, D, generator=g).to(DEV)

    def loss_fn(x, s, w, b, xt):
        y, state = V.causal_conv1d_fn(x.transpose(1, 2), w, b, activation="silu", initial_states=s,
                                      return_final_states=True, state_len=L)
        step = V.causal_conv1d_update(xt, state.detach().clone(), w, b, activation="silu")
        return (y * y).sum() + (state * state).sum() + (step * step).sum()

    grads = []
    for fn in (loss_fn, torch.compile(loss_fn, backend=backend, fullgraph=True)):
        leaves = [t.clone().requires_grad_(True) for t in (x0, s0, w0, b0, xt0)]
        fn(*leaves).backward()
        grads.append([t.grad for t in leaves])
    for a, c in zip(*grads):
        assert a is not None and c is not None
        assert torch.allclose(a, c, rtol=1e-4, atol=1e-3)
