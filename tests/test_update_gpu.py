"""Parity of causal_conv1d_update (CUDA, through the C ABI) with the CPU oracle: outputs within
tolerance, conv_state bit-exact, for the shifting state at every supported length and the
circular state of causal-conv1d-mps; then the decode configuration at full size."""
import pytest
import torch

import viby_model_b200 as V
from viby_model_b200 import workloads as WL
from conftest import GOLDEN_CASES
from oracle import canon_oracle as O
from parity import assert_close_to_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


def bits(t):
    return t.view(torch.int32 if t.dtype == torch.float32 else torch.int16)


def expected_kernel(dtype, L, kernel=None, circular=False):
    """State rows of 16 or 32 bytes (and every such circular state) take the one-channel-per-lane
    kernel, other short shifting states the 8-channels-per-thread kernel, the rest the scalar one."""
    if kernel == "generic":
        return "update_generic"
    row_bytes = L * (4 if dtype == torch.float32 else 2)
    if row_bytes in (16, 32) and not (dtype == torch.float32 and L == 4 and not circular):
        return "update_lane"
    if circular or L not in (1, 2, 3, 4, 8):
        return "update_generic"
    return "update_vec"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("W", [2, 3, 4])
@pytest.mark.parametrize("L", [1, 2, 3, 4, 5, 8, 11])
@pytest.mark.parametrize("kernel", [None, "generic"])
def test_update_steps(dtype, W, L, kernel):
    if L < W - 1:
        pytest.skip("state shorter than the history the taps need")
    B, D = 5, 64
    g = torch.Generator().manual_seed(100 + 10 * W + L)
    w = (torch.rand(D, W, generator=g) - 0.5).to(dtype)
    b = (torch.rand(D, generator=g) - 0.5).to(dtype)
    state = torch.randn(B, D, L, generator=g).to(dtype)
    sd = state.to(DEV)
    wd, bd = w.to(DEV), b.to(DEV)
    for step in range(6):
        xt = torch.randn(B, D, generator=g).to(dtype)
        before = V.launch_count()
        y = V.causal_conv1d_update(xt.to(DEV), sd, wd, bd, activation="silu", kernel=kernel)
        assert V.launch_count() == before + 1
        ref = O.causal_conv1d_update_ref(xt, state, w, b, "silu")
        assert_close_to_oracle(y, ref, f"step {step}")
        assert torch.equal(bits(sd.cpu()), bits(state)), f"state after step {step}"
    assert V.last_kernel() == expected_kernel(dtype, L, kernel)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_update_odd_dim_and_no_bias_no_activation(dtype):
    B, D, W, L = 3, 21, 4, 4
    g = torch.Generator().manual_seed(5)
    w = torch.randn(D, W, generator=g).to(dtype)
    state = torch.randn(B, D, L, generator=g).to(dtype)
    sd = state.to(DEV)
    xt = torch.randn(B, D, generator=g).to(dtype)
    y = V.causal_conv1d_update(xt.to(DEV), sd, w.to(DEV))
    # 21 channels are no multiple of a 128-bit vector: fp32 rows of 16 bytes still take the
    # one-channel-per-lane kernel, bf16 rows of 8 bytes the scalar one
    assert V.last_kernel() == ("update_lane" if dtype == torch.float32 else "update_generic")
    assert_close_to_oracle(y, O.causal_conv1d_update_ref(xt, state, w))
    assert torch.equal(bits(sd.cpu()), bits(state))


def test_update_state_moves_raw_bits():
    """NaN payloads and signed zeros travel through the state unchanged."""
    B, D, L = 2, 16, 4
    state = torch.zeros(B, D, L, dtype=torch.bfloat16)
    raw = bits(state)
    raw[0, :, 1] = 0x7FA5  # NaN with a payload
    raw[1, :, 2] = -0x8000  # -0.0
    xt = torch.randn(B, D).bfloat16()
    w = torch.randn(D, 4).bfloat16()
    sd = state.to(DEV)
    V.causal_conv1d_update(xt.to(DEV), sd, w.to(DEV))
    got = bits(sd.cpu())
    assert torch.equal(got[..., :3], raw[..., 1:])
    assert torch.equal(got[..., 3], bits(xt))


def test_update_accepts_trailing_singleton_and_strided_x():
    B, D, L = 4, 64, 4
    g = torch.Generator().manual_seed(8)
    w = torch.randn(D, 4, generator=g).bfloat16()
    state = torch.randn(B, D, L, generator=g).bfloat16()
    x3 = torch.randn(B, 1, D, generator=g).bfloat16()
    sd = state.to(DEV)
    # the model hands over x[B,1,D].squeeze(1); also accept [B,D,1]
    y = V.causal_conv1d_update(x3.to(DEV).squeeze(1), sd, w.to(DEV), activation="silu")
    ref = O.causal_conv1d_update_ref(x3.squeeze(1), state, w, None, "silu")
    assert_close_to_oracle(y, ref)
    y2 = V.causal_conv1d_update(x3.to(DEV).transpose(1, 2), sd, w.to(DEV), activation="silu")
    ref2 = O.causal_conv1d_update_ref(x3.squeeze(1), state, w, None, "silu")
    assert y2.shape == (B, D, 1)
    assert_close_to_oracle(y2.squeeze(-1), ref2)
    assert torch.equal(bits(sd.cpu()), bits(state))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("W,L,D", [(4, 8, 32), (4, 8, 1001), (3, 8, 64), (2, 16, 40), (4, 4, 48), (4, 5, 32), (3, 2, 32)])
def test_circular_state_update(dtype, W, L, D):
    """cache_seqlens mode (causal_conv1d.metal:586-664), per-sequence write positions."""
    B = 5
    g = torch.Generator().manual_seed(17)
    w = (torch.rand(D, W, generator=g) - 0.5).to(dtype)
    b = (torch.rand(D, generator=g) - 0.5).to(dtype)
    state = torch.randn(B, D, L, generator=g).to(dtype)
    seqlens = torch.tensor([0, 3, 7, 12, 1000003], dtype=torch.int32)
    sd = state.to(DEV)
    for step in range(10):
        xt = torch.randn(B, D, generator=g).to(dtype)
        y = V.causal_conv1d_update(xt.to(DEV), sd, w.to(DEV), b.to(DEV), activation="silu",
                                   cache_seqlens=seqlens.to(DEV), residual=True)
        ref = O.causal_conv1d_update_ref(xt, state, w, b, "silu", cache_seqlens=seqlens, residual=True)
        assert V.last_kernel() == expected_kernel(dtype, L, circular=True)
        assert_close_to_oracle(y, ref, f"circular step {step}")
        assert torch.equal(bits(sd.cpu()), bits(state))
        seqlens = seqlens + 1


@pytest.mark.parametrize("c", [c for c in GOLDEN_CASES if c.T > 1], ids=lambda c: repr(c))
def test_golden_decode_after_prefill(c):
    """Prefill with the kernel, then the reference's recorded decode steps: the 8-wide state
    must equal the reference's bit for bit after every step, outputs within tolerance."""
    x = c.get("x")
    w = c.get("weight")
    b = c.get("bias") if c.has("bias") else None
    m = c.get("mask") if c.has("mask") else None
    act = "silu" if c.activation else None
    wd = w.to(DEV)
    bd = b.to(DEV) if b is not None else None
    _, st = V.causal_conv1d_fn(x.to(DEV).transpose(1, 2), wd, bd, activation=act,
                               attention_mask=m.to(DEV) if m is not None else None,
                               return_final_states=True, state_len=8)
    xs = c.get("decode_x")
    for s in range(xs.shape[0]):
        xt = xs[s].squeeze(1).to(DEV)
        y = V.causal_conv1d_update(xt, st, wd, bd, activation=act)
        out = (xt + y).cpu()
        ref = c.get("decode_out")[s].squeeze(1)
        if c.dtype == torch.float32:
            assert torch.allclose(out, ref, rtol=1e-5, atol=1e-6)
        else:
            assert torch.allclose(out.float(), ref.float(), rtol=2 ** -6, atol=2 ** -6)
        assert torch.equal(bits(st.cpu()), bits(c.get("decode_state")[s]))


@pytest.mark.parametrize("L", [3, 4, 8])
def test_config3_decode_1024_steps(L):
    """batch 256, dim 960, width 4, bf16; conv_state seeded from a 512-token prefill; 1024
    successive steps; every output checked, the final state bit-exact."""
    cfg = WL.DECODE_CANON_B
    w, b = WL.weights(cfg.cfg, cfg.dim, cfg.width, cfg.dtype)
    pre = WL.decode_prefill(cfg)
    toks = WL.decode_tokens(cfg)
    wd, bd = w.to(DEV), b.to(DEV)
    _, st = V.causal_conv1d_fn(pre.to(DEV).transpose(1, 2), wd, bd, return_final_states=True, state_len=L)
    ref_state = pre.transpose(1, 2)[..., -L:].contiguous()
    assert torch.equal(bits(st.cpu()), bits(ref_state))
    toks_d = toks.to(DEV)
    ys = torch.empty_like(toks_d)
    before = V.launch_count()
    for s in range(cfg.steps):
        V.causal_conv1d_update(toks_d[s], st, wd, bd, out=ys[s])
    assert V.launch_count() == before + cfg.steps
    assert V.last_kernel() == expected_kernel(cfg.dtype, L)
    ys = ys.cpu()
    for s in range(cfg.steps):
        ref = O.causal_conv1d_update_ref(toks[s], ref_state, w, b)
        assert_close_to_oracle(ys[s], ref, f"cfg3 step {s}")
    assert torch.equal(bits(st.cpu()), bits(ref_state))
    # decoding continues the prefill: the outputs equal a prefill over [prefill | tokens]
    full = torch.cat([pre, toks.transpose(0, 1)], dim=1).to(DEV)
    y_full = V.causal_conv1d_fn(full.transpose(1, 2), wd, bd)
    assert torch.equal(y_full[..., cfg.prefill_len:].cpu(), ys.permute(1, 2, 0))


def _multi_problems(dtype, seed=7):
    """Decode steps of different shapes, layouts and options: (batch, dim, state_len, width, bias, layout)."""
    g = torch.Generator().manual_seed(seed)
    specs = [(64, 640, 4, 4, False, "dense"), (64, 960, 4, 4, True, "dense"), (64, 3456, 4, 4, True, "dense"),
             (7, 128, 3, 4, True, "dense"), (5, 72, 3, 4, True, "x3d"), (3, 21, 5, 3, True, "dense"),
             (4, 64, 8, 4, False, "dense"), (6, 96, 4, 4, True, "strided_state"), (9, 256, 4, 4, True, "circular"),
             (2, 64, 2, 3, True, "dense"), (1, 8, 4, 4, True, "dense")]
    problems = []
    for B, D, L, W, has_bias, layout in specs:
        x = torch.randn(B, D, generator=g).to(dtype).to(DEV)
        w = (torch.rand(D, W, generator=g) - 0.5).to(dtype).to(DEV)
        b = (torch.rand(D, generator=g) - 0.5).to(dtype).to(DEV) if has_bias else None
        state = torch.randn(B, D, L, generator=g).to(dtype).to(DEV)
        seqlens = None
        if layout == "strided_state":
            state = torch.randn(B, L, D, generator=g).to(dtype).to(DEV).transpose(1, 2)  # [B, D, L] view, channel stride 1
        if layout == "circular":
            seqlens = torch.randint(0, 50, (B,), generator=g).to(torch.int32).to(DEV)
        if layout == "x3d":
            x = x.unsqueeze(-1)
        problems.append((x, state, w, b, seqlens))
    return problems


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("activation", [None, "silu"])
def test_update_multi_matches_separate_calls(dtype, activation):
    """Eleven independent decode steps of different shapes in one launch (vc1d_update_multi): outputs and
    states bit-equal to causal_conv1d_update on each, whichever code a problem takes inside the kernel
    (vectorised for the most common width and state length, scalar for the rest: other lengths, strided or
    circular states, odd channel counts)."""
    problems = _multi_problems(dtype)
    want_y, want_s = [], []
    for x, state, w, b, seqlens in problems:
        s2 = state.clone()
        want_y.append(V.causal_conv1d_update(x, s2, w, b, activation, seqlens))
        want_s.append(s2)
    for step in range(2):  # twice: the states move on
        if step == 1:
            for i, (x, state, w, b, seqlens) in enumerate(problems):
                want_y[i] = V.causal_conv1d_update(x, want_s[i], w, b, activation, seqlens)
        before = V.launch_count()
        ys = V.causal_conv1d_update_multi([p[0] for p in problems], [p[1] for p in problems], [p[2] for p in problems],
                                          [p[3] for p in problems], activation, [p[4] for p in problems])
        assert V.launch_count() == before + 1 and V.last_kernel() == "update_multi"
        for i, (x, state, w, b, seqlens) in enumerate(problems):
            assert ys[i].shape == x.shape, i
            assert torch.equal(bits(ys[i]), bits(want_y[i])), (step, i)
            assert torch.equal(bits(state.contiguous()), bits(want_s[i].contiguous())), (step, i)


def test_update_table_steps_its_buffers_again():
    """A table built once and launched for several tokens: new inputs are written into its x buffers, the
    states move on in place, every step bit-equal to separate calls."""
    dtype = torch.bfloat16
    problems = _multi_problems(dtype, seed=9)[:6]
    table = V.UpdateTable([p[0] for p in problems], [p[1] for p in problems], [p[2] for p in problems],
                          [p[3] for p in problems], "silu")
    assert len(table) == 6
    shadow = [p[1].clone() for p in problems]
    g = torch.Generator(device=DEV).manual_seed(10)
    for step in range(4):
        for x, *_ in problems:
            x.copy_(torch.randn(x.shape, generator=g, device=DEV).to(dtype))
        before = V.launch_count()
        ys = table.launch()
        assert V.launch_count() == before + 1
        for i, (x, state, w, b, _) in enumerate(problems):
            want = V.causal_conv1d_update(x, shadow[i], w, b, "silu")
            assert torch.equal(bits(ys[i]), bits(want)), (step, i)
            assert torch.equal(bits(state), bits(shadow[i])), (step, i)


def test_update_multi_against_oracle_and_in_chunks():
    """More problems than one launch holds (80): split over launches; every result against the CPU oracle."""
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(31)
    n, B, D, L, W = 100, 4, 64, 3, 4
    xs = [torch.randn(B, D, generator=g).to(dtype) for _ in range(n)]
    ws = [(torch.rand(D, W, generator=g) - 0.5).to(dtype) for _ in range(n)]
    bs = [(torch.rand(D, generator=g) - 0.5).to(dtype) for _ in range(n)]
    states = [torch.randn(B, D, L, generator=g).to(dtype) for _ in range(n)]
    sd = [s.to(DEV) for s in states]
    before = V.launch_count()
    ys = V.causal_conv1d_update_multi([x.to(DEV) for x in xs], sd, [w.to(DEV) for w in ws], [b.to(DEV) for b in bs], "silu")
    assert V.launch_count() == before + 2
    for i in range(n):
        ref = O.causal_conv1d_update_ref(xs[i], states[i], ws[i], bs[i], "silu")  # moves states[i] on
        assert_close_to_oracle(ys[i], ref, f"problem {i}")
        assert torch.equal(bits(sd[i].cpu()), bits(states[i])), i


def test_update_multi_argument_errors():
    x = torch.zeros(2, 64, device=DEV)
    s = torch.zeros(2, 64, 3, device=DEV)
    w = torch.zeros(64, 4, device=DEV)
    with pytest.raises(ValueError, match="same length"):
        V.causal_conv1d_update_multi([x, x], [s], [w, w])
    with pytest.raises(ValueError, match="one dtype"):
        V.causal_conv1d_update_multi([x, x.bfloat16()], [s, s.bfloat16()], [w, w.bfloat16()])
    with pytest.raises(ValueError, match="doesn't match conv_state"):
        V.causal_conv1d_update_multi([x], [torch.zeros(3, 64, 3, device=DEV)], [w])
    assert V.causal_conv1d_update_multi([], [], []) == []
