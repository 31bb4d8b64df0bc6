"""The oracle against the golden vectors made by the reference's own CanonLayer, and against an
independent float64 restatement of the tap formula.  CPU only."""
import pytest
import torch

from conftest import GOLDEN_CASES
from oracle import canon_oracle as O
from parity import assert_close_to_oracle

IDS = [repr(c) for c in GOLDEN_CASES]


def _inputs(c):
    x = c.get("x")
    w = c.get("weight")
    b = c.get("bias") if c.has("bias") else None
    m = c.get("mask") if c.has("mask") else None
    return x, w, b, m


def _close(a, b, dtype):
    if dtype == torch.float32:
        return torch.allclose(a, b, rtol=2e-6, atol=2e-6)
    return torch.equal(a, b)


@pytest.mark.parametrize("c", GOLDEN_CASES, ids=IDS)
def test_native_restatement_matches_reference_prefill(c):
    """canon_layer_ref(native_dtype=True) follows the reference op for op: same numbers."""
    x, w, b, m = _inputs(c)
    out, _ = O.canon_layer_ref(x, w, b, c.activation, attention_mask=m, native_dtype=True)
    assert _close(out, c.get("prefill_out"), c.dtype)
    out2, state = O.canon_layer_ref(x, w, b, c.activation, attention_mask=m, use_cache=True, native_dtype=True)
    assert _close(out2, c.get("prefill_cache_out"), c.dtype)
    assert torch.equal(state, c.get("prefill_state"))


@pytest.mark.parametrize("c", GOLDEN_CASES, ids=IDS)
def test_native_restatement_matches_reference_decode_and_chunks(c):
    x, w, b, m = _inputs(c)
    _, state = O.canon_layer_ref(x, w, b, c.activation, attention_mask=m, use_cache=True, native_dtype=True)
    xs = c.get("decode_x")
    for s in range(xs.shape[0]):
        out, state = O.canon_layer_ref(xs[s], w, b, c.activation, conv_state=state, use_cache=True,
                                       native_dtype=True)
        assert _close(out, c.get("decode_out")[s], c.dtype), f"step {s}"
        assert torch.equal(state, c.get("decode_state")[s]), f"state after step {s}"
    _, state = O.canon_layer_ref(x, w, b, c.activation, attention_mask=m, use_cache=True, native_dtype=True)
    for tag in ("chunk5", "chunk12"):
        out, state = O.canon_layer_ref(c.get(f"{tag}_x"), w, b, c.activation, conv_state=state, use_cache=True,
                                       native_dtype=True)
        assert _close(out, c.get(f"{tag}_out"), c.dtype), tag
        assert torch.equal(state, c.get(f"{tag}_state")), tag


@pytest.mark.parametrize("c", GOLDEN_CASES, ids=IDS)
def test_round_once_oracle_agrees_with_reference(c):
    """The fp32-accumulate / round-once oracle (the kernels' contract) vs the reference's own
    arithmetic: equal within fp32 noise for fp32 layers, within 2 bf16 ulp for bf16 layers (the
    reference rounds after the conv and again after SiLU and the residual)."""
    x, w, b, m = _inputs(c)
    act = "silu" if c.activation else None
    xm = x * m.unsqueeze(-1).to(x.dtype) if m is not None else x
    y, state = O.causal_conv1d_ref(x.transpose(1, 2), w, b, act, attention_mask=m, state_len=8)
    out = xm + y.transpose(1, 2)
    ref = c.get("prefill_cache_out")
    if c.dtype == torch.float32:
        assert torch.allclose(out, ref, rtol=1e-5, atol=1e-6)
    else:
        # compare the conv term only: subtracting the residual exactly in fp32
        assert torch.allclose(out.float(), ref.float(), rtol=2 ** -6, atol=2 ** -6)
    if c.T > 1:  # with T == 1 and a cache the reference takes the single-step path
        assert torch.equal(state, c.get("prefill_state"))


@pytest.mark.parametrize("c", GOLDEN_CASES, ids=IDS)
def test_update_oracle_matches_reference_steps(c):
    """causal_conv1d_update_ref with state_len 8, 4 (the CUDA branch's width) and W-1 gives the
    reference's decode outputs; the 8-wide state matches bit for bit."""
    x, w, b, m = _inputs(c)
    act = "silu" if c.activation else None
    W = w.shape[1]
    _, s8 = O.causal_conv1d_ref(x.transpose(1, 2), w, b, act, attention_mask=m, state_len=8)
    if c.T == 1:
        pytest.skip("reference prefill of one token with a cache is already a decode step")
    states = {L: s8[..., 8 - L:].clone() for L in (8, W, W - 1) if L >= 1}
    xs = c.get("decode_x")
    for s in range(xs.shape[0]):
        xt = xs[s].squeeze(1)
        ref_out = c.get("decode_out")[s].squeeze(1)
        for L, st in states.items():
            y = O.causal_conv1d_update_ref(xt, st, w, b, act)
            out = xt + y
            if c.dtype == torch.float32:
                assert torch.allclose(out, ref_out, rtol=1e-5, atol=1e-6), (s, L)
            else:
                assert torch.allclose(out.float(), ref_out.float(), rtol=2 ** -6, atol=2 ** -6), (s, L)
        assert torch.equal(states[8], c.get("decode_state")[s])
        for L, st in states.items():
            assert torch.equal(st, states[8][..., 8 - L:])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("act", [None, "silu"])
@pytest.mark.parametrize("W", [2, 3, 4])
@pytest.mark.parametrize("T", [1, 2, 3, 4, 5, 9, 64])
def test_oracle_matches_float64_tap_formula(dtype, act, W, T):
    x = O.seeded((2, 12, T), 11 + T, "normal", dtype)
    w = O.seeded((12, W), 12, "uniform", dtype)
    b = O.seeded((12,), 13, "uniform", dtype)
    y32 = O.causal_conv1d_ref(x, w, b, act, return_fp32=True)
    y64 = torch.from_numpy(O.causal_conv1d_f64(x, w, b, act))
    assert torch.allclose(y32.double(), y64, rtol=2e-6, atol=2e-6)


def test_circular_update_equals_shifting_update():
    """The circular-buffer step (causal_conv1d.metal:586-664) computes the same outputs as the
    shifting step when both start from an empty history."""
    B, D, W, L = 3, 16, 4, 8
    w = O.seeded((D, W), 1, "uniform")
    b = O.seeded((D,), 2, "uniform")
    shift_state = torch.zeros(B, D, L)
    circ_state = torch.zeros(B, D, L)
    seqlens = torch.zeros(B, dtype=torch.int32)
    for s in range(20):
        xt = O.seeded((B, D), 100 + s)
        y1 = O.causal_conv1d_update_ref(xt, shift_state, w, b, "silu", residual=True)
        y2 = O.causal_conv1d_update_ref(xt, circ_state, w, b, "silu", cache_seqlens=seqlens, residual=True)
        assert torch.allclose(y1, y2, rtol=1e-6, atol=1e-6)
        seqlens += 1


def test_initial_states_continue_a_sequence():
    """Splitting a sequence and passing the first part's final state as initial_states gives
    the same outputs as one pass (the chunked continuation of model/model.py:607-661)."""
    x = O.seeded((2, 16, 40), 5)
    w = O.seeded((16, 4), 6, "uniform")
    y_full, s_full = O.causal_conv1d_ref(x, w, None, "silu", state_len=4)
    y1, s1 = O.causal_conv1d_ref(x[..., :17], w, None, "silu", state_len=4)
    y2, s2 = O.causal_conv1d_ref(x[..., 17:], w, None, "silu", initial_states=s1, state_len=4)
    assert torch.allclose(torch.cat([y1, y2], -1), y_full, rtol=1e-6, atol=1e-6)
    assert torch.equal(s2, s_full)


def _pack_valid(x_btd, m):
    """Right-padded [B,T,D] + mask [B,T] -> packed [1, sum(len), D], seq_idx [1, sum(len)], lengths."""
    lens = [int(v) for v in (m != 0).sum(1)]
    rows = [x_btd[b, :n] for b, n in enumerate(lens)]
    ids = torch.cat([torch.full((n,), b, dtype=torch.int32) for b, n in enumerate(lens)])
    return torch.cat(rows, 0).unsqueeze(0), ids.unsqueeze(0), lens


RIGHT_PADDED = [c for c in GOLDEN_CASES if c.has("mask") and c.mask == "right"]


@pytest.mark.parametrize("c", RIGHT_PADDED, ids=[repr(c) for c in RIGHT_PADDED])
def test_packed_oracle_reproduces_reference_on_valid_positions(c):
    """Packing the valid prefixes of a right-padded batch end to end and convolving with seq_idx gives,
    at every valid position, what the reference's CanonLayer gives for the padded batch."""
    x, w, b, m = _inputs(c)
    act = "silu" if c.activation else None
    xp, ids, lens = _pack_valid(x, m)
    if xp.shape[1] == 0:
        pytest.skip("no valid position")
    yp = O.causal_conv1d_packed_ref(xp.transpose(1, 2), w, b, act, seq_idx=ids).transpose(1, 2)
    ref = c.get("prefill_out")
    at = 0
    for bi, n in enumerate(lens):
        out = x[bi, :n] + yp[0, at:at + n]
        if c.dtype == torch.float32:
            assert torch.allclose(out, ref[bi, :n], rtol=1e-5, atol=1e-6)
        else:
            assert torch.allclose(out.float(), ref[bi, :n].float(), rtol=2 ** -6, atol=2 ** -6)
        at += n
    # and bit for bit what the padded oracle computes there
    ypad = O.causal_conv1d_ref(x.transpose(1, 2), w, b, act, attention_mask=m).transpose(1, 2)
    at = 0
    for bi, n in enumerate(lens):
        assert_close_to_oracle(yp[0, at:at + n], ypad[bi, :n], f"sequence {bi}")
        at += n
