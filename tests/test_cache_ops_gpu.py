"""Canon cache bookkeeping on states the kernels update in place.

The reference keeps one ``[B, D, L]`` state tensor per Canon layer on the HF cache object
(model/model.py:227-259), reorders them for beam search with ``index_select(0, beam_idx)``
(model/model.py:1340-1364) and moves them between devices with ``.to(device)``
(eval_model.py:41-54).  Between such operations the decode kernel must keep working on whatever
tensor it is handed -- a fresh copy, a host round trip, a non-contiguous view -- and stay
bit-equal to the oracle run on the same rows.
"""
import pytest
import torch

import viby_model_b200 as V
from oracle import canon_oracle as O
from parity import assert_close_to_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


def bits(t):
    return t.view(torch.int32 if t.dtype == torch.float32 else torch.int16)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("L", [3, 4, 8])
def test_beam_reorder_and_device_round_trip_between_decode_steps(L, dtype):
    B, T, D, W = 6, 40, 960, 4
    g = torch.Generator().manual_seed(90 + L)
    x = torch.randn(B, T, D, generator=g).to(dtype)
    w = (torch.rand(D, W, generator=g) - 0.5).to(dtype)
    b = (torch.rand(D, generator=g) - 0.5).to(dtype)
    lens = torch.tensor([T, 33, 5, 1, 17, T])
    m = (torch.arange(T)[None, :] < lens[:, None]).to(torch.int64)
    wd, bd = w.to(DEV), b.to(DEV)

    _, st = V.causal_conv1d_fn(x.to(DEV).transpose(1, 2), wd, bd, activation="silu", attention_mask=m.to(DEV),
                               return_final_states=True, state_len=L)
    _, ref_st = O.causal_conv1d_ref(x.transpose(1, 2), w, b, "silu", attention_mask=m, state_len=L)
    assert torch.equal(bits(st.cpu()), bits(ref_st))

    beams = [torch.tensor([0, 0, 2, 5, 5, 1]), torch.tensor([5, 4, 3, 2, 1, 0]), torch.tensor([1, 1, 1, 1, 1, 1])]
    for step in range(9):
        if step in (2, 5, 7):
            # beam search: a new tensor with rows gathered from the old one (model/model.py:1340-1364)
            idx = beams[(step // 2) % 3]
            st = st.index_select(0, idx.to(DEV))
            ref_st = ref_st.index_select(0, idx)
        if step == 4:
            # hybrid prefill / decode across devices: the state leaves the GPU and comes back (eval_model.py:41-54)
            st = st.to("cpu").to(DEV)
        if step == 6:
            # a state that is a view of a larger allocation: the batch stride is not D * L
            big = torch.zeros(B, 2, D, L, dtype=dtype, device=DEV)
            big[:, 1] = st
            st = big[:, 1]
            assert not st.is_contiguous()
        xt = torch.randn(B, D, generator=g).to(dtype)
        before = V.launch_count()
        y = V.causal_conv1d_update(xt.to(DEV), st, wd, bd, activation="silu")
        assert V.launch_count() == before + 1
        ref = O.causal_conv1d_update_ref(xt, ref_st, w, b, "silu")
        assert_close_to_oracle(y, ref, f"step {step}")
        assert torch.equal(bits(st.cpu()), bits(ref_st)), f"state after step {step}"


def test_reordered_circular_state_keeps_its_positions():
    """The circular state of causal-conv1d-mps travels with its cache_seqlens
    (model/model.py:1352-1364 reorders both lists)."""
    B, D, W, L = 4, 256, 4, 8
    g = torch.Generator().manual_seed(4)
    w = (torch.rand(D, W, generator=g) - 0.5).bfloat16()
    state = torch.randn(B, D, L, generator=g).bfloat16()
    seqlens = torch.tensor([0, 5, 9, 30], dtype=torch.int32)
    st, sl = state.to(DEV), seqlens.to(DEV)
    for step in range(6):
        if step == 3:
            idx = torch.tensor([3, 3, 0, 2])
            st, sl = st.index_select(0, idx.to(DEV)), sl.index_select(0, idx.to(DEV))
            state, seqlens = state.index_select(0, idx), seqlens.index_select(0, idx)
        xt = torch.randn(B, D, generator=g).bfloat16()
        y = V.causal_conv1d_update(xt.to(DEV), st, w.to(DEV), None, "silu", sl)
        ref = O.causal_conv1d_update_ref(xt, state, w, None, "silu", cache_seqlens=seqlens)
        assert_close_to_oracle(y, ref, f"step {step}")
        assert torch.equal(bits(st.cpu()), bits(state))
        sl, seqlens = sl + 1, seqlens + 1


def test_requests_decoded_side_by_side_from_their_caches():
    """Two independent requests, each with its own cache of Canon states (viby_model_b200.canon_cache): one
    table launch per token steps every state of both (UpdateTable), a beam reorder of one request in between;
    bit-equal to a causal_conv1d_update call per state, with the oracle as the arbiter of the first step."""
    import types

    from viby_model_b200 import canon_cache as CC

    dtype, W, L, layers = torch.bfloat16, 4, 4, 3
    dims = {"a": 640, "b": 960, "c": 640, "d": 3456}
    g = torch.Generator().manual_seed(77)
    weights = {(pos, l): (torch.rand(D, W, generator=g) - 0.5).to(dtype) for pos, D in dims.items() for l in range(layers)}
    requests = []
    for batch in (5, 2):
        cache, shadow = types.SimpleNamespace(_max_layers=layers), types.SimpleNamespace(_max_layers=layers)
        for pos, D in dims.items():
            for l in range(layers):
                s = torch.randn(batch, D, L, generator=g).to(dtype)
                CC.set_state(cache, pos, l, s.to(DEV))
                CC.set_state(shadow, pos, l, s.clone().to(DEV))
        requests.append((batch, cache, shadow))

    def build_table():
        xs, states, ws = [], [], []
        for batch, cache, _ in requests:
            for name, layer, state in CC.states(cache):
                xs.append(torch.zeros(batch, state.shape[1], dtype=dtype, device=DEV))
                states.append(state)
                ws.append(weights[(name[-1], layer)].to(DEV))
        return xs, V.UpdateTable(xs, states, ws, None, "silu")

    xs, table = build_table()
    assert len(table) == 2 * 4 * layers
    gen = torch.Generator(device=DEV).manual_seed(78)
    for step in range(4):
        if step == 2:
            # beam search picks other rows of the first request: the states are new tensors, so is the table
            beam = torch.tensor([4, 4, 0, 1, 2], device=DEV)
            CC.reorder(requests[0][1], beam)
            CC.reorder(requests[0][2], beam)
            xs, table = build_table()
        for x in xs:
            x.copy_(torch.randn(x.shape, generator=gen, device=DEV).to(dtype))
        before = V.launch_count()
        ys = table.launch()
        assert V.launch_count() == before + 1
        i = 0
        for batch, cache, shadow in requests:
            for name, layer, state in CC.states(cache):
                w = weights[(name[-1], layer)]
                twin = CC.get_state(shadow, name, layer)
                if step == 0:
                    cpu_state = twin.cpu().clone()
                    ref = O.causal_conv1d_update_ref(xs[i].cpu(), cpu_state, w, None, "silu")
                    assert_close_to_oracle(ys[i], ref, f"{name}[{layer}]")
                want = V.causal_conv1d_update(xs[i], twin, w.to(DEV), None, "silu")
                assert torch.equal(bits(ys[i]), bits(want)), (step, name, layer)
                assert torch.equal(bits(state), bits(twin)), (step, name, layer)
                i += 1
