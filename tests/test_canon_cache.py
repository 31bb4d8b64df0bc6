"""Host-side bookkeeping of the Canon decode states on a generation cache (viby_model_b200/canon_cache.py)
against the behaviour of the reference's accessors (model/model.py:227-259), beam reorder
(model/model.py:1330-1366) and device transfer (eval_model.py:41-54).  CPU tensors; no kernel runs."""
import types

import torch

from viby_model_b200 import canon_cache as CC


def _cache_with_states(layers=3, batch=4):
    cache = types.SimpleNamespace(_max_layers=layers + 2)
    g = torch.Generator().manual_seed(5)
    for k, pos in enumerate(CC.CANON_POSITIONS):
        for layer in range(layers):
            if (layer + k) % 3 == 2:
                continue  # some layers have not been prefilled yet
            CC.set_state(cache, pos, layer, torch.randn(batch, 8 + k, 4, generator=g))
    CC.set_seqlens(cache, "a", 0, torch.arange(batch, dtype=torch.int32))
    return cache


def test_accessors_create_the_lists_the_reference_creates():
    cache = types.SimpleNamespace()
    assert CC.get_state(cache, "b", 7) is None
    assert isinstance(cache.canon_cache_b, list) and len(cache.canon_cache_b) == 256  # the reference's default
    small = types.SimpleNamespace(_max_layers=5)
    s = torch.zeros(2, 3, 4)
    CC.set_state(small, "canon_cache_d", 4, s)  # full attribute names pass too
    assert len(small.canon_cache_d) == 5 and CC.get_state(small, "d", 4) is s
    assert CC.get_seqlens(small, "d", 4) is None and len(small.canon_cache_d_seqlens) == 5
    v = torch.zeros(2, dtype=torch.int32)
    CC.set_seqlens(small, "d", 4, v)
    assert small.canon_cache_d_seqlens[4] is v


def test_reorder_selects_rows_of_every_state_and_seqlens():
    cache = _cache_with_states()
    before = {(n, i): t.clone() for n, i, t in CC.states(cache)}
    lens_before = cache.canon_cache_a_seqlens[0].clone()
    empty_before = [[e is None for e in getattr(cache, CC.cache_name(p))] for p in CC.CANON_POSITIONS]
    beam = torch.tensor([2, 2, 0, 1])
    out = CC.reorder(cache, beam)
    assert out is cache
    assert len(before) == sum(1 for _ in CC.states(cache))
    for name, layer, t in CC.states(cache):
        assert torch.equal(t, before[(name, layer)].index_select(0, beam))
    assert torch.equal(cache.canon_cache_a_seqlens[0], lens_before.index_select(0, beam))
    assert empty_before == [[e is None for e in getattr(cache, CC.cache_name(p))] for p in CC.CANON_POSITIONS]  # empty slots stay empty
    assert CC.reorder(None, beam) is None


def test_to_device_in_place_and_into_a_fresh_cache():
    cache = _cache_with_states()
    want = {(n, i): t.clone() for n, i, t in CC.states(cache)}
    fresh = types.SimpleNamespace()
    moved = CC.to_device(cache, torch.device("cpu"), into=fresh)
    assert moved is fresh and fresh._max_layers == cache._max_layers
    assert {(n, i) for n, i, _ in CC.states(fresh)} == set(want)
    for n, i, t in CC.states(fresh):
        assert torch.equal(t, want[(n, i)])
    assert torch.equal(fresh.canon_cache_a_seqlens[0], cache.canon_cache_a_seqlens[0])
    assert len(fresh.canon_cache_c) == len(cache.canon_cache_c)
    same = CC.to_device(cache, "cpu")
    assert same is cache
    assert CC.to_device(None, "cpu") is None


def test_against_the_reference_functions_when_a_checkout_is_present():
    """The reference's own `_reorder_cache` on a cache filled through these helpers gives what `reorder` gives."""
    import importlib
    import os
    import sys
    from pathlib import Path

    import pytest

    roots = [os.environ.get("VIBY_REFERENCE"), "/root/reference", str(Path(__file__).resolve().parents[1] / "baseline" / "_ref")]
    root = next((r for r in roots if r and (Path(r) / "model" / "model.py").exists()), None)
    if root is None:
        pytest.skip("no reference checkout on this machine")
    sys.path.insert(0, root)
    sys.dont_write_bytecode = True
    try:
        model = importlib.import_module("model.model")
    finally:
        sys.path.remove(root)
    a, b = _cache_with_states(), _cache_with_states()
    beam = torch.tensor([3, 1, 1, 0])
    model.VibyForCausalLM._reorder_cache(None, a, beam)
    CC.reorder(b, beam)
    got = {(n, i): t for n, i, t in CC.states(b)}
    for n, i, t in CC.states(a):
        assert torch.equal(t, got[(n, i)])
    assert torch.equal(a.canon_cache_a_seqlens[0], b.canon_cache_a_seqlens[0])
