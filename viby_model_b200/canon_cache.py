"""Bookkeeping of the Canon decode states on a generation cache.

The reference hangs its Canon states on the Hugging Face ``Cache`` object it is given: one Python list per
Canon position, ``cache.canon_cache_a`` ... ``canon_cache_d``, indexed by layer, created on first use with
``getattr(cache, "_max_layers", 256)`` slots (model/model.py:227-241), and for the circular state of its Metal
branch a parallel list ``<name>_seqlens`` of int32 positions (model/model.py:243-259).  Beam search reorders
every entry along the batch dimension (model/model.py:1330-1366) and the evaluation script moves them to another
device (eval_model.py:41-54).

The states this package's kernels update are plain ``[batch, dim, state_len]`` tensors, changed in place, so all
of that is index and attribute work on the host; these helpers do it for any object that allows attributes (a
``Cache``, a ``types.SimpleNamespace``).  They hold no state of their own and launch nothing themselves.
"""
from __future__ import annotations

from typing import Iterable, Iterator, Optional, Tuple

import torch

CANON_POSITIONS = ("a", "b", "c", "d")
_PREFIX = "canon_cache_"
_SEQLENS = "_seqlens"


def cache_name(position: str) -> str:
    """Attribute name of one Canon position's list: ``"a"`` -> ``"canon_cache_a"`` (names given in full pass)."""
    return position if position.startswith(_PREFIX) else _PREFIX + position


def _slots(cache, name: str) -> list:
    slots = getattr(cache, name, None)
    if slots is None:
        slots = [None] * int(getattr(cache, "_max_layers", 256))
        setattr(cache, name, slots)
    return slots


def get_state(cache, position: str, layer_idx: int) -> Optional[torch.Tensor]:
    """The state of one layer's Canon position, or None before its prefill (model/model.py:227-232)."""
    return _slots(cache, cache_name(position))[layer_idx]


def set_state(cache, position: str, layer_idx: int, state: Optional[torch.Tensor]) -> None:
    """Stores the state a prefill returned (``return_final_states=True``), model/model.py:234-241."""
    _slots(cache, cache_name(position))[layer_idx] = state


def get_seqlens(cache, position: str, layer_idx: int) -> Optional[torch.Tensor]:
    """Write positions of the circular state (``cache_seqlens`` of causal_conv1d_update), model/model.py:243-249."""
    return _slots(cache, cache_name(position) + _SEQLENS)[layer_idx]


def set_seqlens(cache, position: str, layer_idx: int, seqlens: Optional[torch.Tensor]) -> None:
    _slots(cache, cache_name(position) + _SEQLENS)[layer_idx] = seqlens


def _canon_lists(cache) -> Iterator[Tuple[str, list]]:
    for name, value in list(vars(cache).items()) if hasattr(cache, "__dict__") else []:
        if name.startswith(_PREFIX) and isinstance(value, list):
            yield name, value


def reorder(cache, beam_idx: torch.Tensor):
    """Beam search: row ``i`` of every Canon state (and of every seqlens vector) becomes row ``beam_idx[i]``
    (model/model.py:1340-1364).  The entries are replaced by new tensors, as ``index_select`` makes them;
    the key/value part of the cache is the cache's own business (``cache.reorder_cache``).  Returns the cache."""
    if cache is None:
        return None
    for _, slots in _canon_lists(cache):
        for i, entry in enumerate(slots):
            if entry is not None:
                slots[i] = entry.index_select(0, beam_idx.to(entry.device))
    return cache


def to_device(cache, device, into=None):
    """Moves every Canon state and seqlens vector to ``device`` (eval_model.py:41-54).  With ``into`` (a fresh
    cache object, as the reference builds one for the key/value tensors) the moved lists are set on that object
    and ``cache`` keeps its own; otherwise ``cache`` is changed in place.  Returns the object that holds the
    moved states."""
    if cache is None:
        return None
    target = cache if into is None else into
    for name, slots in _canon_lists(cache):
        setattr(target, name, [None if entry is None else entry.to(device) for entry in slots])
    if into is not None and hasattr(cache, "_max_layers"):
        target._max_layers = cache._max_layers
    return target


def states(cache, positions: Iterable[str] = CANON_POSITIONS) -> Iterator[Tuple[str, int, torch.Tensor]]:
    """Every stored state as ``(position name, layer, tensor)``: what a decode step over several independent
    requests hands to ``UpdateTable`` (one table entry per state)."""
    for position in positions:
        name = cache_name(position)
        for layer_idx, entry in enumerate(getattr(cache, name, None) or []):
            if entry is not None:
                yield name, layer_idx, entry
