"""Generate tests/golden/canon_golden.npz from the UNMODIFIED reference implementation.

Usage:  python tests/golden/make_golden.py --reference <path to a Viby-Model checkout>

The script imports ``model.model.CanonLayer`` from the reference tree (neither optional
kernel package is installed, so its PyTorch branch runs: model/model.py:587-675 and
372-398), feeds it seeded inputs and records inputs and outputs.  Nothing of the reference
is copied; only numbers are stored.  bf16 tensors are stored as their uint16 bit patterns, with
the dtype recorded in the case's metadata.

Cases (all small; the whole file is a few hundred KB):
  prefill        no cache: out = layer(x, attention_mask)
  prefill_cache  with a cache object: also the conv_state left behind (state_len 8)
  decode         prefill_cache followed by N single-token steps: every output and state
  chunked        prefill_cache followed by a multi-token continuation (history path)
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import numpy as np
import torch

OUT = Path(__file__).resolve().parent / "canon_golden.npz"


class FakeCache:
    """CanonLayer only does hasattr/getattr/setattr on the cache (model/model.py:227-259)."""


def to_np(t: torch.Tensor) -> np.ndarray:
    t = t.detach()
    if t.dtype == torch.bfloat16:  # bit patterns, half the bytes of float32
        return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()
    return t.float().numpy().copy()


def make_mask(kind: str, B: int, T: int, g: torch.Generator):
    if kind == "none":
        return None
    m = torch.ones(B, T, dtype=torch.int64)
    if kind == "right":  # right padding, valid length in [T/2, T) as causal-conv1d-mps/test.py:177-180
        for b in range(B):
            valid = int(torch.randint(max(T // 2, 1), max(T, 2), (1,), generator=g))
            m[b, valid:] = 0
    elif kind == "left":
        for b in range(B):
            pad = int(torch.randint(0, max(T // 2, 1), (1,), generator=g))
            m[b, :pad] = 0
    elif kind == "holes":
        m = (torch.rand(B, T, generator=g) > 0.3).to(torch.int64)
    return m


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    os.environ["PYTHONDONTWRITEBYTECODE"] = "1"
    sys.dont_write_bytecode = True
    sys.path.insert(0, args.reference)
    from model.model import CanonLayer, VibyConfig  # noqa: E402  (the reference, unmodified)
    import model.model as ref_model

    assert not ref_model.HAS_CAUSAL_CONV1D_CUDA and not ref_model.HAS_CAUSAL_CONV1D_MPS

    arrays = {}
    meta = []

    def layer_for(D, K, has_bias, act, dtype, seed):
        cfg = VibyConfig(canon_kernel=K, canon_bias=has_bias, canon_activation=act)
        layer = CanonLayer(D, cfg, "a")
        g = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            layer.weight.copy_(torch.rand(D, 1, K, generator=g) - 0.5)
            if has_bias:
                layer.bias_param.copy_(torch.rand(D, generator=g) - 0.5)
        return layer.to(dtype).eval()

    cid = 0
    specs = []
    rich = ((2, 5, 24), (3, 16, 24))
    for dtype in (torch.float32, torch.bfloat16):
        for (B, T, D) in ((2, 1, 8), (2, 3, 8), (2, 5, 24), (3, 16, 24), (2, 37, 16)):
            for mask_kind in ("none", "right"):
                specs.append((dtype, B, T, D, 4, True, True, mask_kind))
            if (B, T, D) not in rich:
                continue
            for has_bias, act in ((False, False), (True, False), (False, True)):
                specs.append((dtype, B, T, D, 4, has_bias, act, "none"))
            for mask_kind in ("left", "holes"):
                specs.append((dtype, B, T, D, 4, True, True, mask_kind))
            for K in (2, 3):
                for mask_kind in ("none", "right"):
                    specs.append((dtype, B, T, D, K, True, True, mask_kind))

    with torch.no_grad():
        for (dtype, B, T, D, K, has_bias, act, mask_kind) in specs:
            seed = 1000 + cid
            g = torch.Generator().manual_seed(seed)
            layer = layer_for(D, K, has_bias, act, dtype, seed + 7)
            x = torch.randn(B, T, D, generator=g).to(dtype)
            mask = make_mask(mask_kind, B, T, g)
            name = f"c{cid:03d}"
            arrays[f"{name}.x"] = to_np(x)
            arrays[f"{name}.weight"] = to_np(layer.weight.squeeze(1))
            if has_bias:
                arrays[f"{name}.bias"] = to_np(layer.bias_param)
            if mask is not None:
                arrays[f"{name}.mask"] = mask.numpy().copy()

            # prefill without cache
            out = layer(x, attention_mask=mask)
            arrays[f"{name}.prefill_out"] = to_np(out)

            # prefill with cache, then decode steps
            cache = FakeCache()
            out_c = layer(x, attention_mask=mask, cache=cache, layer_idx=0)
            state = cache.canon_cache_a[0]
            arrays[f"{name}.prefill_cache_out"] = to_np(out_c)
            arrays[f"{name}.prefill_state"] = to_np(state)
            n_steps = 6
            xs = torch.randn(n_steps, B, 1, D, generator=g).to(dtype)
            outs, states = [], []
            for s in range(n_steps):
                o = layer(xs[s], attention_mask=None, cache=cache, layer_idx=0)
                outs.append(to_np(o))
                states.append(to_np(cache.canon_cache_a[0]))
            arrays[f"{name}.decode_x"] = to_np(xs)
            arrays[f"{name}.decode_out"] = np.stack(outs)
            arrays[f"{name}.decode_state"] = np.stack(states)

            # chunked continuation on a fresh cache: prefill, then a 5-token and a 12-token chunk
            cache2 = FakeCache()
            layer(x, attention_mask=mask, cache=cache2, layer_idx=0)
            for tag, Tc in (("chunk5", 5), ("chunk12", 12)):
                xc = torch.randn(B, Tc, D, generator=g).to(dtype)
                oc = layer(xc, attention_mask=None, cache=cache2, layer_idx=0)
                arrays[f"{name}.{tag}_x"] = to_np(xc)
                arrays[f"{name}.{tag}_out"] = to_np(oc)
                arrays[f"{name}.{tag}_state"] = to_np(cache2.canon_cache_a[0])

            meta.append(
                dict(name=name, dtype=str(dtype).replace("torch.", ""), B=B, T=T, D=D, K=K,
                     bias=has_bias, activation=act, mask=mask_kind, seed=seed)
            )
            cid += 1

    arrays["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(OUT, **arrays)
    print(f"wrote {OUT} ({OUT.stat().st_size / 1024:.0f} KB, {len(meta)} cases, torch {torch.__version__})")


if __name__ == "__main__":
    main()
