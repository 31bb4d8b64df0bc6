"""Generate tests/golden/canon_bwd_golden.npz: gradients of the UNMODIFIED reference CanonLayer.

Usage:  python tests/golden/make_bwd_golden.py --reference <path to a Viby-Model checkout>

``model.model.CanonLayer`` is imported from the reference tree (its PyTorch branch runs, as neither
optional kernel package is installed), fed seeded inputs with requires_grad, and torch.autograd
differentiates ``sum(layer(x, mask) * dy)``.  Recorded per case: x, weight, bias, mask, dy and the
gradients dx, dweight, dbias.  Nothing of the reference is copied; only numbers are stored (bf16 as
uint16 bit patterns).  In that branch the residual adds the MASKED input (model/model.py:595-602,
675), which the oracle reproduces with ``residual_masked=True``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import numpy as np
import torch

OUT = Path(__file__).resolve().parent / "canon_bwd_golden.npz"
sys.path.insert(0, str(Path(__file__).resolve().parent))
from make_golden import make_mask, to_np  # noqa: E402


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

    arrays, meta = {}, []
    specs = []
    for dtype in (torch.float32, torch.bfloat16):
        for (B, T, D) in ((2, 1, 8), (2, 3, 8), (2, 9, 24), (3, 16, 24), (2, 37, 16)):
            for mask_kind in ("none", "right", "holes"):
                specs.append((dtype, B, T, D, 4, True, True, mask_kind))
            if T < 9:
                continue
            for has_bias, act in ((False, False), (True, False), (False, True)):
                specs.append((dtype, B, T, D, 4, has_bias, act, "right"))
            for K in (2, 3):
                specs.append((dtype, B, T, D, K, True, True, "left"))

    for cid, (dtype, B, T, D, K, has_bias, act, mask_kind) in enumerate(specs):
        seed = 5000 + cid
        g = torch.Generator().manual_seed(seed)
        cfg = VibyConfig(canon_kernel=K, canon_bias=has_bias, canon_activation=act)
        layer = CanonLayer(D, cfg, "a")
        with torch.no_grad():
            layer.weight.copy_(torch.rand(D, 1, K, generator=g) - 0.5)
            if has_bias:
                layer.bias_param.copy_(torch.rand(D, generator=g) - 0.5)
        layer = layer.to(dtype)
        x = torch.randn(B, T, D, generator=g).to(dtype).requires_grad_(True)
        dy = torch.randn(B, T, D, generator=g).to(dtype)
        mask = make_mask(mask_kind, B, T, g)
        out = layer(x, attention_mask=mask)
        (out.float() * dy.float()).sum().backward()
        name = f"g{cid:03d}"
        arrays[f"{name}.x"] = to_np(x)
        arrays[f"{name}.dy"] = to_np(dy)
        arrays[f"{name}.weight"] = to_np(layer.weight.squeeze(1))
        arrays[f"{name}.dx"] = to_np(x.grad)
        arrays[f"{name}.dweight"] = to_np(layer.weight.grad.squeeze(1))
        if has_bias:
            arrays[f"{name}.bias"] = to_np(layer.bias_param)
            arrays[f"{name}.dbias"] = to_np(layer.bias_param.grad)
        if mask is not None:
            arrays[f"{name}.mask"] = mask.numpy().copy()
        meta.append(dict(name=name, dtype=str(dtype).replace("torch.", ""), B=B, T=T, D=D, K=K,
                         bias=has_bias, activation=act, mask=mask_kind, seed=seed))

    arrays["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(OUT, **arrays)
    print(f"wrote {OUT} ({OUT.stat().st_size / 1024:.0f} KB, {len(meta)} cases, torch {torch.__version__})")


if __name__ == "__main__":
    main()
