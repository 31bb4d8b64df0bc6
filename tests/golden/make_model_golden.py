"""Generate tests/golden/viby_tiny.npz: a tiny Viby model from the UNMODIFIED reference
(weights, inputs, logits of a prefill and of three cached decode steps, on CPU, fp32).

Usage:  python tests/golden/make_model_golden.py --reference <path to a Viby-Model checkout>

Only numbers are stored.  tests/test_model_harness.py checks that tests/viby_harness.py (written
from scratch) reproduces them, which pins the harness that the whole-model GPU test relies on.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import numpy as np
import torch

OUT = Path(__file__).resolve().parent / "viby_tiny.npz"
CFG = dict(hidden_size=32, intermediate_size=48, num_attention_heads=4, num_key_value_heads=1, num_hidden_layers=6,
           vocab_size=64, rms_norm_eps=1e-6, rope_theta=1e6, sliding_window=4, canon_kernel=4, canon_bias=True,
           canon_activation=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    os.environ["PYTHONDONTWRITEBYTECODE"] = "1"
    sys.dont_write_bytecode = True
    sys.path.insert(0, args.reference)
    from model.model import VibyConfig, VibyForCausalLM  # the reference, unmodified

    torch.manual_seed(1234)
    model = VibyForCausalLM(VibyConfig(max_position_embeddings=256, **CFG)).eval()
    g = torch.Generator().manual_seed(99)
    with torch.no_grad():
        for name, prm in model.named_parameters():
            prm.copy_(torch.randn(prm.shape, generator=g) * (0.3 if "canon" in name or "sinks" in name else 0.15))
    B, T = 2, 12
    ids = torch.randint(0, CFG["vocab_size"], (B, T), generator=g)
    mask = torch.ones(B, T, dtype=torch.int64)
    mask[1, 9:] = 0  # right padding on the second sequence
    arrays = {k: v.detach().numpy().copy() for k, v in model.state_dict().items() if k != "lm_head.weight"}
    arrays["ids"] = ids.numpy()
    arrays["mask"] = mask.numpy()
    with torch.no_grad():
        out = model(input_ids=ids, attention_mask=mask, use_cache=True)
        arrays["logits_prefill"] = out.logits.numpy().copy()
        nocache = model(input_ids=ids, attention_mask=mask, use_cache=False)
        arrays["logits_nocache"] = nocache.logits.numpy().copy()
        past = out.past_key_values
        cur_mask = mask
        for s in range(3):
            nxt = torch.randint(0, CFG["vocab_size"], (B, 1), generator=g)
            cur_mask = torch.cat([cur_mask, torch.ones(B, 1, dtype=torch.int64)], 1)
            o = model(input_ids=nxt, attention_mask=cur_mask, past_key_values=past, use_cache=True)
            past = o.past_key_values
            arrays[f"decode_ids_{s}"] = nxt.numpy()
            arrays[f"decode_logits_{s}"] = o.logits.numpy().copy()
    arrays["cfg"] = np.frombuffer(json.dumps(CFG).encode(), dtype=np.uint8)
    np.savez_compressed(OUT, **arrays)
    print(f"wrote {OUT} ({OUT.stat().st_size / 1024:.0f} KB)")


if __name__ == "__main__":
    main()
