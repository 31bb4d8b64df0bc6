"""Seeded synthetic inputs for the five benchmark / parity configurations.

Every sequence (batch row) is generated from its own seed ``base + 1000*cfg + b``, so any
sharding of the batch over GPUs reproduces exactly the same data.  Values follow the
configuration text: activations ~ N(0,1), weight and bias ~ U(-0.5, 0.5), generated in
fp32 and then cast to the I/O dtype.  Tensors are produced in the channel-contiguous
``[B, T, D]`` layout the Canon layers hold them in; the operators see ``x.transpose(1, 2)``.

Nothing here stands in for an external dataset: the configurations are synthetic by
definition.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

BASE_SEED = 20240


@dataclass(frozen=True)
class PrefillConfig:
    name: str
    cfg: int
    batch: int
    dim: int
    seqlen: int
    width: int
    dtype: torch.dtype
    activation: Optional[str]
    masked: bool
    len_lo: int = 0
    len_hi: int = 0
    len_dist: str = "uniform"  # "uniform" | "loguniform"


CANON_B_FP32 = PrefillConfig("canon_b_fp32", 1, 4, 960, 1024, 4, torch.float32, None, False)
CANON_D_PREFILL = PrefillConfig("canon_d_prefill_bf16", 2, 32, 3456, 1024, 4, torch.bfloat16, "silu", True, 128, 1024,
                                "uniform")
RAGGED_SWEEP = PrefillConfig("ragged_sweep_bf16", 5, 512, 3456, 4096, 4, torch.bfloat16, "silu", True, 16, 4096,
                             "loguniform")


@dataclass(frozen=True)
class DecodeConfig:
    name: str
    cfg: int
    batch: int
    dim: int
    width: int
    state_len: int
    prefill_len: int
    steps: int
    dtype: torch.dtype
    activation: Optional[str]


DECODE_CANON_B = DecodeConfig("decode_canon_b_bf16", 3, 256, 960, 4, 3, 512, 1024, torch.bfloat16, None)


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def weights(cfg_id: int, dim: int, width: int, dtype: torch.dtype, device="cpu", bias: bool = True):
    """weight [dim, width] and bias [dim] ~ U(-0.5, 0.5); always generated on the CPU."""
    g = _gen(BASE_SEED + 1000 * cfg_id + 999, "cpu")
    w = (torch.rand(dim, width, generator=g, dtype=torch.float32) - 0.5).to(dtype)
    b = (torch.rand(dim, generator=g, dtype=torch.float32) - 0.5).to(dtype) if bias else None
    return w.to(device), (b.to(device) if b is not None else None)


def sequence_lengths(cfg: PrefillConfig, rows: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Valid length of each sequence (int64, CPU).  Unmasked configs return seqlen everywhere."""
    rows = list(range(cfg.batch)) if rows is None else list(rows)
    out = torch.empty(len(rows), dtype=torch.int64)
    for i, b in enumerate(rows):
        if not cfg.masked:
            out[i] = cfg.seqlen
            continue
        g = _gen(BASE_SEED + 1000 * cfg.cfg + 500_000 + b, "cpu")
        u = float(torch.rand(1, generator=g))
        if cfg.len_dist == "loguniform":
            v = math.exp(math.log(cfg.len_lo) + u * (math.log(cfg.len_hi) - math.log(cfg.len_lo)))
            n = int(round(v))
        else:
            n = cfg.len_lo + int(u * (cfg.len_hi - cfg.len_lo + 1))
        out[i] = max(cfg.len_lo, min(cfg.len_hi, n))
    return out


def attention_mask(cfg: PrefillConfig, rows: Optional[Sequence[int]] = None, device="cpu",
                   dtype=torch.int64) -> Optional[torch.Tensor]:
    """Right-padded [rows, seqlen] mask (1 = valid) or None for unmasked configs."""
    if not cfg.masked:
        return None
    lens = sequence_lengths(cfg, rows)
    t = torch.arange(cfg.seqlen)
    return (t[None, :] < lens[:, None]).to(dtype).to(device)


def prefill_inputs(cfg: PrefillConfig, rows: Optional[Sequence[int]] = None, device="cpu",
                   generate_on: Optional[str] = None) -> torch.Tensor:
    """x [rows, seqlen, dim] ~ N(0,1) in cfg.dtype.

    ``generate_on="cpu"`` (default for CPU targets) draws from the CPU generator so CPU and GPU
    runs share bit-identical inputs; ``generate_on="cuda"`` draws on the GPU per sequence for
    workloads too large to synthesise on the host (the values then differ from the CPU stream
    but remain a pure function of the sequence index).
    """
    rows = list(range(cfg.batch)) if rows is None else list(rows)
    gen_dev = generate_on or "cpu"
    x = torch.empty(len(rows), cfg.seqlen, cfg.dim, dtype=cfg.dtype, device=device)
    for i, b in enumerate(rows):
        seed = BASE_SEED + 1000 * cfg.cfg + b
        if gen_dev == "cpu":
            v = torch.randn(cfg.seqlen, cfg.dim, generator=_gen(seed, "cpu"), dtype=torch.float32)
            x[i].copy_(v.to(cfg.dtype))
        else:
            v = torch.randn(cfg.seqlen, cfg.dim, generator=_gen(seed, device), dtype=torch.float32, device=device)
            x[i].copy_(v.to(cfg.dtype))
    return x


def decode_prefill(cfg: DecodeConfig, rows: Optional[Sequence[int]] = None, device="cpu") -> torch.Tensor:
    """The prefill tokens [rows, prefill_len, dim] that seed conv_state for the decode config."""
    rows = list(range(cfg.batch)) if rows is None else list(rows)
    x = torch.empty(len(rows), cfg.prefill_len, cfg.dim, dtype=cfg.dtype, device=device)
    for i, b in enumerate(rows):
        g = _gen(BASE_SEED + 1000 * cfg.cfg + b, "cpu")
        x[i].copy_(torch.randn(cfg.prefill_len, cfg.dim, generator=g, dtype=torch.float32).to(cfg.dtype))
    return x


def decode_tokens(cfg: DecodeConfig, rows: Optional[Sequence[int]] = None, device="cpu",
                  steps: Optional[int] = None) -> torch.Tensor:
    """x_t for every step: [steps, rows, dim] ~ N(0,1)."""
    rows = list(range(cfg.batch)) if rows is None else list(rows)
    steps = cfg.steps if steps is None else steps
    x = torch.empty(steps, len(rows), cfg.dim, dtype=cfg.dtype, device=device)
    for i, b in enumerate(rows):
        g = _gen(BASE_SEED + 1000 * cfg.cfg + 100_000 + b, "cpu")
        x[:, i].copy_(torch.randn(steps, cfg.dim, generator=g, dtype=torch.float32).to(cfg.dtype))
    return x


def shard_rows(batch: int, rank: int, world: int) -> range:
    """Contiguous, equal-count (+-1) slice of the batch owned by ``rank``."""
    base, rem = divmod(batch, world)
    start = rank * base + min(rank, rem)
    return range(start, start + base + (1 if rank < rem else 0))


# ---- algorithmic HBM bytes ----------------------------------------------------------------------
def prefill_bytes(batch: int, dim: int, seqlen: int, width: int, elem: int, valid_tokens: Optional[int] = None,
                  mask_bytes: int = 0, bias: bool = True) -> int:
    """Bytes one prefill launch has to move: x read (only valid rows when masked rows are
    skipped) + y written + weights/bias + mask."""
    read_tok = batch * seqlen if valid_tokens is None else valid_tokens
    return (read_tok + batch * seqlen) * dim * elem + dim * (width + (1 if bias else 0)) * elem + mask_bytes


def decode_bytes(batch: int, dim: int, width: int, state_len: int, elem: int, bias: bool = True) -> int:
    """Bytes of one decode step: x + state read, state + y written, weights/bias."""
    return batch * dim * elem * (2 + 2 * state_len) + dim * (width + (1 if bias else 0)) * elem
