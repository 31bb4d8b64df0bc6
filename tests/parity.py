"""Tolerances of the parity tests, in one place.

fp32 outputs:  |a - ref| <= 1e-5 * |ref| + 1e-6   (1e-5 relative; the absolute term covers
               cancellation, where two fp32 summation orders differ by ~1e-7 absolute).
bf16 outputs:  within 1 bf16 ulp of the fp32-accumulated, once-rounded oracle; elements whose
               fp32 values differ by less than 1e-6 absolute are accepted whatever the ulp
               count (results that straddle zero or a binade after cancellation).
fp16 outputs:  same rule with fp16 ulps.
conv_state:    bit-exact (torch.equal on the raw values).
"""
import torch


def _ordered_bits(t: torch.Tensor) -> torch.Tensor:
    bits = t.contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
    mag = bits & 0x7FFF
    return torch.where((bits >> 15) == 1, -mag, mag)


def ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    assert a.dtype == b.dtype and a.dtype in (torch.bfloat16, torch.float16)
    return (_ordered_bits(a) - _ordered_bits(b)).abs()


def assert_close_to_oracle(got: torch.Tensor, ref: torch.Tensor, what: str = "", max_ulp: int = 1):
    """got: kernel output (any device); ref: oracle output in the same dtype (CPU)."""
    got = got.detach().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert got.dtype == ref.dtype, f"{what}: dtype {got.dtype} vs {ref.dtype}"
    if got.numel() == 0:
        return
    if got.dtype == torch.float32:
        err = (got - ref).abs()
        tol = 1e-5 * ref.abs() + 1e-6
        bad = err > tol
        assert not bool(bad.any()), (
            f"{what}: {int(bad.sum())} of {got.numel()} fp32 elements outside 1e-5 rel + 1e-6 abs; "
            f"max abs err {float(err.max()):.3e}"
        )
        return
    ulp = ulp_distance(got, ref)
    err = (got.float() - ref.float()).abs()
    bad = (ulp > max_ulp) & (err > 1e-6)
    bad |= got.float().isnan() != ref.float().isnan()
    assert not bool(bad.any()), (
        f"{what}: {int(bad.sum())} of {got.numel()} elements differ by more than {max_ulp} ulp; "
        f"max ulp {int(ulp.max())}, max abs err {float(err.max()):.3e}"
    )


def exact_fraction(got: torch.Tensor, ref: torch.Tensor) -> float:
    got = got.detach().cpu()
    return float((got == ref).float().mean()) if got.numel() else 1.0
