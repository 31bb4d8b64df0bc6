"""The second API surface of the reference: the ``[B, T, D]`` operators of causal-conv1d-mps
(causal_conv1d_mps/__init__.py:81-419), here backed by the same CUDA kernels.

  causal_conv1d_fwd(x[B,D,T], weight, bias, silu_activation)                 __init__.py:81-151
  short_conv_fused(x[B,T,D], weight, bias, attention_mask, activation, residual)   :154-301
  short_conv_update(x[B,D], conv_state[B,D,S], weight, bias, cache_seqlens, activation, residual)  :304-419

Argument meaning, validation order and error messages follow the reference; device checks ask
for CUDA instead of MPS.  Two documented differences in arithmetic: the residual is added with
the two roundings of ``x + y`` (the Metal kernel adds in fp32 and rounds once,
causal_conv1d.metal:334-336), and widths 2 and 3 are accepted besides 4.
"""
from __future__ import annotations

from typing import Optional

import torch

from .ops import causal_conv1d_fn, causal_conv1d_update


def _check_cuda(t: Optional[torch.Tensor], what: str) -> None:
    if t is not None and t.device.type != "cuda":
        raise ValueError(f"{what} must be on CUDA device")


def causal_conv1d_fwd(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                      silu_activation: bool = False) -> torch.Tensor:
    """Causal conv over ``x[batch, dim, seqlen]``; returns a contiguous ``[batch, dim, seqlen]`` tensor."""
    if x.dim() != 3:
        raise ValueError(f"Expected 3D input tensor (batch, dim, seqlen), got {x.dim()}D")
    if weight.dim() != 2:
        raise ValueError(f"Expected 2D weight tensor (dim, width), got {weight.dim()}D")
    dim = x.shape[1]
    if dim != weight.shape[0]:
        raise ValueError(f"Input dim {dim} does not match weight dim {weight.shape[0]}")
    if bias is not None:
        if bias.dim() != 1:
            raise ValueError(f"Expected 1D bias tensor, got {bias.dim()}D")
        if bias.shape[0] != dim:
            raise ValueError(f"Bias dim {bias.shape[0]} does not match input dim {dim}")
    _check_cuda(x, "Input tensor")
    _check_cuda(weight, "Weight tensor")
    _check_cuda(bias, "Bias tensor")
    return causal_conv1d_fn(x.contiguous(), weight, bias, activation="silu" if silu_activation else None)


def short_conv_fused(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                     attention_mask: Optional[torch.Tensor] = None, activation: bool = True,
                     residual: bool = True) -> torch.Tensor:
    """Whole Canon layer in one launch over ``x[batch, seqlen, dim]``: mask, conv, SiLU, residual.

    The residual is the UNMASKED input, as in the reference's fused kernel
    (causal_conv1d.metal:334-336) and in CanonLayer's CUDA branch (model/model.py:491).
    """
    if x.dim() != 3:
        raise ValueError(f"Expected 3D input tensor (batch, seqlen, dim), got {x.dim()}D")
    if weight.dim() != 2:
        raise ValueError(f"Expected 2D weight tensor (dim, width), got {weight.dim()}D")
    B, T, D = x.shape
    if D != weight.shape[0]:
        raise ValueError(f"Input dim {D} does not match weight dim {weight.shape[0]}")
    if bias is not None:
        if bias.dim() != 1:
            raise ValueError(f"Expected 1D bias tensor, got {bias.dim()}D")
        if bias.shape[0] != D:
            raise ValueError(f"Bias dim {bias.shape[0]} does not match input dim {D}")
    if attention_mask is not None:
        if attention_mask.dim() != 2:
            raise ValueError(f"Expected 2D attention mask, got {attention_mask.dim()}D")
        if tuple(attention_mask.shape) != (B, T):
            raise ValueError(
                f"Attention mask shape {attention_mask.shape} does not match input shape ({B}, {T})"
            )
    _check_cuda(x, "Input tensor")
    _check_cuda(weight, "Weight tensor")
    _check_cuda(bias, "Bias tensor")
    _check_cuda(attention_mask, "Attention mask")
    x = x.contiguous()
    # (the reference goes on to squeeze / broadcast / transpose other mask shapes, __init__.py:238-293, but its
    # own check above, :215-221, lets nothing but [batch, seqlen] through: that code is unreachable and has
    # no counterpart here)
    m = attention_mask
    y = causal_conv1d_fn(x.transpose(1, 2), weight, bias, activation="silu" if activation else None,
                         attention_mask=m, residual=True if residual else None)
    return y.transpose(1, 2)


def short_conv_update(x: torch.Tensor, conv_state: torch.Tensor, weight: torch.Tensor,
                      bias: Optional[torch.Tensor] = None, cache_seqlens: Optional[torch.Tensor] = None,
                      activation: bool = True, residual: bool = True) -> torch.Tensor:
    """Single-token step on the circular ``conv_state[batch, dim, state_len]`` (updated in place):
    the token is written at ``cache_seqlens[b] % state_len`` and the W-1 slots before it are the
    history (causal_conv1d.metal:586-664).  Without ``cache_seqlens`` the reference substitutes
    ``arange(batch)`` (__init__.py:376-380); so does this function."""
    if x.dim() != 2:
        raise ValueError(f"Expected 2D input tensor (batch, dim), got {x.dim()}D")
    if conv_state.dim() != 3:
        raise ValueError(f"Expected 3D conv_state tensor (batch, dim, state_len), got {conv_state.dim()}D")
    if weight.dim() != 2:
        raise ValueError(f"Expected 2D weight tensor (dim, width), got {weight.dim()}D")
    batch, dim = x.shape
    if batch != conv_state.shape[0] or dim != conv_state.shape[1]:
        raise ValueError(
            f"Input shape {x.shape} doesn't match conv_state batch/dim {(conv_state.shape[0], conv_state.shape[1])}"
        )
    if dim != weight.shape[0]:
        raise ValueError(f"Input dim {dim} does not match weight dim {weight.shape[0]}")
    _check_cuda(x, "Input tensor")
    _check_cuda(conv_state, "Convolution state tensor")
    _check_cuda(weight, "Weight tensor")
    _check_cuda(bias, "Bias tensor")
    if cache_seqlens is None:
        cache_seqlens = torch.arange(batch, device=x.device, dtype=torch.int32)
    else:
        _check_cuda(cache_seqlens, "cache_seqlens")
        if cache_seqlens.dim() != 1:
            raise ValueError(f"Expected 1D cache_seqlens, got {cache_seqlens.dim()}D")
        if cache_seqlens.shape[0] != batch:
            raise ValueError(f"cache_seqlens batch size {cache_seqlens.shape[0]} != input batch {batch}")
    return causal_conv1d_update(x, conv_state, weight, bias, activation="silu" if activation else None,
                                cache_seqlens=cache_seqlens, residual=residual)
