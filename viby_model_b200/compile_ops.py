"""torch.library registration of the operators, so that ``torch.compile(fullgraph=True)`` (how the
reference compiles its model for evaluation, eval_model.py:157) can trace a model that calls
``causal_conv1d_fn`` / ``causal_conv1d_update``: each becomes one opaque node of the graph, with a
shape function (``register_fake``) and a backward formula (``register_autograd``).

The eager entry points keep calling the C ABI directly (a decode step is launch-bound and the
dispatcher costs more than the launch); ``ops.py`` switches to these custom ops only while
``torch.compiler.is_compiling()``.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import ops

_ACT = {0: None, 1: "silu"}


@torch.library.custom_op("vc1d::prefill", mutates_args=(), device_types="cuda")
def prefill(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], mask: Optional[torch.Tensor],
            residual: Optional[torch.Tensor], initial_states: Optional[torch.Tensor], activation: int,
            residual_is_x: bool, skip_masked_loads: bool, state_len: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """y (and, when state_len > 0, the final state) of causal_conv1d_fn."""
    res = True if residual_is_x else residual
    out = ops._prefill_forward(x, weight, bias, None, initial_states, state_len > 0, None, _ACT[activation],
                               attention_mask=mask, skip_masked_loads=skip_masked_loads, residual=res,
                               state_len=state_len if state_len > 0 else None)
    if state_len > 0:
        return out[0], out[1]
    return out, x.new_empty(0)


@prefill.register_fake
def _(x, weight, bias, mask, residual, initial_states, activation, residual_is_x, skip_masked_loads, state_len):
    y = torch.empty_strided(x.shape, x.stride(), dtype=x.dtype, device=x.device)
    state = x.new_empty((x.shape[0], x.shape[1], state_len)) if state_len > 0 else x.new_empty(0)
    return y, state


@torch.library.custom_op("vc1d::prefill_bwd", mutates_args=(), device_types="cuda")
def prefill_bwd(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], dy: torch.Tensor,
                mask: Optional[torch.Tensor], activation: int, residual_is_x: bool
                ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    dx, dw, db = ops.causal_conv1d_bwd(x, weight, bias, dy, _ACT[activation], attention_mask=mask,
                                       residual=residual_is_x)
    # the eager op returns dweight and dbias as views of one buffer; outputs of a custom op must not alias
    return dx, dw.clone(), db.clone() if db is not None else x.new_empty(0, dtype=torch.float32)


@prefill_bwd.register_fake
def _(x, weight, bias, dy, mask, activation, residual_is_x):
    dx = torch.empty_strided(x.shape, x.stride(), dtype=x.dtype, device=x.device)
    dw = x.new_empty(weight.shape, dtype=torch.float32)
    db = x.new_empty((weight.shape[0],) if bias is not None else (0,), dtype=torch.float32)
    return dx, dw, db


def _prefill_setup(ctx, inputs, output):
    x, weight, bias, mask, residual, initial_states, activation, residual_is_x, _skip, _state_len = inputs
    if initial_states is not None:
        raise NotImplementedError("backward with initial_states is not supported")
    ctx.save_for_backward(x, weight, bias, mask)
    ctx.activation = activation
    ctx.residual_is_x = residual_is_x
    ctx.has_res_tensor = residual is not None


def _prefill_backward(ctx, dy, _dstate):
    x, weight, bias, mask = ctx.saved_tensors
    dx, dw, db = torch.ops.vc1d.prefill_bwd(x, weight, bias, dy, mask, ctx.activation, ctx.residual_is_x)
    return (dx, dw.to(weight.dtype), db.to(bias.dtype) if bias is not None else None, None,
            dy if ctx.has_res_tensor else None, None, None, None, None, None)


torch.library.register_autograd("vc1d::prefill", _prefill_backward, setup_context=_prefill_setup)


@torch.library.custom_op("vc1d::update", mutates_args=("conv_state",), device_types="cuda")
def update(x: torch.Tensor, conv_state: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
           cache_seqlens: Optional[torch.Tensor], activation: int, residual: bool) -> torch.Tensor:
    """y of causal_conv1d_update; conv_state is updated in place.  Forward only."""
    return ops._update_forward(x, conv_state, weight, bias, _ACT[activation], cache_seqlens, residual=residual)


@update.register_fake
def _(x, conv_state, weight, bias, cache_seqlens, activation, residual):
    return torch.empty_like(x)
