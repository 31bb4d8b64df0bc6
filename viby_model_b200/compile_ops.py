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
    with ops.fresh_scratch():
        out = ops._prefill_forward(x, weight, bias, None, initial_states, state_len > 0, None, _ACT[activation],
                                   attention_mask=mask, skip_masked_loads=skip_masked_loads, residual=res,
                                   state_len=state_len if state_len > 0 else None)
    if state_len > 0:
        return out[0], out[1]
    return out, x.new_empty(0)


@prefill.register_fake
def _(x, weight, bias, mask, residual, initial_states, activation, residual_is_x, skip_masked_loads, state_len):
    y = torch.empty_like(x)  # what the launch wrapper allocates: x's strides when x is dense, else a dense layout
    state = x.new_empty((x.shape[0], x.shape[1], state_len)) if state_len > 0 else x.new_empty(0)
    return y, state


@torch.library.custom_op("vc1d::prefill_bwd", mutates_args=(), device_types="cuda")
def prefill_bwd(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], dy: torch.Tensor,
                mask: Optional[torch.Tensor], initial_states: Optional[torch.Tensor], activation: int,
                residual_is_x: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    with ops.fresh_scratch():
        grads = ops.causal_conv1d_bwd(x, weight, bias, dy, _ACT[activation], attention_mask=mask,
                                      residual=residual_is_x, initial_states=initial_states)
    dx, dw, db = grads[0], grads[1], grads[2]
    dinit = grads[3] if initial_states is not None else x.new_empty(0)
    # the eager op returns dweight and dbias as views of one buffer; outputs of a custom op must not alias
    return dx, dw.clone(), db.clone() if db is not None else x.new_empty(0, dtype=torch.float32), dinit


@prefill_bwd.register_fake
def _(x, weight, bias, dy, mask, initial_states, activation, residual_is_x):
    dx = torch.empty_strided(x.shape, x.stride(), dtype=x.dtype, device=x.device)
    dw = x.new_empty(weight.shape, dtype=torch.float32)
    db = x.new_empty((weight.shape[0],) if bias is not None else (0,), dtype=torch.float32)
    dinit = torch.empty_like(initial_states.contiguous()) if initial_states is not None else x.new_empty(0)
    return dx, dw, db, dinit


def _prefill_setup(ctx, inputs, output):
    x, weight, bias, mask, residual, initial_states, activation, residual_is_x, _skip, _state_len = inputs
    ctx.save_for_backward(x, weight, bias, mask, initial_states)
    ctx.activation = activation
    ctx.residual_is_x = residual_is_x
    ctx.has_res_tensor = residual is not None


def _prefill_backward(ctx, dy, dstate):
    x, weight, bias, mask, init = ctx.saved_tensors
    dx, dw, db, dinit = torch.ops.vc1d.prefill_bwd(x, weight, bias, dy, mask, init, ctx.activation, ctx.residual_is_x)
    if dstate is not None and dstate.numel() > 0:
        dx, dinit = ops.add_state_gradient(dx, dinit if init is not None else None, dstate, mask)
    return (dx, dw.to(weight.dtype), db.to(bias.dtype) if bias is not None else None, None,
            dy if ctx.has_res_tensor else None, dinit if init is not None else None, None, None, None, None)


torch.library.register_autograd("vc1d::prefill", _prefill_backward, setup_context=_prefill_setup)


@torch.library.custom_op("vc1d::update", mutates_args=("conv_state",), device_types="cuda")
def update(x: torch.Tensor, conv_state: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
           cache_seqlens: Optional[torch.Tensor], activation: int, residual: bool) -> torch.Tensor:
    """y of causal_conv1d_update; conv_state is updated in place.  Forward only."""
    return ops._update_forward(x, conv_state, weight, bias, _ACT[activation], cache_seqlens, residual=residual)


@update.register_fake
def _(x, conv_state, weight, bias, cache_seqlens, activation, residual):
    return torch.empty_like(x)


@torch.library.custom_op("vc1d::update_fn", mutates_args=(), device_types="cuda")
def update_fn(x: torch.Tensor, conv_state: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
              cache_seqlens: Optional[torch.Tensor], activation: int, residual: bool
              ) -> Tuple[torch.Tensor, torch.Tensor]:
    """The decode step as a function: (y, state after the step); conv_state itself is left alone.  The
    differentiable form of vc1d::update (a graph cannot differentiate through an in-place update whose
    old value the backward formula needs)."""
    new_state = conv_state.clone()
    y = ops._update_forward(x, new_state, weight, bias, _ACT[activation], cache_seqlens, residual=residual)
    return y, new_state


@update_fn.register_fake
def _(x, conv_state, weight, bias, cache_seqlens, activation, residual):
    return torch.empty_like(x), torch.empty_like(conv_state)


def _update_setup(ctx, inputs, output):
    x, conv_state, weight, bias, cache_seqlens, activation, residual = inputs
    ctx.save_for_backward(x, conv_state, weight, bias, cache_seqlens)
    ctx.activation = activation
    ctx.residual = residual


def _update_backward(ctx, dy, dstate_after):
    x, before, weight, bias, seqlens = ctx.saved_tensors
    dx, dstate, dw, db = torch.ops.vc1d.update_bwd(x, before, weight, bias, dy.contiguous(), seqlens, ctx.activation,
                                                   ctx.residual)
    if dstate_after is not None:
        dx, dstate = ops.add_updated_state_gradient(dx, dstate, dstate_after, seqlens)
    return (dx, dstate, dw.to(weight.dtype), db.to(bias.dtype) if bias is not None else None, None, None, None)


@torch.library.custom_op("vc1d::update_bwd", mutates_args=(), device_types="cuda")
def update_bwd(x: torch.Tensor, conv_state: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
               dy: torch.Tensor, cache_seqlens: Optional[torch.Tensor], activation: int, residual: bool
               ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    dx, dstate, dw, db = ops.causal_conv1d_update_bwd(x, conv_state, weight, bias, dy, _ACT[activation],
                                                      cache_seqlens, residual=residual)
    return dx, dstate, dw, db if db is not None else x.new_empty(0, dtype=torch.float32)


@update_bwd.register_fake
def _(x, conv_state, weight, bias, dy, cache_seqlens, activation, residual):
    return (torch.empty_like(x), torch.empty_like(conv_state.contiguous()), x.new_empty(weight.shape, dtype=torch.float32),
            x.new_empty((weight.shape[0],) if bias is not None else (0,), dtype=torch.float32))


torch.library.register_autograd("vc1d::update_fn", _update_backward, setup_context=_update_setup)
