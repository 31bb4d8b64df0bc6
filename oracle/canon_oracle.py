"""CPU oracle for the Canon depthwise causal conv1d path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch/numpy on the CPU, the algorithm the reference runs
when neither optional kernel package is present.  Only the test-suite, the smoke check and
the CPU-baseline leg of the benchmark may import it; the product (viby_model_b200) never
does and has no CPU path of its own.

What each function follows (paths inside the reference project):
  causal_conv1d_ref         causal-conv1d-mps/test.py:83-107 (inputs rounded to the I/O dtype,
                            upcast to fp32, F.pad(W-1,0) + F.conv1d(groups=dim) + F.silu) and
                            model/model.py:604-620, 664-670 (history or zero left-padding);
                            mask multiply model/model.py:454-457 / 590-602; state window
                            model/model.py:470-489 and 623-661; residual model/model.py:491.
  causal_conv1d_packed_ref  the same operator on packed variable-length rows (seq_idx): every run of
                            equal ids is one sequence of causal_conv1d_ref.
  causal_conv1d_update_ref  model/model.py:372-398 (roll left, insert, dot over the last W
                            columns, bias, SiLU), generalised to any state_len >= W-1 exactly as
                            the call at model/model.py:305-311 needs; circular variant
                            causal-conv1d-mps/causal_conv1d_mps/causal_conv1d.metal:586-664.
  canon_layer_ref           model/model.py:400-422 and 587-675 (CanonLayer.forward, PyTorch
                            branch: prefill, chunked continuation, single-token step).
  causal_conv1d_f64         the tap formula of causal_conv1d.metal:160-179 as explicit shifted
                            sums in float64 -- an independent check of the tap order.

Parity pin: tests/golden/canon_golden.npz holds inputs and outputs produced by the
reference's own CanonLayer (imported unmodified; generator tests/golden/make_golden.py);
tests/test_oracle.py checks every function here against those vectors.

Arithmetic contract of the oracle (and of the CUDA kernels): inputs are values of the I/O
dtype, accumulation is fp32, the result is rounded once to the I/O dtype.  The reference's
bf16 fallback instead rounds after the conv and again after SiLU; ``native_dtype=True``
reproduces that for pinning against golden vectors made in bf16.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as F


def _act(name) -> bool:
    if name is None or name is False:
        return False
    if name is True or name in ("silu", "swish"):
        return True
    raise NotImplementedError("activation must be None, silu, or swish")


def apply_mask(x_bdt: torch.Tensor, attention_mask: Optional[torch.Tensor]) -> torch.Tensor:
    """``x * mask`` in the I/O dtype, mask [B,T] broadcast over channels (model/model.py:454-457)."""
    if attention_mask is None:
        return x_bdt
    m = attention_mask.to(x_bdt.dtype) if attention_mask.dtype != x_bdt.dtype else attention_mask
    return x_bdt * m.unsqueeze(1)


def causal_conv1d_ref(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    activation=None,
    *,
    attention_mask: Optional[torch.Tensor] = None,
    initial_states: Optional[torch.Tensor] = None,
    residual: Optional[torch.Tensor] = None,
    state_len: Optional[int] = None,
    return_fp32: bool = False,
):
    """Oracle of causal_conv1d_fn.  x [B,D,T] (any strides), weight [D,W], bias [D]|None.

    Returns y (dtype of x), or (y, final_state[B,D,state_len]) when state_len is given.
    With return_fp32 the first result is the fp32 value before the single rounding
    (before the residual add).
    """
    B, D, T = x.shape
    W = weight.shape[1]
    dt = x.dtype
    xm = apply_mask(x, attention_mask)  # I/O dtype
    w32 = weight.to(dt).float() if weight.dtype != torch.float32 else weight.float()
    b32 = None
    if bias is not None:
        b32 = bias.to(dt).float() if bias.dtype != torch.float32 else bias.float()
    if initial_states is not None:
        hist = initial_states[..., initial_states.shape[-1] - (W - 1):].to(dt).float()
        xin = torch.cat([hist, xm.float()], dim=-1)
    else:
        xin = F.pad(xm.float(), (W - 1, 0))
    y32 = F.conv1d(xin, w32.unsqueeze(1), bias=b32, groups=D)
    if _act(activation):
        y32 = F.silu(y32)
    if return_fp32:
        y = y32
    else:
        y = y32.to(dt)
        if residual is not None:
            y = y + residual  # I/O-dtype add: second rounding, as `x + output` (model/model.py:491)
    if state_len is None:
        return y
    L = int(state_len)
    if initial_states is not None:
        prev = initial_states.to(dt)
        if prev.shape[-1] < L:
            prev = F.pad(prev, (L - prev.shape[-1], 0))
    else:
        prev = torch.zeros(B, D, L, dtype=dt)
    state = torch.cat([prev, xm], dim=-1)[..., -L:].contiguous()
    return y, state


def causal_conv1d_packed_ref(x: torch.Tensor, weight: torch.Tensor, bias=None, activation=None, *,
                             seq_idx: torch.Tensor, return_fp32: bool = False) -> torch.Tensor:
    """Oracle of causal_conv1d_fn with ``seq_idx`` (signature at
    causal-conv1d-mps/causal_conv1d_mps/autograd.py:501-510; the reference itself passes None,
    model/model.py:465).  x [B,D,T] holds, in every row, sequences laid end to end; seq_idx[B,T] names
    the sequence of each step.  Each maximal run of equal ids is convolved on its own with
    causal_conv1d_ref (zeros left of its first step), which is what a right-padded batch computes at
    its valid positions (model/model.py:454-466)."""
    B, D, T = x.shape
    out = torch.empty((B, D, T), dtype=torch.float32 if return_fp32 else x.dtype)
    ids = seq_idx.to(torch.int64)
    for b in range(B):
        row = ids[b]
        cuts = [0] + (torch.nonzero(row[1:] != row[:-1]).flatten() + 1).tolist() + [T]
        for t0, t1 in zip(cuts[:-1], cuts[1:]):
            if t1 > t0:
                out[b:b + 1, :, t0:t1] = causal_conv1d_ref(x[b:b + 1, :, t0:t1], weight, bias, activation,
                                                          return_fp32=return_fp32)
    return out


def causal_conv1d_f64(x: torch.Tensor, weight: torch.Tensor, bias=None, activation=None) -> np.ndarray:
    """y[b,d,t] = act(bias[d] + sum_w weight[d,w] * x[b,d,t-(W-1-w)]) as shifted sums in float64."""
    xn = x.double().numpy()
    wn = weight.double().numpy()
    B, D, T = xn.shape
    W = wn.shape[1]
    y = np.zeros((B, D, T), dtype=np.float64)
    if bias is not None:
        y += bias.double().numpy()[None, :, None]
    for w in range(W):
        shift = W - 1 - w
        if shift >= T:
            continue
        y[:, :, shift:] += wn[None, :, w, None] * xn[:, :, : T - shift]
    if _act(activation):
        y = y / (1.0 + np.exp(-y))
    return y


def causal_conv1d_update_ref(
    x: torch.Tensor,
    conv_state: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    activation=None,
    cache_seqlens: Optional[torch.Tensor] = None,
    residual: bool = False,
    return_fp32: bool = False,
) -> torch.Tensor:
    """Oracle of causal_conv1d_update.  x [B,D], conv_state [B,D,L] updated IN PLACE."""
    B, D = x.shape
    L = conv_state.shape[-1]
    W = weight.shape[1]
    dt = x.dtype
    w32 = weight.to(dt).float() if weight.dtype != torch.float32 else weight.float()
    if cache_seqlens is None:
        cat = torch.cat([conv_state, x.unsqueeze(-1)], dim=-1)  # [B,D,L+1]
        taps = cat[..., -W:].float()
        conv_state.copy_(cat[..., -L:])
    else:
        pos = (cache_seqlens.long() % L)  # [B]
        offs = torch.arange(W - 1, 0, -1)  # W-1 .. 1
        idx = (pos[:, None] - offs[None, :]) % L  # [B, W-1]
        hist = torch.gather(conv_state, 2, idx[:, None, :].expand(B, D, W - 1))
        taps = torch.cat([hist, x.unsqueeze(-1)], dim=-1).float()
        conv_state.scatter_(2, pos[:, None, None].expand(B, D, 1), x.unsqueeze(-1))
    y32 = torch.sum(taps * w32.unsqueeze(0), dim=-1)
    if bias is not None:
        b32 = bias.to(dt).float() if bias.dtype != torch.float32 else bias.float()
        y32 = b32.unsqueeze(0) + y32
    if _act(activation):
        y32 = F.silu(y32)
    if return_fp32:
        return y32
    y = y32.to(dt)
    if residual:
        y = y + x
    return y


def canon_layer_ref(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    activation: bool,
    attention_mask: Optional[torch.Tensor] = None,
    conv_state: Optional[torch.Tensor] = None,
    use_cache: bool = False,
    native_dtype: bool = False,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """CanonLayer.forward, PyTorch branch (model/model.py:400-422, 587-675).

    x [B,T,D]; weight [D,1,K] or [D,K]; returns (x_masked + conv, new_state or None).
    State length is max(8, K) when created here (model/model.py:626, 286).
    native_dtype=True computes conv and SiLU in x.dtype as the reference does; False uses the
    fp32-accumulate / round-once contract.
    """
    if weight.dim() == 3:
        weight = weight.squeeze(1)
    B, T, D = x.shape
    K = weight.shape[1]
    dt = x.dtype

    if use_cache and T == 1:
        # _step_with_cache + _pytorch_step (model/model.py:262-398)
        xt = x.squeeze(1)
        if attention_mask is not None and attention_mask.dim() == 2 and attention_mask.shape[0] == B:
            xt = xt * attention_mask[:, -1].unsqueeze(-1).to(dt)
        if conv_state is None:
            conv_state = torch.zeros(B, D, max(8, K), dtype=dt)
        if native_dtype:
            conv_state.copy_(torch.roll(conv_state, shifts=-1, dims=-1))
            conv_state[:, :, -1] = xt
            res = bias.unsqueeze(0).expand(B, -1).clone() if bias is not None else torch.zeros_like(xt)
            res = res + torch.sum(conv_state[:, :, -K:] * weight.unsqueeze(0), dim=-1)
            if activation:
                res = F.silu(res)
        else:
            res = causal_conv1d_update_ref(xt, conv_state, weight, bias, activation)
        # the step adds the ORIGINAL token (model/model.py:370)
        return x + res.unsqueeze(1), conv_state

    if attention_mask is not None and attention_mask.dim() == 2:
        if tuple(attention_mask.shape) == (B, T):
            x = x * attention_mask.unsqueeze(-1)
        elif attention_mask.size(0) == B and attention_mask.size(1) >= T:
            x = x * attention_mask[:, -T:].unsqueeze(-1)
    x = x.to(dt)
    x_conv = x.transpose(1, 2)
    history = conv_state[:, :, -(K - 1):] if (conv_state is not None and K > 1) else None

    if use_cache:
        if conv_state is None:
            conv_state = torch.zeros(B, D, max(8, K), dtype=dt)
        S = conv_state.size(-1)
        if history is None:
            if T <= S:
                conv_state[:, :, -T:] = x_conv
            else:
                conv_state[:, :, :] = x_conv[:, :, -S:]
        else:
            history = history.clone()
            if T >= S:
                conv_state[:, :, :] = x_conv[:, :, -S:]
            else:
                conv_state.copy_(torch.roll(conv_state, shifts=-T, dims=-1))
                conv_state[:, :, -T:] = x_conv

    if native_dtype:
        xin = torch.cat([history, x_conv], dim=-1) if history is not None else F.pad(x_conv, (K - 1, 0))
        y = F.conv1d(xin, weight.unsqueeze(1).to(dt), bias=bias, groups=D)
        if activation:
            y = F.silu(y)
    else:
        init = None
        if history is not None:
            init = history
        y = causal_conv1d_ref(x_conv, weight, bias, "silu" if activation else None, initial_states=init)
    return x + y.transpose(1, 2), (conv_state if use_cache else None)


# ----------------------------------------------------------------------------------------------
# ulp helpers used by the parity tests
# ----------------------------------------------------------------------------------------------
def bf16_ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in representable bf16 values between two bf16 tensors (signed zeros coincide)."""
    def key(t):
        bits = t.contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
        sign = bits >> 15
        mag = bits & 0x7FFF
        return torch.where(sign == 1, -mag, mag)
    return (key(a) - key(b)).abs()


def seeded(shape, seed: int, dist: str = "normal", dtype=torch.float32) -> torch.Tensor:
    """Deterministic CPU tensor: N(0,1) or U(-0.5,0.5), generated in fp32 then cast."""
    g = torch.Generator().manual_seed(int(seed))
    if dist == "normal":
        t = torch.randn(shape, generator=g, dtype=torch.float32)
    elif dist == "uniform":
        t = torch.rand(shape, generator=g, dtype=torch.float32) - 0.5
    else:
        raise ValueError(dist)
    return t.to(dtype)


def causal_conv1d_bwd_ref(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    dy: torch.Tensor,
    activation=None,
    *,
    attention_mask: Optional[torch.Tensor] = None,
    residual: bool = False,
    residual_masked: bool = False,
    compute_dtype: torch.dtype = torch.float64,
):
    """Oracle of the backward pass of causal_conv1d_fn (+ fused mask / residual), as explicit
    shifted sums.  x, dy [B,D,T]; weight [D,W]; returns (dx [B,D,T] in x's dtype, dweight [D,W],
    dbias [D] or None), the last two in ``compute_dtype``.

    Follows the arithmetic of causal-conv1d-mps/causal_conv1d_mps/causal_conv1d.metal:1354-1483
    (fused BTD backward) and :803-854 (plain backward):
        pre[t]   = bias + sum_w weight[w] * (x*mask)[t-(W-1-w)]
        g[t]     = dy[t] * silu'(pre[t])           silu'(z) = s(z) * (1 + z*(1 - s(z)))
        dx[t]    = [residual] dy[t] + mask[t] * sum_w weight[w] * g[t+(W-1-w)]
        dweight[w] = sum_{b,t} (x*mask)[t-(W-1-w)] * g[t];   dbias = sum_{b,t} g[t]
    ``residual`` adds the unmasked input (model/model.py:491); ``residual_masked`` the masked one
    (the PyTorch branch, model/model.py:595-602, 675).
    """
    B, D, T = x.shape
    W = weight.shape[1]
    cd = compute_dtype
    xm = apply_mask(x, attention_mask).to(cd)  # the mask multiply is rounded to the I/O dtype first
    w = weight.to(x.dtype).to(cd) if weight.dtype != torch.float32 else weight.to(cd)
    g = dy.to(cd).clone()
    if _act(activation):
        pre = torch.zeros(B, D, T, dtype=cd)
        if bias is not None:
            pre += (bias.to(x.dtype) if bias.dtype != torch.float32 else bias).to(cd).view(1, D, 1)
        for k in range(W):
            s = W - 1 - k
            if s < T:
                pre[..., s:] += w[:, k].view(1, D, 1) * xm[..., : T - s]
        sig = torch.sigmoid(pre)
        g = g * sig * (1 + pre * (1 - sig))
    dconv = torch.zeros(B, D, T, dtype=cd)
    dweight = torch.zeros(D, W, dtype=cd)
    for k in range(W):
        s = W - 1 - k
        if s < T:
            dconv[..., : T - s] += w[:, k].view(1, D, 1) * g[..., s:]
            dweight[:, k] = (xm[..., : T - s] * g[..., s:]).sum(dim=(0, 2))
    if attention_mask is not None:
        m = attention_mask.to(cd).unsqueeze(1)
        dconv = dconv * m
    dx = dconv
    if residual_masked:
        dx = dx + dy.to(cd) * (attention_mask.to(cd).unsqueeze(1) if attention_mask is not None else 1)
    elif residual:
        dx = dx + dy.to(cd)
    dbias = g.sum(dim=(0, 2)) if bias is not None else None
    return dx.to(x.dtype), dweight, dbias


def causal_conv1d_packed_bwd_ref(x, weight, bias, dy, activation=None, *, seq_idx, residual: bool = False,
                                 compute_dtype: torch.dtype = torch.float64):
    """Oracle of the backward pass on packed variable-length rows (``seq_idx``): every maximal run of
    equal ids is one sequence of causal_conv1d_bwd_ref; dweight and dbias add up over the runs."""
    B, D, T = x.shape
    dx = torch.zeros_like(x)
    dweight = torch.zeros(D, weight.shape[1], dtype=compute_dtype)
    dbias = torch.zeros(D, dtype=compute_dtype) if bias is not None else None
    ids = seq_idx.to(torch.int64)
    for b in range(B):
        row = ids[b]
        cuts = [0] + (torch.nonzero(row[1:] != row[:-1]).flatten() + 1).tolist() + [T]
        for t0, t1 in zip(cuts[:-1], cuts[1:]):
            if t1 > t0:
                sdx, sdw, sdb = causal_conv1d_bwd_ref(x[b:b + 1, :, t0:t1], weight, bias, dy[b:b + 1, :, t0:t1], activation,
                                                      residual=residual, compute_dtype=compute_dtype)
                dx[b:b + 1, :, t0:t1] = sdx
                dweight += sdw
                if dbias is not None:
                    dbias += sdb
    return dx, dweight, dbias


def causal_conv1d_update_bwd_ref(x, conv_state, weight, bias, dy, activation=None, *, residual: bool = False,
                                 compute_dtype: torch.dtype = torch.float64):
    """Oracle of the backward pass of one decode step (shifting state), restating
    causal_conv1d.metal:1738-1845 for a shifting state: cat = [state | x]; y = act(bias + cat[-W:] . weight) [+ x].
    Returns (dx [B,D], dstate [B,D,L], dweight [D,W], dbias [D]|None); dstate is the gradient of y
    with respect to the state the step started from (columns that no tap reads get zero)."""
    B, D = x.shape
    L = conv_state.shape[-1]
    W = weight.shape[1]
    cd = compute_dtype
    cat = torch.cat([conv_state.to(cd), x.to(cd).unsqueeze(-1)], dim=-1)  # [B,D,L+1]
    w = weight.to(x.dtype).to(cd) if weight.dtype != torch.float32 else weight.to(cd)
    win = cat[..., -W:]
    g = dy.to(cd).clone()
    if _act(activation):
        pre = (win * w.unsqueeze(0)).sum(-1)
        if bias is not None:
            pre = pre + (bias.to(x.dtype) if bias.dtype != torch.float32 else bias).to(cd)
        sig = torch.sigmoid(pre)
        g = g * sig * (1 + pre * (1 - sig))
    dwin = g.unsqueeze(-1) * w.unsqueeze(0)  # [B,D,W]
    dcat = torch.zeros_like(cat)
    dcat[..., -W:] = dwin
    dx = dcat[..., -1] + (dy.to(cd) if residual else 0)
    dstate = dcat[..., :-1]
    dweight = (g.unsqueeze(-1) * win).sum(0)
    dbias = g.sum(0) if bias is not None else None
    return dx.to(x.dtype), dstate.to(x.dtype), dweight, dbias
