"""CUDA-slot operators of Viby's CanonLayer: ``causal_conv1d_fn`` and ``causal_conv1d_update``.

Call signatures follow the reference's call sites (model/model.py:460-466 and 305-311) and
its own mirror of the prefill signature (causal-conv1d-mps/causal_conv1d_mps/autograd.py:
501-510).  Everything after the bare ``*`` is an extension that fuses work the reference's
CanonLayer does in separate PyTorch passes around the kernel; with the extensions left at
their defaults the functions are drop-in for the reference's CUDA branch.

Host code only marshals pointers, sizes and strides into the C ABI (include/vc1d.h).
There is no PyTorch or CPU implementation behind these functions.
"""
from __future__ import annotations

import ctypes as C
import threading
from typing import Optional, Tuple, Union

import torch

from . import _cabi

_IO_DTYPES = {torch.float32: _cabi.VC1D_F32, torch.bfloat16: _cabi.VC1D_BF16, torch.float16: _cabi.VC1D_F16}
_MASK_DTYPES = {
    torch.bool: _cabi.VC1D_U8,
    torch.uint8: _cabi.VC1D_U8,
    torch.int32: _cabi.VC1D_I32,
    torch.int64: _cabi.VC1D_I64,
    torch.float32: _cabi.VC1D_F32,
    torch.bfloat16: _cabi.VC1D_BF16,
    torch.float16: _cabi.VC1D_F16,
}


_TMA_TUNING = {"stages", "ctas_per_sm", "slab_bytes", "rows_per_thread", "claim_chunk", "empty_store", "classify", "pdl", "static_first", "test_expire"}


def _activation_code(activation) -> int:
    # reference: autograd.py:527-530 accepts None, "silu", "swish"; the BTD API passes a bool
    if activation is None or activation is False:
        return _cabi.VC1D_ACT_NONE
    if activation is True or activation in ("silu", "swish"):
        return _cabi.VC1D_ACT_SILU
    raise NotImplementedError("activation must be None, silu, or swish")


def _require_cuda(t: torch.Tensor, what: str) -> None:
    if t.device.type != "cuda":
        raise ValueError(f"{what} tensor must be on a CUDA device, got {t.device}")


def _check_weight_shapes(weight: torch.Tensor, bias: Optional[torch.Tensor], dim: int) -> int:
    """Shape checks with the reference's messages (causal_conv1d_mps/__init__.py:116-135)."""
    if weight.dim() != 2:
        raise ValueError(f"Expected 2D weight tensor (dim, width), got {weight.dim()}D")
    weight_dim, width = weight.shape
    if dim != weight_dim:
        raise ValueError(f"Input dim {dim} does not match weight dim {weight_dim}")
    if width not in (2, 3, 4):
        raise ValueError(f"width must be 2, 3 or 4, got {width}")
    if bias is not None:
        if bias.dim() != 1:
            raise ValueError(f"Expected 1D bias tensor, got {bias.dim()}D")
        if bias.shape[0] != dim:
            raise ValueError(f"Bias dim {bias.shape[0]} does not match input dim {dim}")
    return width


def _align_weights(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]):
    """Weight/bias dtype: same as x, or float32 (converted in-kernel); bias follows weight."""
    _require_cuda(weight, "Weight")
    if weight.dtype != x.dtype and weight.dtype != torch.float32:
        weight = weight.to(x.dtype)
    if bias is not None:
        _require_cuda(bias, "Bias")
        if bias.dtype != weight.dtype:
            bias = bias.to(weight.dtype)
        if not bias.is_contiguous():
            bias = bias.contiguous()
    return weight, bias


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream_handle(device: torch.device) -> int:
    if _raw_stream is not None and device.index is not None:
        return _raw_stream(device.index)
    return torch.cuda.current_stream(device).cuda_stream


# Scratch of the dynamic tile scheduler: one small zeroed buffer per (device, stream), because
# launches that can overlap on the GPU must not share it.  The kernel leaves it zeroed.
_DYNAMIC_DEFAULT = True
_SCRATCH = {}
_TLS = threading.local()  # per host thread: prepared argument structs, and the fresh-scratch switch


class fresh_scratch:
    """Within this context the launch wrappers allocate their scheduler scratch per call instead of
    keeping one buffer per stream (used by the torch.compile custom ops)."""

    def __enter__(self):
        _TLS.fresh_scratch = getattr(_TLS, "fresh_scratch", 0) + 1

    def __exit__(self, *exc):
        _TLS.fresh_scratch -= 1


def _scheduler_scratch(device: torch.device, stream: int, nbytes: int) -> torch.Tensor:
    if getattr(_TLS, "fresh_scratch", 0) or torch.cuda.is_current_stream_capturing():
        # Memory allocated while a CUDA graph is being captured, or inside a compiled region (whose
        # allocations may go to a graph's private pool also while it warms up), belongs to that graph: it
        # must not be kept for later launches.  A buffer of its own, zeroed by a memset on the stream.
        return torch.zeros(max(16384, (nbytes + 3) // 4), dtype=torch.int32, device=device)
    key = (device.index, stream)
    buf = _SCRATCH.get(key)
    if buf is None or buf.numel() * 4 < nbytes:
        buf = torch.zeros(max(16384, (nbytes + 3) // 4), dtype=torch.int32, device=device)
        _SCRATCH[key] = buf
    return buf


def causal_conv1d_fn(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    seq_idx: Optional[torch.Tensor] = None,
    initial_states: Optional[torch.Tensor] = None,
    return_final_states: bool = False,
    final_states_out: Optional[torch.Tensor] = None,
    activation: Optional[str] = None,
    *,
    attention_mask: Optional[torch.Tensor] = None,
    skip_masked_loads: bool = True,
    residual: Union[None, bool, torch.Tensor] = None,
    state_len: Optional[int] = None,
    out: Optional[torch.Tensor] = None,
    kernel: Optional[str] = None,
    rows_per_thread: int = 0,
    block_threads: int = 0,
    unroll: int = 0,
    tma: Optional[dict] = None,
    dynamic_schedule: Optional[bool] = None,
) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
    """Depthwise causal conv1d over ``x[batch, dim, seqlen]`` (prefill).

    ``y[b,d,t] = act(bias[d] + sum_w weight[d,w] * x[b,d,t-(W-1-w)])`` with zeros (or
    ``initial_states``) left of t=0, fp32 accumulation, one rounding to ``x.dtype``.  ``x`` may
    have any strides; the channel-last view ``x_btd.transpose(1, 2)`` that CanonLayer passes
    (model/model.py:459) and contiguous ``[B,D,T]`` both take 128-bit vectorised kernels.
    The result has the shape, dtype and (for dense inputs) the strides of ``x``.

    Reference arguments (model/model.py:460-466; autograd.py:501-510):
      weight ``[dim, width]`` (width 2..4), bias ``[dim]`` or None, activation None|"silu"|"swish",
      ``seq_idx[batch, seqlen]`` (int32): packed variable-length rows.  Each time step names the
        sequence it belongs to and a tap only counts when it carries the same value as the output
        step, so sequences laid end to end in one row (``seq_idx_from_lengths``) give exactly the
        results of a right-padded batch at the valid positions, without reading or writing padding.
        The reference passes None (model/model.py:465); not combined with a mask or states; differentiable,
      ``initial_states[batch, dim, >=width-1]``: history used instead of zeros (its last width-1 columns),
      ``return_final_states`` / ``final_states_out``: also return the last ``state_len`` inputs as
      ``[batch, dim, state_len]`` (default state_len = width-1), right-aligned like
      model/model.py:470-489.

    Extensions (keyword-only), each replacing a separate PyTorch pass of CanonLayer.forward:
      attention_mask ``[batch, seqlen]`` (bool / int / float): inputs are multiplied by the mask
        before the conv (model/model.py:454-457); outputs at masked positions are still produced.
        With ``skip_masked_loads`` rows whose mask is 0 are not read at all and count as +0
        (identical results for finite inputs).
      residual: a tensor shaped like ``x`` (or True for ``x`` itself) added after the activation,
        with the same two roundings as ``x + y`` (model/model.py:491).
      state_len: width of the returned final state (CanonLayer keeps ``kernel_size`` columns).
      out: preallocated output; kernel / rows_per_thread / block_threads / unroll: tuning overrides;
      tma: dict of tuning overrides of the TMA-staged kernel (stages, ctas_per_sm, slab_bytes,
        rows_per_thread).
      dynamic_schedule: let the CTAs of the TMA-staged kernel claim tiles from per-slab counters in a
        small scratch buffer (one per device and stream, allocated on first use) instead of a fixed
        assignment; evens out ragged batches.

    Differentiable in ``x``, ``weight``, ``bias`` and a separate ``residual`` tensor (the contract of
    causal-conv1d-mps autograd.py:116-151, 305-338): when any of them requires grad the backward
    pass runs ``causal_conv1d_bwd`` (``initial_states`` receives a gradient too).  ``out=`` is forward-only.
    """
    if torch.compiler.is_compiling():
        # inside torch.compile the operator is one opaque graph node (compile_ops.py)
        if seq_idx is not None:
            raise NotImplementedError("seq_idx is not supported")
        if out is not None or final_states_out is not None:
            raise ValueError("out= / final_states_out= cannot be used under torch.compile")
        want_state = bool(return_final_states)
        L = int(state_len) if state_len is not None else weight.shape[1] - 1
        y, state = torch.ops.vc1d.prefill(
            x, weight, bias, attention_mask, residual if isinstance(residual, torch.Tensor) else None,
            initial_states, _activation_code(activation), residual is True, bool(skip_masked_loads),
            L if want_state else 0)
        return (y, state) if want_state else y
    needs_grad = torch.is_grad_enabled() and (
        x.requires_grad or weight.requires_grad or (bias is not None and bias.requires_grad)
        or (isinstance(residual, torch.Tensor) and residual.requires_grad)
        or (initial_states is not None and initial_states.requires_grad)
    )
    kw = dict(attention_mask=attention_mask, skip_masked_loads=skip_masked_loads, residual=residual,
              state_len=state_len, out=out, kernel=kernel, rows_per_thread=rows_per_thread,
              block_threads=block_threads, unroll=unroll, tma=tma, dynamic_schedule=dynamic_schedule)
    if not needs_grad:
        return _prefill_forward(x, weight, bias, seq_idx, initial_states, return_final_states, final_states_out,
                                activation, **kw)
    if out is not None:
        raise ValueError("out= cannot be used when a gradient is required")
    res_tensor = residual if isinstance(residual, torch.Tensor) else None
    kw["seq_idx"] = seq_idx
    result = _CausalConv1dFunction.apply(x, weight, bias, res_tensor, activation, attention_mask,
                                         residual is True, return_final_states, final_states_out, kw,
                                         initial_states)
    return result if (return_final_states or final_states_out is not None) else result[0]


def seq_idx_from_lengths(lengths, device=None) -> torch.Tensor:
    """``seq_idx[1, sum(lengths)]`` (int32) for sequences of the given lengths packed end to end in one
    row: 0 for every step of the first sequence, 1 for the second, and so on."""
    lengths = torch.as_tensor(lengths, dtype=torch.int64, device="cpu")
    ids = torch.repeat_interleave(torch.arange(lengths.numel(), dtype=torch.int32), lengths)
    return ids.unsqueeze(0).to(device) if device is not None else ids.unsqueeze(0)


def causal_conv1d_fn_multi(xs, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, activation=None, **kwargs):
    """``causal_conv1d_fn`` over tensors that together form the channel dimension, without
    concatenating them: ``xs`` is a sequence of ``[batch, dim_i, seqlen]`` tensors (e.g. the q, k and
    v projections, or gate and up), ``weight[sum(dim_i), width]`` / ``bias[sum(dim_i)]`` cover them in
    order.  Returns the list of outputs.  Replaces the ``torch.cat`` before and the split after the
    Canon-B and Canon-D calls of the reference (model/model.py:772-789, 962-971): one launch per
    tensor on its own rows of the weights, no extra pass over the activations.  Keyword arguments
    are those of ``causal_conv1d_fn`` (``residual=True`` adds each tensor to its own output)."""
    total = sum(int(x.shape[1]) for x in xs)
    if weight.dim() != 2 or weight.shape[0] != total:
        raise ValueError(f"weight rows {tuple(weight.shape)} do not match the summed dims {total}")
    if isinstance(kwargs.get("residual"), torch.Tensor) or kwargs.get("out") is not None:
        raise ValueError("a residual tensor or out= applies to one tensor: call causal_conv1d_fn per tensor")
    outs, d0 = [], 0
    for x in xs:
        d1 = d0 + int(x.shape[1])
        outs.append(causal_conv1d_fn(x, weight[d0:d1], None if bias is None else bias[d0:d1], activation=activation,
                                     **kwargs))
        d0 = d1
    return outs


# The tile classes of a masked (or packed) launch are a function of the mask alone, and a model hands one
# mask to every Canon call of a forward pass (72 of them in the reference's network).  Per scratch buffer
# this remembers whose pre-pass filled the class table: the mask tensor itself (kept alive, so that its
# address cannot pass to another tensor), its version counter (torch counts every in-place write), and
# the other things the classes depend on.  A launch that finds its own record there skips the pre-pass.
# Writes that torch does not see (a foreign kernel given the raw pointer) are not noticed: such callers
# switch this off with reuse_tile_classes(False).
_CLASS_TABLES = {}  # (device, stream) -> {tile-height slot: (scratch buffer, mask, version, signature)}
_REUSE_CLASSES = True


def reuse_tile_classes(enabled: bool) -> bool:
    """Let consecutive masked launches on one stream share their tile classes while the mask tensor is
    unchanged (default on).  Returns the previous setting."""
    global _REUSE_CLASSES
    previous, _REUSE_CLASSES = _REUSE_CLASSES, bool(enabled)
    _CLASS_TABLES.clear()
    return previous


def _mask_version(m: torch.Tensor):
    try:
        return m._version
    except RuntimeError:  # inference tensors keep no version counter
        return None


def _scratch_bytes(batch: int, seqlen: int) -> int:
    """Claim counters plus room for a class table per tile height."""
    return 4096 + 4 * batch * ((seqlen + 31) // 32) + 128


def _class_table_begin(a, sc: Optional[torch.Tensor], slot, m: torch.Tensor, sig):
    """Before a forward launch with mask (or seq_idx) `m` on scratch `sc`: names the kept tables whose record
    matches.  Returns what _class_table_end needs to make a record of this launch, or None."""
    a.tma_kept_tables = 0
    if sc is None or not _REUSE_CLASSES or a.tma_classify not in (0, 1) or _SCRATCH.get(slot) is not sc:
        return None  # switched off, an explicit choice, or a scratch buffer of this call's own (graph capture, compiled region)
    version = _mask_version(m)
    if version is None:
        return None
    for region, (rsc, rm, rversion, rsig) in _CLASS_TABLES.get(slot, {}).items():
        if (rsc is sc and rsig == sig and rversion == version and rm._version == version
                and rm.data_ptr() == m.data_ptr() and rm.shape == m.shape and rm.stride() == m.stride()
                and rm.dtype == m.dtype):
            a.tma_kept_tables |= 1 << region
    return version


def _class_table_end(a, sc, slot, m, version, sig) -> None:
    """After the launch: the table it wrote (if it wrote one) replaces the record of its place."""
    a.tma_kept_tables = 0  # argument structs are kept for later calls
    st = _cabi.lib.vc1d_last_class_table()
    state, region = st & 0xFF, st >> 8
    if state == 1:
        if version is not None:
            _CLASS_TABLES.setdefault(slot, {})[region] = (sc, m, version, sig)
        else:
            _CLASS_TABLES.get(slot, {}).pop(region, None)
    elif state == 3:
        _CLASS_TABLES.pop(slot, None)


def _prefill_fast(x, weight, bias, activation, attention_mask, skip_masked_loads, residual, want_state, state_len):
    """Cached-signature path of _prefill_forward for the calls a Canon layer makes (no initial state,
    no preallocated outputs, no tuning overrides).  Returns (result, key); result is None when the
    signature has not been validated yet."""
    m = attention_mask
    key = (x.shape, x.stride(), x.dtype, x.device.index, weight.shape, weight.stride(), weight.dtype,
           None if bias is None else (bias.shape, bias.stride(), bias.dtype), activation,
           None if m is None else (m.shape, m.stride(), m.dtype, m.device.index), bool(skip_masked_loads),
           residual is True, want_state, state_len)
    cache = getattr(_TLS, "prefill_args", None)
    a = cache.get(key) if cache is not None else None
    if a is None:
        return None, key
    out = torch.empty_like(x)
    a.x = x.data_ptr()
    a.y = out.data_ptr()
    a.weight = weight.data_ptr()
    a.bias = bias.data_ptr() if bias is not None else None
    if m is not None:
        a.mask = m.data_ptr()
    if residual is True:
        a.residual = a.x
    final_states = None
    if want_state:
        final_states = torch.empty((x.shape[0], x.shape[1], a.state_len), dtype=x.dtype, device=x.device)
        a.final_state = final_states.data_ptr()
    dev = x.device
    stream = _stream_handle(dev)
    sc = None
    if _DYNAMIC_DEFAULT:
        sc = _scheduler_scratch(dev, stream, _scratch_bytes(x.shape[0], x.shape[2]))
        a.scratch = sc.data_ptr()
        a.scratch_bytes = sc.numel() * 4
    if m is not None:
        slot = (dev.index, stream)
        sig = ("mask", x.shape[0], x.shape[2], weight.shape[-1], bool(skip_masked_loads), residual is True, False, 0)
        version = _class_table_begin(a, sc, slot, m, sig)
    if dev.index != torch.cuda.current_device():
        with torch.cuda.device(dev):
            st = _cabi.lib.vc1d_prefill(C.byref(a), stream)
    else:
        st = _cabi.lib.vc1d_prefill(C.byref(a), stream)
    if m is not None:
        _class_table_end(a, sc, slot, m, version, sig)
    if st != 0:
        _cabi.check(st, "causal_conv1d_fn")
    return ((out, final_states) if want_state else out), key


def _prefill_forward(
    x, weight, bias=None, seq_idx=None, initial_states=None, return_final_states=False, final_states_out=None,
    activation=None, *, attention_mask=None, skip_masked_loads=True, residual=None, state_len=None, out=None,
    kernel=None, rows_per_thread=0, block_threads=0, unroll=0, tma=None, dynamic_schedule=None,
):
    """The forward launch behind causal_conv1d_fn (no autograd bookkeeping)."""
    fast_key = None
    plain = (seq_idx is None and initial_states is None and final_states_out is None and out is None
             and kernel is None and tma is None and dynamic_schedule is None and rows_per_thread == 0
             and block_threads == 0 and unroll == 0 and (residual is None or residual is True)
             and x.is_cuda and weight.is_cuda)
    if plain:
        result, fast_key = _prefill_fast(x, weight, bias, activation, attention_mask, skip_masked_loads, residual,
                                         bool(return_final_states), state_len)
        if result is not None:
            return result
    weight_given, bias_given = weight, bias
    if x.dim() != 3:
        raise ValueError(f"Expected 3D input tensor (batch, dim, seqlen), got {x.dim()}D")
    batch, dim, seqlen = x.shape
    width = _check_weight_shapes(weight, bias, dim)
    if x.dtype not in _IO_DTYPES:
        raise ValueError(f"unsupported dtype {x.dtype}: expected float32, bfloat16 or float16")
    act = _activation_code(activation)
    _require_cuda(x, "Input")
    weight, bias = _align_weights(x, weight, bias)
    if seq_idx is not None:
        _require_cuda(seq_idx, "seq_idx")
        if tuple(seq_idx.shape) != (batch, seqlen):
            raise ValueError(f"seq_idx shape {tuple(seq_idx.shape)} does not match input shape ({batch}, {seqlen})")
        if attention_mask is not None or initial_states is not None or return_final_states or final_states_out is not None:
            raise ValueError("seq_idx cannot be combined with attention_mask, initial_states or final states")
        if seq_idx.dtype != torch.int32:
            seq_idx = seq_idx.to(torch.int32)

    if out is None:
        out = torch.empty_like(x)
    elif out.shape != x.shape or out.dtype != x.dtype or out.device != x.device:
        raise ValueError("out must match x in shape, dtype and device")

    a = _cabi.PrefillArgs()
    a.struct_size = C.sizeof(_cabi.PrefillArgs)
    a.dtype = _IO_DTYPES[x.dtype]
    a.wdtype = _IO_DTYPES[weight.dtype]
    a.activation = act
    a.batch, a.dim, a.seqlen, a.width = batch, dim, seqlen, width
    a.x = x.data_ptr()
    a.y = out.data_ptr()
    a.weight = weight.data_ptr()
    a.bias = bias.data_ptr() if bias is not None else None
    a.x_stride_b, a.x_stride_d, a.x_stride_t = x.stride()
    a.y_stride_b, a.y_stride_d, a.y_stride_t = out.stride()
    a.w_stride_d, a.w_stride_w = weight.stride()

    if seq_idx is not None:
        a.seq_idx = seq_idx.data_ptr()
        a.seq_stride_b, a.seq_stride_t = seq_idx.stride()

    if attention_mask is not None:
        m = attention_mask
        _require_cuda(m, "Attention mask")
        if m.dim() != 2:
            raise ValueError(f"Expected 2D attention mask, got {m.dim()}D")
        if tuple(m.shape) != (batch, seqlen):
            raise ValueError(
                f"Attention mask shape {tuple(m.shape)} does not match input shape ({batch}, {seqlen})"
            )
        if m.dtype not in _MASK_DTYPES:
            raise ValueError(f"unsupported attention mask dtype {m.dtype}")
        a.mask = m.data_ptr()
        a.mask_dtype = _MASK_DTYPES[m.dtype]
        a.mask_stride_b, a.mask_stride_t = m.stride()
        a.skip_masked_loads = 1 if skip_masked_loads else 0

    if residual is not None and residual is not False:
        r = x if residual is True else residual
        if r.shape != x.shape or r.dtype != x.dtype or r.device != x.device:
            raise ValueError("residual must match x in shape, dtype and device")
        a.residual = r.data_ptr()
        a.r_stride_b, a.r_stride_d, a.r_stride_t = r.stride()

    if initial_states is not None:
        s0 = initial_states
        if s0.dim() != 3 or s0.shape[0] != batch or s0.shape[1] != dim or s0.shape[2] < width - 1:
            raise ValueError(
                f"initial_states shape {tuple(s0.shape)} does not match (batch, dim, >=width-1) = "
                f"({batch}, {dim}, >={width - 1})"
            )
        if s0.dtype != x.dtype or s0.device != x.device:
            raise ValueError("initial_states must match x in dtype and device")
        if not s0.is_contiguous():
            s0 = s0.contiguous()
        a.initial_state = s0.data_ptr()
        a.init_len = s0.shape[2]

    final_states = None
    if return_final_states or final_states_out is not None:
        L = int(state_len) if state_len is not None else (
            final_states_out.shape[2] if final_states_out is not None else width - 1
        )
        if L < 1:
            raise ValueError(f"state_len must be >= 1, got {L}")
        if final_states_out is not None:
            final_states = final_states_out
            if tuple(final_states.shape) != (batch, dim, L) or final_states.dtype != x.dtype:
                raise ValueError(
                    f"final_states_out shape {tuple(final_states.shape)} does not match ({batch}, {dim}, {L})"
                )
            if not final_states.is_contiguous():
                raise ValueError("final_states_out must be contiguous [batch, dim, state_len]")
        else:
            final_states = torch.empty((batch, dim, L), dtype=x.dtype, device=x.device)
        a.final_state = final_states.data_ptr()
        a.state_len = L

    if kernel not in _cabi.KERNEL_BY_NAME:
        raise ValueError(f"unknown kernel {kernel!r}")
    a.kernel = _cabi.KERNEL_BY_NAME[kernel]
    a.rows_per_thread = int(rows_per_thread)
    a.block_threads = int(block_threads)
    a.unroll = int(unroll)
    if tma:
        for key, value in tma.items():
            if key not in _TMA_TUNING:
                raise ValueError(f"unknown TMA tuning key {key!r}; expected one of {sorted(_TMA_TUNING)}")
            setattr(a, "tma_" + key, int(value))

    stream = _stream_handle(x.device)
    sc = None
    if dynamic_schedule or (dynamic_schedule is None and _DYNAMIC_DEFAULT):
        sc = _scheduler_scratch(x.device, stream, _scratch_bytes(batch, seqlen))
        a.scratch = sc.data_ptr()
        a.scratch_bytes = sc.numel() * sc.element_size()
    classes_of = seq_idx if seq_idx is not None else attention_mask
    if classes_of is not None:
        slot = (x.device.index, stream)
        sig = ("ids" if seq_idx is not None else "mask", batch, seqlen, width, bool(skip_masked_loads),
               a.residual is not None, initial_states is not None, int(a.tma_classify))
        version = _class_table_begin(a, sc, slot, classes_of, sig)
    if x.device.index != torch.cuda.current_device():
        with torch.cuda.device(x.device):
            st = _cabi.lib.vc1d_prefill(C.byref(a), stream)
    else:
        st = _cabi.lib.vc1d_prefill(C.byref(a), stream)
    if classes_of is not None:
        _class_table_end(a, sc, slot, classes_of, version, sig)
    _cabi.check(st, "causal_conv1d_fn")
    if fast_key is not None and weight is weight_given and bias is bias_given:
        # remember the validated struct for later calls with the same shapes, strides and options
        cache = getattr(_TLS, "prefill_args", None)
        if cache is None:
            cache = _TLS.prefill_args = {}
        if len(cache) < 256:
            cache[fast_key] = a
    if return_final_states or final_states_out is not None:
        return out, final_states
    return out


def causal_conv1d_bwd(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    dy: torch.Tensor,
    activation: Optional[str] = None,
    *,
    attention_mask: Optional[torch.Tensor] = None,
    residual: bool = False,
    initial_states: Optional[torch.Tensor] = None,
    need_dweight: bool = True,
    need_dbias: bool = True,
    kernel: Optional[str] = None,
    dynamic_schedule: Optional[bool] = None,
    tma: Optional[dict] = None,
    seq_idx: Optional[torch.Tensor] = None,
):
    """Gradients of ``causal_conv1d_fn`` (with its fused mask / residual) for ``x[batch, dim, seqlen]``
    and the upstream gradient ``dy`` of the same shape: returns ``(dx, dweight, dbias)``.

    ``dx`` has the dtype and strides of ``x``; ``dweight[dim, width]`` and ``dbias[dim]`` are summed in
    fp32 and returned in fp32 (the caller casts), as the reference's backward does
    (causal-conv1d-mps/causal_conv1d_mps/causal_conv1d_kernel.mm:553-557, 771-776).
    ``residual=True`` means the forward added ``x`` to its output.  Formulas: include/vc1d.h.
    With ``initial_states[batch, dim, >=width-1]`` (the history of a chunked continuation) a fourth
    result is returned: the gradient with respect to it.  ``tma``: tuning overrides of the TMA-staged
    kernel (stages, ctas_per_sm, variant).  ``seq_idx[batch, seqlen]`` (int32): the forward ran on packed
    rows; gradients stay inside each run of equal ids (no mask, no initial state).
    """
    if x.dim() != 3:
        raise ValueError(f"Expected 3D input tensor (batch, dim, seqlen), got {x.dim()}D")
    if dy.shape != x.shape or dy.dtype != x.dtype or dy.device != x.device:
        raise ValueError("dy must match x in shape, dtype and device")
    batch, dim, seqlen = x.shape
    width = _check_weight_shapes(weight, bias, dim)
    if x.dtype not in _IO_DTYPES:
        raise ValueError(f"unsupported dtype {x.dtype}: expected float32, bfloat16 or float16")
    act = _activation_code(activation)
    _require_cuda(x, "Input")
    weight, bias = _align_weights(x, weight, bias)
    # a gradient with several zero strides (e.g. from sum().backward()) is not addressable as a tensor map
    if any(st == 0 for st, n in zip(dy.stride(), dy.shape) if n > 1):
        dy = dy.contiguous() if x.stride(2) == 1 else dy.transpose(1, 2).contiguous().transpose(1, 2)
    dx = torch.empty_like(x)
    if dx.stride() != x.stride():
        dx = torch.empty_strided(x.shape, x.stride(), dtype=x.dtype, device=x.device)
    # both fp32 accumulators in one allocation; the library clears it (inside its pre-pass when it has one)
    want_db = need_dbias and bias is not None
    acc = torch.empty(dim * (width + 1), dtype=torch.float32, device=x.device) if (need_dweight or want_db) else None
    dweight = acc[: dim * width].view(dim, width) if need_dweight else None
    dbias = acc[dim * width:] if want_db else None

    a = _cabi.PrefillBwdArgs()
    a.struct_size = C.sizeof(_cabi.PrefillBwdArgs)
    a.dtype = _IO_DTYPES[x.dtype]
    a.wdtype = _IO_DTYPES[weight.dtype]
    a.activation = act
    a.batch, a.dim, a.seqlen, a.width = batch, dim, seqlen, width
    a.x, a.dy, a.dx = x.data_ptr(), dy.data_ptr(), dx.data_ptr()
    a.weight = weight.data_ptr()
    a.bias = bias.data_ptr() if bias is not None else None
    a.x_stride_b, a.x_stride_d, a.x_stride_t = x.stride()
    a.dy_stride_b, a.dy_stride_d, a.dy_stride_t = dy.stride()
    a.dx_stride_b, a.dx_stride_d, a.dx_stride_t = dx.stride()
    a.w_stride_d, a.w_stride_w = weight.stride()
    if attention_mask is not None:
        m = attention_mask
        _require_cuda(m, "Attention mask")
        if tuple(m.shape) != (batch, seqlen):
            raise ValueError(
                f"Attention mask shape {tuple(m.shape)} does not match input shape ({batch}, {seqlen})"
            )
        if m.dtype not in _MASK_DTYPES:
            raise ValueError(f"unsupported attention mask dtype {m.dtype}")
        a.mask = m.data_ptr()
        a.mask_dtype = _MASK_DTYPES[m.dtype]
        a.mask_stride_b, a.mask_stride_t = m.stride()
    a.residual = 1 if residual else 0
    a.dweight = dweight.data_ptr() if dweight is not None else None
    a.dbias = dbias.data_ptr() if dbias is not None else None
    a.zero_grads = 1
    if seq_idx is not None:
        _require_cuda(seq_idx, "seq_idx")
        if tuple(seq_idx.shape) != (batch, seqlen):
            raise ValueError(f"seq_idx shape {tuple(seq_idx.shape)} does not match input shape ({batch}, {seqlen})")
        if attention_mask is not None or initial_states is not None:
            raise ValueError("seq_idx cannot be combined with attention_mask, initial_states or final states")
        if seq_idx.dtype != torch.int32:
            seq_idx = seq_idx.to(torch.int32)
        a.seq_idx = seq_idx.data_ptr()
        a.seq_stride_b, a.seq_stride_t = seq_idx.stride()
    dinit = None
    if initial_states is not None:
        s0 = initial_states
        if s0.dim() != 3 or s0.shape[0] != batch or s0.shape[1] != dim or s0.shape[2] < width - 1:
            raise ValueError(
                f"initial_states shape {tuple(s0.shape)} does not match (batch, dim, >=width-1) = "
                f"({batch}, {dim}, >={width - 1})"
            )
        if s0.dtype != x.dtype or s0.device != x.device:
            raise ValueError("initial_states must match x in dtype and device")
        s0 = s0.contiguous()
        dinit = torch.empty_like(s0)
        a.initial_state = s0.data_ptr()
        a.dinitial_state = dinit.data_ptr()
        a.init_len = s0.shape[2]
    if kernel not in (None, "auto", "generic", "tma"):
        raise ValueError(f"unknown backward kernel {kernel!r}")
    a.kernel = _cabi.KERNEL_BY_NAME[kernel]
    if tma:
        for key, value in tma.items():
            if key not in ("stages", "ctas_per_sm", "variant"):
                raise ValueError(f"unknown TMA tuning key {key!r}; expected stages, ctas_per_sm or variant")
            setattr(a, "tma_" + key, int(value))
    stream = _stream_handle(x.device)
    if dynamic_schedule or (dynamic_schedule is None and _DYNAMIC_DEFAULT):
        sc = _scheduler_scratch(x.device, stream, _scratch_bytes(batch, seqlen))
        a.scratch = sc.data_ptr()
        a.scratch_bytes = sc.numel() * sc.element_size()
        _CLASS_TABLES.pop((x.device.index, stream), None)  # the backward pre-pass writes its own classes there
    if x.device.index != torch.cuda.current_device():
        with torch.cuda.device(x.device):
            st = _cabi.lib.vc1d_prefill_bwd(C.byref(a), stream)
    else:
        st = _cabi.lib.vc1d_prefill_bwd(C.byref(a), stream)
    _cabi.check(st, "causal_conv1d_bwd")
    if initial_states is not None:
        return dx, dweight, dbias, dinit
    return dx, dweight, dbias


def add_state_gradient(dx, dinit, dstate, mask):
    """Gradient arriving through the final state returned by causal_conv1d_fn.  Column j of the state
    ``[batch, dim, L]`` is the masked input of step ``T - L + j`` (model/model.py:470-489), or, left of step
    0, a column of the initial state: add ``dstate`` there.  Returns (dx, dinit)."""
    L, T = dstate.shape[2], dx.shape[2]
    n = min(L, T)
    g = dstate[..., L - n:]
    if mask is not None:
        g = g * mask[:, None, T - n:].to(g.dtype)
    dx[..., T - n:] += g.to(dx.dtype)
    if T < L and dinit is not None:
        k = min(L - T, dinit.shape[2])
        dinit[..., dinit.shape[2] - k:] += dstate[..., L - T - k: L - T].to(dinit.dtype)
    return dx, dinit


def add_updated_state_gradient(dx, dstate, dstate_after, seqlens):
    """Gradient arriving through the state a decode step left behind: the step moved the old columns
    (or kept them in place, circular state) and stored x in one column.  Returns (dx, dstate)."""
    L = dstate_after.shape[2]
    if seqlens is not None:
        pos = (seqlens.long() % L).view(-1, 1, 1).expand(-1, dstate_after.shape[1], 1)
        dx = dx + dstate_after.gather(2, pos).squeeze(-1)
        if dstate is not None:
            dstate = dstate + dstate_after.scatter(2, pos, 0.0)
    else:
        dx = dx + dstate_after[..., L - 1]
        if dstate is not None and L > 1:
            dstate = dstate.clone()
            dstate[..., 1:] += dstate_after[..., : L - 1]
    return dx, dstate


class _CausalConv1dFunction(torch.autograd.Function):
    """Autograd glue of causal_conv1d_fn: forward launches the prefill kernel, backward launches
    causal_conv1d_bwd (contract: causal-conv1d-mps/causal_conv1d_mps/autograd.py:116-151, 305-338)."""

    @staticmethod
    def forward(ctx, x, weight, bias, res_tensor, activation, attention_mask, residual_is_x, return_final_states,
                final_states_out, kw, initial_states):
        kw = dict(kw)
        kw["residual"] = True if residual_is_x else res_tensor
        seq_idx = kw.pop("seq_idx", None)
        ctx.seq_idx = seq_idx
        result = _prefill_forward(x, weight, bias, seq_idx, initial_states, return_final_states, final_states_out,
                                  activation, **kw)
        y, state = result if isinstance(result, tuple) else (result, None)
        ctx.save_for_backward(x, weight, bias if bias is not None else x.new_empty(0),
                              attention_mask if attention_mask is not None else x.new_empty(0),
                              initial_states if initial_states is not None else x.new_empty(0))
        ctx.has_init = initial_states is not None
        ctx.has_bias = bias is not None
        ctx.has_mask = attention_mask is not None
        ctx.activation = activation
        ctx.residual_is_x = residual_is_x
        ctx.has_res_tensor = res_tensor is not None
        ctx.has_state = state is not None
        if state is None:
            state = x.new_empty(0)
            ctx.mark_non_differentiable(state)
        return y, state

    @staticmethod
    def backward(ctx, dy, dstate):
        x, weight, bias, mask, init = ctx.saved_tensors
        need_x, need_w, need_b = ctx.needs_input_grad[0], ctx.needs_input_grad[1], ctx.needs_input_grad[2]
        grads = causal_conv1d_bwd(
            x, weight, bias if ctx.has_bias else None, dy, ctx.activation,
            attention_mask=mask if ctx.has_mask else None, residual=ctx.residual_is_x,
            initial_states=init if ctx.has_init else None,
            need_dweight=need_w, need_dbias=need_b and ctx.has_bias, seq_idx=ctx.seq_idx,
        )
        dx, dw, db = grads[0], grads[1], grads[2]
        dinit = grads[3] if ctx.has_init else None
        if ctx.has_state and dstate is not None:
            # the returned final state is part of the graph (chunked training feeds it to the next
            # chunk as initial_states): its gradient lands on the last inputs of this chunk
            dx, dinit = add_state_gradient(dx, dinit, dstate, mask if ctx.has_mask else None)
        return (
            dx if need_x else None,
            dw.to(weight.dtype) if (need_w and dw is not None) else None,
            db.to(bias.dtype) if (need_b and db is not None) else None,
            dy if (ctx.has_res_tensor and ctx.needs_input_grad[3]) else None,
            None, None, None, None, None, None,
            dinit if (ctx.has_init and ctx.needs_input_grad[10]) else None,
        )


def causal_conv1d_update(
    x: torch.Tensor,
    conv_state: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    activation: Optional[str] = None,
    cache_seqlens: Optional[torch.Tensor] = None,
    *,
    residual: bool = False,
    out: Optional[torch.Tensor] = None,
    kernel: Optional[str] = None,
    block_threads: int = 0,
) -> torch.Tensor:
    """Single-token causal conv step against a rolling ``conv_state`` (decode); see ``_update_forward``
    for the arithmetic.  Differentiable in ``x``, ``conv_state`` (the state before the step),
    ``weight`` and ``bias`` like ``short_conv_update_fn`` of causal-conv1d-mps (autograd.py:322-482):
    when one of them requires grad, the state before the step is kept for the backward pass."""
    if torch.compiler.is_compiling():
        if out is not None:
            raise ValueError("out= cannot be used under torch.compile")
        squeeze = x.dim() == 3
        x2 = x.squeeze(-1) if squeeze else x
        wants_grad = torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad or conv_state.requires_grad
                                                  or (bias is not None and bias.requires_grad))
        if wants_grad:
            # differentiable form: the step as a function of the old state; the caller's tensor then takes
            # the new values, detached (inside a compiled graph the updated state carries no gradient)
            # (a copy goes in: the backward formula needs the state the step started from, and the caller's
            # tensor is overwritten below)
            y, new_state = torch.ops.vc1d.update_fn(x2, conv_state.clone(), weight, bias, cache_seqlens,
                                                    _activation_code(activation), bool(residual))
            conv_state.detach().copy_(new_state.detach())
        else:
            y = torch.ops.vc1d.update(x2, conv_state, weight, bias, cache_seqlens, _activation_code(activation),
                                      bool(residual))
        return y.unsqueeze(-1) if squeeze else y
    needs_grad = torch.is_grad_enabled() and (
        x.requires_grad or weight.requires_grad or conv_state.requires_grad
        or (bias is not None and bias.requires_grad)
    )
    if not needs_grad:
        return _update_forward(x, conv_state, weight, bias, activation, cache_seqlens, residual=residual, out=out,
                               kernel=kernel, block_threads=block_threads)
    if out is not None:
        raise ValueError("out= cannot be used when a gradient is required")
    return _CausalConv1dUpdateFunction.apply(x, conv_state, weight, bias, activation, cache_seqlens, residual)[0]


class UpdateTable:
    """A table of independent decode steps that one kernel launch runs (vc1d_update_multi): step i is
    ``causal_conv1d_update(xs[i], conv_states[i], weights[i], biases[i], activation)``, each with its own batch,
    channel count and state length, all of one dtype and on one device.  The table is validated and built
    once; ``launch()`` then costs one library call per 80 steps.  The buffers are the ones given here: write
    the next inputs into ``xs[i]`` (or pass tensors that something else fills), read ``outs[i]``; the states
    are updated in place.

    The steps must not depend on each other.  The Canon steps of one token of one network do (Canon A feeds
    attention, whose output feeds Canon C, ...; model/model.py:1021-1055): a table is for the steps of
    several requests, beams or networks that are decoded side by side.  No gradient."""

    def __init__(self, xs, conv_states, weights, biases=None, activation=None, cache_seqlens=None, *,
                 residual: bool = False, outs=None):
        n = len(xs)
        if not (len(conv_states) == n and len(weights) == n):
            raise ValueError("xs, conv_states and weights must have the same length")
        biases = [None] * n if biases is None else biases
        cache_seqlens = [None] * n if cache_seqlens is None else cache_seqlens
        outs = [None] * n if outs is None else outs
        if not (len(biases) == n and len(cache_seqlens) == n and len(outs) == n):
            raise ValueError("biases, cache_seqlens and outs must have one entry per step")
        self.device = xs[0].device if n else None
        self.outs = []
        self._keep = []  # every tensor whose memory the table names
        self._table = (_cabi.UpdateArgs * max(n, 1))()
        self._n = n
        for i in range(n):
            x = xs[i]
            squeeze = x.dim() == 3 and x.shape[-1] == 1
            if squeeze:
                x = x.squeeze(-1)
            if x.device != self.device:
                raise ValueError("all steps of one launch must live on one device")
            if x.dtype != xs[0].dtype:
                raise ValueError("all steps of one launch must have one dtype")
            a, out, w, b, cs = _build_update_args(x, conv_states[i], weights[i], biases[i], activation,
                                                  cache_seqlens[i], residual, outs[i], None, 0)
            self._table[i] = a
            self._keep.append((x, conv_states[i], w, b, cs, out))
            self.outs.append(out.unsqueeze(-1) if squeeze else out)

    def __len__(self):
        return self._n

    def launch(self):
        """Enqueues the steps on the device's current stream; returns ``outs``."""
        if self._n == 0:
            return self.outs
        stream = _stream_handle(self.device)
        limit = _cabi.UPDATE_MULTI_MAX
        size = C.sizeof(_cabi.UpdateArgs)
        base = C.addressof(self._table)
        other = self.device.index != torch.cuda.current_device()
        if other:
            prev = torch.cuda.current_device()
            torch.cuda.set_device(self.device)
        try:
            for first in range(0, self._n, limit):
                st = _cabi.lib.vc1d_update_multi(C.cast(base + first * size, C.POINTER(_cabi.UpdateArgs)),
                                                 min(limit, self._n - first), stream)
                if st != 0:
                    _cabi.check(st, "causal_conv1d_update_multi")
        finally:
            if other:
                torch.cuda.set_device(prev)
        return self.outs


def causal_conv1d_update_multi(xs, conv_states, weights, biases=None, activation=None, cache_seqlens=None, *,
                               residual: bool = False, outs=None):
    """Several independent decode steps in one kernel launch: ``causal_conv1d_update(xs[i], conv_states[i],
    weights[i], biases[i], activation)`` for every i (see UpdateTable, which this builds and launches once;
    keep the table when the same buffers are stepped again).  The states are updated in place; returns the
    list of outputs, bit-equal to the separate calls."""
    return UpdateTable(xs, conv_states, weights, biases, activation, cache_seqlens, residual=residual,
                       outs=outs).launch()


def causal_conv1d_update_bwd(
    x: torch.Tensor,
    conv_state: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    dy: torch.Tensor,
    activation: Optional[str] = None,
    cache_seqlens: Optional[torch.Tensor] = None,
    *,
    residual: bool = False,
    need_dstate: bool = True,
):
    """Gradients of one decode step: ``(dx, dstate, dweight, dbias)`` for ``x[batch, dim]``,
    ``conv_state[batch, dim, state_len]`` AS IT WAS BEFORE the step, and the upstream ``dy[batch, dim]``.
    ``dweight`` / ``dbias`` are fp32 sums (causal-conv1d-mps causal_conv1d.metal:1738-1845)."""
    if x.dim() != 2 or conv_state.dim() != 3:
        raise ValueError("expected x [batch, dim] and conv_state [batch, dim, state_len]")
    batch, dim = x.shape
    L = conv_state.shape[2]
    if tuple(conv_state.shape[:2]) != (batch, dim) or dy.shape != x.shape:
        raise ValueError("x, dy and conv_state do not agree in batch/dim")
    width = _check_weight_shapes(weight, bias, dim)
    if L < width - 1:
        raise ValueError(f"conv_state length {L} is shorter than width-1 = {width - 1}")
    if x.dtype not in _IO_DTYPES or conv_state.dtype != x.dtype or dy.dtype != x.dtype:
        raise ValueError("x, conv_state and dy must share one of float32, bfloat16, float16")
    act = _activation_code(activation)
    _require_cuda(x, "Input")
    _require_cuda(conv_state, "Convolution state")
    weight, bias = _align_weights(x, weight, bias)
    dx = torch.empty_like(x)
    dstate = torch.empty((batch, dim, L), dtype=x.dtype, device=x.device) if need_dstate else None
    dweight = torch.zeros(dim, width, dtype=torch.float32, device=x.device)
    dbias = torch.zeros(dim, dtype=torch.float32, device=x.device) if bias is not None else None
    a = _cabi.UpdateBwdArgs()
    a.struct_size = C.sizeof(_cabi.UpdateBwdArgs)
    a.dtype = _IO_DTYPES[x.dtype]
    a.wdtype = _IO_DTYPES[weight.dtype]
    a.activation = act
    a.batch, a.dim, a.width, a.state_len = batch, dim, width, L
    a.x, a.conv_state, a.dy, a.dx = x.data_ptr(), conv_state.data_ptr(), dy.data_ptr(), dx.data_ptr()
    a.dstate = dstate.data_ptr() if dstate is not None else None
    a.weight = weight.data_ptr()
    a.bias = bias.data_ptr() if bias is not None else None
    a.x_stride_b, a.x_stride_d = x.stride()
    a.dy_stride_b, a.dy_stride_d = dy.stride()
    a.dx_stride_b, a.dx_stride_d = dx.stride()
    a.s_stride_b, a.s_stride_d, a.s_stride_l = conv_state.stride()
    a.w_stride_d, a.w_stride_w = weight.stride()
    if cache_seqlens is not None:
        _require_cuda(cache_seqlens, "cache_seqlens")
        if cache_seqlens.dtype != torch.int32 or not cache_seqlens.is_contiguous():
            cache_seqlens = cache_seqlens.to(torch.int32).contiguous()
        a.cache_seqlens = cache_seqlens.data_ptr()
    a.residual = 1 if residual else 0
    a.dweight = dweight.data_ptr()
    a.dbias = dbias.data_ptr() if dbias is not None else None
    if x.device.index != torch.cuda.current_device():
        with torch.cuda.device(x.device):
            st = _cabi.lib.vc1d_update_bwd(C.byref(a), _stream_handle(x.device))
    else:
        st = _cabi.lib.vc1d_update_bwd(C.byref(a), _stream_handle(x.device))
    _cabi.check(st, "causal_conv1d_update_bwd")
    return dx, dstate, dweight, dbias


class _CausalConv1dUpdateFunction(torch.autograd.Function):
    """Autograd glue of causal_conv1d_update.  The kernel overwrites conv_state, so the state the step
    started from is cloned for the backward pass (as autograd.py:440-447 of causal-conv1d-mps does)."""

    @staticmethod
    def forward(ctx, x, conv_state, weight, bias, activation, cache_seqlens, residual):
        before = conv_state.detach().clone()
        y = _update_forward(x.detach(), conv_state.detach(), weight.detach(),
                            bias.detach() if bias is not None else None, activation, cache_seqlens, residual=residual)
        ctx.mark_dirty(conv_state)
        ctx.save_for_backward(x, before, weight, bias if bias is not None else x.new_empty(0),
                              cache_seqlens if cache_seqlens is not None else x.new_empty(0))
        ctx.has_bias = bias is not None
        ctx.has_seqlens = cache_seqlens is not None
        ctx.activation = activation
        ctx.residual = residual
        ctx.squeeze = x.dim() == 3
        return y, conv_state

    @staticmethod
    def backward(ctx, dy, dstate_after):
        x, before, weight, bias, seqlens = ctx.saved_tensors
        x2 = x.squeeze(-1) if ctx.squeeze else x
        dy2 = dy.squeeze(-1) if ctx.squeeze else dy
        dx, dstate, dw, db = causal_conv1d_update_bwd(
            x2, before, weight, bias if ctx.has_bias else None, dy2.contiguous(), ctx.activation,
            seqlens if ctx.has_seqlens else None, residual=ctx.residual, need_dstate=ctx.needs_input_grad[1],
        )
        if dstate_after is not None:
            dx, dstate = add_updated_state_gradient(dx, dstate, dstate_after, seqlens if ctx.has_seqlens else None)
        if ctx.squeeze:
            dx = dx.unsqueeze(-1)
        return (
            dx if ctx.needs_input_grad[0] else None,
            dstate if ctx.needs_input_grad[1] else None,
            dw.to(weight.dtype) if ctx.needs_input_grad[2] else None,
            db.to(bias.dtype) if (ctx.has_bias and ctx.needs_input_grad[3]) else None,
            None, None, None,
        )


# Prepared vc1d_update_args per call signature (shapes, strides, dtypes, options): a decode step is
# launch-bound, so a repeated call only refreshes the five pointers instead of re-validating and
# re-filling the whole struct.
# (_TLS, per host thread: the library call releases the GIL while it reads the struct)


def _update_fast(x, conv_state, weight, bias, activation, cache_seqlens, residual, out, kernel, block_threads):
    """The cached-signature path of _update_forward; returns None when the signature is new."""
    key = (x.shape, x.stride(), x.dtype, x.device.index, conv_state.shape, conv_state.stride(), conv_state.dtype,
           weight.shape, weight.stride(), weight.dtype,
           None if bias is None else (bias.shape, bias.dtype, bias.stride()),
           activation, bool(residual), kernel, block_threads, None if out is None else (out.shape, out.stride(), out.dtype))
    cache = getattr(_TLS, "update_args", None)
    a = cache.get(key) if cache is not None else None
    if a is None:
        return None, key
    if out is None:
        out = torch.empty_like(x)
    a.x = x.data_ptr()
    a.y = out.data_ptr()
    a.conv_state = conv_state.data_ptr()
    a.weight = weight.data_ptr()
    a.bias = bias.data_ptr() if bias is not None else None
    dev = x.device
    if dev.index != torch.cuda.current_device():
        with torch.cuda.device(dev):
            st = _cabi.lib.vc1d_update(C.byref(a), _stream_handle(dev))
    else:
        st = _cabi.lib.vc1d_update(C.byref(a), _stream_handle(dev))
    if st != 0:
        _cabi.check(st, "causal_conv1d_update")
    return out, key


def _build_update_args(x, conv_state, weight, bias, activation, cache_seqlens, residual, out, kernel, block_threads):
    """Validates one decode step and fills its argument struct.  Returns (struct, out, weight, bias,
    cache_seqlens): the last three are the tensors whose memory the struct names (possibly converted copies,
    which the caller has to keep alive until the launch is enqueued)."""
    if x.dim() != 2:
        raise ValueError(f"Expected 2D input tensor (batch, dim), got {x.dim()}D")
    if conv_state.dim() != 3:
        raise ValueError(f"Expected 3D conv_state tensor (batch, dim, state_len), got {conv_state.dim()}D")
    batch, dim = x.shape
    conv_batch, conv_dim, L = conv_state.shape
    if batch != conv_batch or dim != conv_dim:
        raise ValueError(f"Input shape {tuple(x.shape)} doesn't match conv_state batch/dim {(conv_batch, conv_dim)}")
    width = _check_weight_shapes(weight, bias, dim)
    if L < width - 1 or L < 1:
        raise ValueError(f"conv_state length {L} is shorter than width-1 = {width - 1}")
    if x.dtype not in _IO_DTYPES:
        raise ValueError(f"unsupported dtype {x.dtype}: expected float32, bfloat16 or float16")
    if conv_state.dtype != x.dtype:
        raise ValueError(f"conv_state dtype {conv_state.dtype} does not match input dtype {x.dtype}")
    act = _activation_code(activation)
    _require_cuda(x, "Input")
    _require_cuda(conv_state, "Convolution state")
    weight, bias = _align_weights(x, weight, bias)

    if out is None:
        out = torch.empty_like(x)
    elif out.shape != x.shape or out.dtype != x.dtype or out.device != x.device:
        raise ValueError("out must match x in shape, dtype and device")

    a = _cabi.UpdateArgs()
    a.struct_size = C.sizeof(_cabi.UpdateArgs)
    a.dtype = _IO_DTYPES[x.dtype]
    a.wdtype = _IO_DTYPES[weight.dtype]
    a.activation = act
    a.batch, a.dim, a.width, a.state_len = batch, dim, width, L
    a.x = x.data_ptr()
    a.y = out.data_ptr()
    a.conv_state = conv_state.data_ptr()
    a.weight = weight.data_ptr()
    a.bias = bias.data_ptr() if bias is not None else None
    a.x_stride_b, a.x_stride_d = x.stride()
    a.y_stride_b, a.y_stride_d = out.stride()
    a.s_stride_b, a.s_stride_d, a.s_stride_l = conv_state.stride()
    a.w_stride_d, a.w_stride_w = weight.stride()
    if cache_seqlens is not None:
        _require_cuda(cache_seqlens, "cache_seqlens")
        if cache_seqlens.dim() != 1:
            raise ValueError(f"Expected 1D cache_seqlens, got {cache_seqlens.dim()}D")
        if cache_seqlens.shape[0] != batch:
            raise ValueError(f"cache_seqlens batch size {cache_seqlens.shape[0]} != input batch {batch}")
        if cache_seqlens.dtype != torch.int32 or not cache_seqlens.is_contiguous():
            cache_seqlens = cache_seqlens.to(torch.int32).contiguous()
        a.cache_seqlens = cache_seqlens.data_ptr()
    a.residual = 1 if residual else 0
    if kernel not in (None, "auto", "generic"):
        raise ValueError(f"unknown update kernel {kernel!r}")
    a.kernel = _cabi.KERNEL_GENERIC if kernel == "generic" else _cabi.KERNEL_AUTO
    a.block_threads = int(block_threads)

    return a, out, weight, bias, cache_seqlens


def _update_forward(
    x: torch.Tensor,
    conv_state: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    activation: Optional[str] = None,
    cache_seqlens: Optional[torch.Tensor] = None,
    *,
    residual: bool = False,
    out: Optional[torch.Tensor] = None,
    kernel: Optional[str] = None,
    block_threads: int = 0,
) -> torch.Tensor:
    """Single-token causal conv step against a rolling ``conv_state`` (decode).

    ``cat = [conv_state | x]``; ``y = act(bias + cat[..., -W:] . weight)``;
    ``conv_state <- cat[..., -state_len:]`` **in place**; returns ``y`` shaped like ``x``.
    Matches the reference call at model/model.py:305-311 and the PyTorch step at
    model/model.py:372-398 for any ``state_len >= width-1`` (the reference's CUDA branch uses
    ``state_len == width``, its fallback 8).

    x ``[batch, dim]`` (or ``[batch, dim, 1]``), conv_state ``[batch, dim, state_len]``.
    ``cache_seqlens[batch]`` (int32) switches to the circular-buffer state of
    causal-conv1d-mps (causal_conv1d.metal:586-664): write position ``cache_seqlens[b] % state_len``.
    ``residual=True`` adds ``x`` to the result (causal_conv1d.metal:655-658).
    """
    squeeze = False
    if x.dim() == 3 and x.shape[-1] == 1:
        x = x.squeeze(-1)
        squeeze = True
    fast_key = None
    if cache_seqlens is None and x.is_cuda and conv_state.is_cuda and weight.is_cuda and (bias is None or bias.is_cuda):
        y, fast_key = _update_fast(x, conv_state, weight, bias, activation, cache_seqlens, residual, out, kernel,
                                   block_threads)
        if y is not None:
            return y.unsqueeze(-1) if squeeze else y
    weight_given, bias_given = weight, bias
    a, out, weight, bias, cache_seqlens = _build_update_args(x, conv_state, weight, bias, activation, cache_seqlens,
                                                             residual, out, kernel, block_threads)
    if x.device.index != torch.cuda.current_device():
        with torch.cuda.device(x.device):
            st = _cabi.lib.vc1d_update(C.byref(a), _stream_handle(x.device))
    else:
        st = _cabi.lib.vc1d_update(C.byref(a), _stream_handle(x.device))
    _cabi.check(st, "causal_conv1d_update")
    # remember the validated struct for calls with the same signature (weights whose dtype had to be
    # converted are a fresh tensor every call: those keep the full path)
    if fast_key is not None and weight is weight_given and bias is bias_given:
        cache = getattr(_TLS, "update_args", None)
        if cache is None:
            cache = _TLS.update_args = {}
        if len(cache) < 256:
            cache[fast_key] = a
    return out.unsqueeze(-1) if squeeze else out
