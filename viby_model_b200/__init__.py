"""B200 (sm_100a) depthwise causal conv1d for Viby's Canon A/B/C/D layers.

Public surface:
  causal_conv1d_fn, causal_conv1d_update  -- the CUDA slot of the reference's CanonLayer
                                             (model/model.py:20-30, 305-311, 460-466)
  causal_conv1d_bwd, causal_conv1d_update_bwd  -- their backward passes (causal_conv1d_fn is differentiable;
                                             contract: causal_conv1d_mps/autograd.py:116-151, 305-338)
  causal_conv1d_fwd, short_conv_fused,
  short_conv_update                       -- the [B,T,D] operators of causal-conv1d-mps
                                             (causal_conv1d_mps/__init__.py:81-419)
  launch_count, last_kernel               -- proof that the CUDA kernels ran

The operators call hand-written CUDA kernels through the C ABI of include/vc1d.h
(libvc1d.so, built by ``python viby_model_b200/build.py``).  Importing the package without
that library raises ImportError: there is no CPU or PyTorch fallback.
"""
from ._cabi import last_kernel, launch_count, library_path, set_pdl, tma_timeouts
from .ops import (UpdateTable, causal_conv1d_bwd, causal_conv1d_fn, causal_conv1d_fn_multi, causal_conv1d_update,
                  causal_conv1d_update_bwd, causal_conv1d_update_multi, reuse_tile_classes, seq_idx_from_lengths)
from .short_conv import causal_conv1d_fwd, short_conv_fused, short_conv_update
from . import canon_cache  # noqa: F401  (Canon states on a generation cache: accessors, beam reorder, device transfer)
from . import compile_ops  # noqa: F401  (registers torch.ops.vc1d.* for torch.compile)

__all__ = [
    "causal_conv1d_fn",
    "causal_conv1d_update",
    "causal_conv1d_bwd",
    "causal_conv1d_fn_multi",
    "seq_idx_from_lengths",
    "causal_conv1d_update_bwd",
    "causal_conv1d_update_multi",
    "UpdateTable",
    "causal_conv1d_fwd",
    "short_conv_fused",
    "short_conv_update",
    "launch_count",
    "last_kernel",
    "library_path",
    "tma_timeouts",
    "set_pdl",
    "reuse_tile_classes",
]
__version__ = "0.1.0"
