"""Drop-in module for the reference's optional CUDA import (model/model.py:20-30):

    from causal_conv1d import causal_conv1d_fn, causal_conv1d_update

With the repository root on ``sys.path`` the reference's ``model/model.py`` binds these two
names to the B200 kernels of :mod:`viby_model_b200` and sets ``HAS_CAUSAL_CONV1D_CUDA``.
"""
from viby_model_b200 import causal_conv1d_fn, causal_conv1d_update

__all__ = ["causal_conv1d_fn", "causal_conv1d_update"]
