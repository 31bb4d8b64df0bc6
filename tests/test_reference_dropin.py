"""The drop-in, proven through the reference's own code.

The reference binds its CUDA conv kernels by module name at import (model/model.py:20-30) and calls
them with keywords inside try/except blocks that print and fall through (model/model.py:293-317,
426-495).  These tests import the reference's ``model/model.py`` UNMODIFIED with this repository's
root on ``sys.path`` and check that

  * the import picks up this package's functions and sets ``HAS_CAUSAL_CONV1D_CUDA`` (CPU test);
  * ``CanonLayer.forward`` on CUDA tensors really launches the kernels for prefill and for cached
    decode steps (the launch counter advances: an exception swallowed by the layer would leave it
    where it was), keeps ``[B, D, kernel_size]`` states, and agrees with the layer's own PyTorch
    branch (``HAS_CAUSAL_CONV1D_CUDA = False``) on valid positions, states bit for bit (GPU test);
  * the reference's cache bookkeeping -- beam reorder (model/model.py:1330-1366) and device transfer
    (eval_model.py:14-56) -- works on states the kernels update in place (GPU test).

They need a checkout of the reference: ``$VIBY_REFERENCE``, ``/root/reference`` or ``baseline/_ref``.
Without one they are skipped; tests/test_model_harness.py and tests/test_cache_ops_gpu.py cover the
same call pattern and the same bookkeeping with a restated model.
"""
import importlib
import os
import sys
from pathlib import Path

import pytest
import torch

from conftest import ROOT


def find_tree():
    for cand in (os.environ.get("VIBY_REFERENCE"), "/root/reference", str(ROOT / "baseline" / "_ref")):
        if cand and (Path(cand) / "model" / "model.py").exists():
            return Path(cand).resolve()
    return None


TREE = find_tree()
needs_tree = pytest.mark.skipif(TREE is None, reason="no checkout of the reference on this machine")


def reference_model():
    """model/model.py of the reference, imported as it is.  The repository root precedes the checkout on
    sys.path (tests/conftest.py puts it there), so ``from causal_conv1d import ...`` finds the drop-in."""
    if "model.model" in sys.modules:
        return sys.modules["model.model"]
    sys.dont_write_bytecode = True  # the checkout is read-only
    sys.path.append(str(TREE))
    try:
        return importlib.import_module("model.model")
    finally:
        sys.path.remove(str(TREE))


@needs_tree
def test_reference_import_binds_this_package():
    import viby_model_b200 as V

    M = reference_model()
    assert M.HAS_CAUSAL_CONV1D_CUDA is True
    assert M.cuda_causal_conv1d_fn is V.causal_conv1d_fn
    assert M.cuda_causal_conv1d_update is V.causal_conv1d_update


def _layer(M, D, K, bias, act, dtype, dev, seed):
    conf = M.VibyConfig(canon_bias=bias, canon_activation=act, canon_kernel=K)
    torch.manual_seed(seed)
    layer = M.CanonLayer(D, conf, "a")
    layer.reset_parameters()
    if bias:
        with torch.no_grad():
            layer.bias_param.uniform_(-0.5, 0.5)
    return layer.to(device=dev, dtype=dtype).eval()


def _close(a, b, x, dtype, what):
    """a, b: layer outputs (input + conv term); compare the conv terms."""
    if dtype == torch.float32:
        assert torch.allclose(a, b, rtol=1e-5, atol=2e-6), what
    else:
        # the PyTorch branch rounds after the conv, after SiLU and after the residual: 2^-6 of the conv term
        ta, tb = a.float() - x.float(), b.float() - x.float()
        assert torch.allclose(ta, tb, rtol=2 ** -6, atol=2 ** -6), what


@needs_tree
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("K", [4, 3])
@pytest.mark.parametrize("bias,act", [(False, False), (True, True)])
def test_reference_canon_layer_runs_on_the_kernels(bias, act, K, dtype):
    from transformers.cache_utils import DynamicCache

    import viby_model_b200 as V

    M = reference_model()
    dev = torch.device("cuda")
    B, T, D = 3, 50, 640
    layer = _layer(M, D, K, bias, act, dtype, dev, seed=K)
    g = torch.Generator().manual_seed(17)
    x = torch.randn(B, T, D, generator=g).to(dtype).to(dev)
    lens = torch.tensor([T, 31, 7])
    mask = (torch.arange(T)[None, :] < lens[:, None]).to(torch.int64).to(dev)
    steps = [torch.randn(B, 1, D, generator=g).to(dtype).to(dev) for _ in range(4)]

    def run(with_kernels):
        M.HAS_CAUSAL_CONV1D_CUDA = with_kernels
        try:
            cache = DynamicCache()
            outs, states, launches = [], [], []
            m = mask
            with torch.no_grad():
                before = V.launch_count()
                outs.append(layer(x, attention_mask=m, cache=cache, layer_idx=0))
                launches.append(V.launch_count() - before)
                states.append(cache.canon_cache_a[0].clone())
                for xt in steps:
                    m = torch.cat([m, torch.ones(B, 1, dtype=m.dtype, device=dev)], 1)
                    before = V.launch_count()
                    outs.append(layer(xt, attention_mask=m, cache=cache, layer_idx=0))
                    launches.append(V.launch_count() - before)
                    states.append(cache.canon_cache_a[0].clone())
            return outs, states, launches
        finally:
            M.HAS_CAUSAL_CONV1D_CUDA = True

    outs_k, states_k, launches_k = run(True)
    outs_f, states_f, launches_f = run(False)
    assert all(n >= 1 for n in launches_k), f"the layer fell back without launching: {launches_k}"
    assert all(n == 0 for n in launches_f)
    assert V.last_kernel() in ("update_vec", "update_lane", "update_generic")
    valid = mask.bool()
    _close(outs_k[0][valid], outs_f[0][valid], x[valid], dtype, "prefill, valid positions")
    for s in range(len(steps) + 1):
        assert states_k[s].shape[-1] == K and states_f[s].shape[-1] == max(8, K)
        assert torch.equal(states_k[s], states_f[s][..., -K:]), f"state after {'prefill' if s == 0 else f'step {s}'}"
        if s > 0:
            _close(outs_k[s], outs_f[s], steps[s - 1], dtype, f"decode step {s}")
    torch.cuda.synchronize()
    assert V.tma_timeouts() == 0


@needs_tree
@pytest.mark.gpu
def test_reference_cache_reorder_and_transfer_with_kernel_states():
    """Beam reorder by the reference's own ``_reorder_cache`` and a device round trip by its
    ``transfer_cache_to_device`` between decode steps: the kernels keep updating the moved states, and
    the layer's PyTorch branch, given the same reordering, agrees bit for bit on the states."""
    from transformers.cache_utils import DynamicCache

    import viby_model_b200 as V

    M = reference_model()
    sys.path.append(str(TREE))
    try:
        E = importlib.import_module("eval_model")
    finally:
        sys.path.remove(str(TREE))
    dev = torch.device("cuda")
    B, T, D, K = 4, 20, 960, 4
    layer = _layer(M, D, K, True, True, torch.bfloat16, dev, seed=2)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(B, T, D, generator=g).bfloat16().to(dev)
    steps = [torch.randn(B, 1, D, generator=g).bfloat16().to(dev) for _ in range(6)]
    beam = torch.tensor([2, 2, 0, 1], device=dev)

    def run(with_kernels):
        M.HAS_CAUSAL_CONV1D_CUDA = with_kernels
        try:
            cache = DynamicCache()
            states = []
            with torch.no_grad():
                layer(x, cache=cache, layer_idx=0)
                for i, xt in enumerate(steps):
                    if i == 2:
                        cache = M.VibyForCausalLM._reorder_cache(None, cache, beam)
                    if i == 4:
                        cache = E.transfer_cache_to_device(E.transfer_cache_to_device(cache, "cpu"), dev)
                    before = V.launch_count()
                    layer(xt, cache=cache, layer_idx=0)
                    assert (V.launch_count() - before >= 1) == with_kernels
                    states.append(cache.canon_cache_a[0].clone())
            return states
        finally:
            M.HAS_CAUSAL_CONV1D_CUDA = True

    for sk, sf in zip(run(True), run(False)):
        assert torch.equal(sk, sf[..., -K:])
