"""Host-side argument checking of the Python operators: the reference's error messages
(causal-conv1d-mps/test.py:226-236, causal_conv1d_mps/__init__.py:107-135) and the refusal to
compute anything on the CPU.  Runs without a GPU."""
import pytest
import torch

import causal_conv1d
import viby_model_b200 as V


def test_drop_in_module_exports_the_two_reference_names():
    # the reference imports exactly these (model/model.py:22-25)
    assert causal_conv1d.causal_conv1d_fn is V.causal_conv1d_fn
    assert causal_conv1d.causal_conv1d_update is V.causal_conv1d_update


def test_dim_mismatch_message():
    x = torch.randn(2, 4, 8)
    w = torch.randn(5, 4)
    with pytest.raises(ValueError, match="does not match"):
        V.causal_conv1d_fn(x, w, None)


def test_rank_message():
    with pytest.raises(ValueError, match="Expected 3D input tensor"):
        V.causal_conv1d_fn(torch.randn(4, 8), torch.randn(4, 4))
    with pytest.raises(ValueError, match="Expected 2D weight tensor"):
        V.causal_conv1d_fn(torch.randn(1, 4, 8), torch.randn(4, 1, 4))
    with pytest.raises(ValueError, match="Expected 2D input tensor"):
        V.causal_conv1d_update(torch.randn(2, 4, 8), torch.randn(2, 4, 3), torch.randn(4, 4))


def test_bias_and_width_checks():
    x = torch.randn(2, 4, 8)
    with pytest.raises(ValueError, match="Bias dim 3 does not match"):
        V.causal_conv1d_fn(x, torch.randn(4, 4), torch.randn(3))
    with pytest.raises(ValueError, match="width must be 2, 3 or 4"):
        V.causal_conv1d_fn(x, torch.randn(4, 5))


def test_activation_and_seq_idx():
    x = torch.randn(2, 4, 8)
    w = torch.randn(4, 4)
    with pytest.raises(NotImplementedError, match="activation must be None, silu, or swish"):
        V.causal_conv1d_fn(x, w, activation="gelu")
    # seq_idx is an operand like any other: host tensors are refused, never computed on the CPU
    with pytest.raises(ValueError, match="must be on a CUDA device"):
        V.causal_conv1d_fn(x, w, seq_idx=torch.zeros(2, 8, dtype=torch.int32))
    with pytest.raises(ValueError, match="must be on a CUDA device"):
        V.causal_conv1d_fn(x.requires_grad_(), w, seq_idx=torch.zeros(2, 8, dtype=torch.int32))


def test_update_shape_checks():
    with pytest.raises(ValueError, match="doesn't match conv_state"):
        V.causal_conv1d_update(torch.randn(2, 4), torch.randn(2, 5, 3), torch.randn(4, 4))
    with pytest.raises(ValueError, match="shorter than width-1"):
        V.causal_conv1d_update(torch.randn(2, 4), torch.randn(2, 4, 2), torch.randn(4, 4))
    with pytest.raises(ValueError, match="does not match input dtype"):
        V.causal_conv1d_update(torch.randn(2, 4), torch.randn(2, 4, 3).bfloat16(), torch.randn(4, 4))


def test_cpu_tensors_are_refused_not_computed():
    x = torch.randn(2, 4, 8)
    with pytest.raises(ValueError, match="must be on a CUDA device"):
        V.causal_conv1d_fn(x, torch.randn(4, 4))
    with pytest.raises(ValueError, match="must be on a CUDA device"):
        V.causal_conv1d_update(torch.randn(2, 4), torch.randn(2, 4, 3), torch.randn(4, 4))
    assert V.launch_count() == 0 or not torch.cuda.is_available()


def test_valid_prefix_lengths_of_a_host_mask():
    from viby_model_b200.host_io import HostPrefill

    m = torch.tensor([[1, 1, 0, 0], [0, 0, 0, 0], [1, 0, 1, 0], [1, 1, 1, 1], [0, 0, 0, 2]])
    assert HostPrefill.valid_prefix_lengths(m) == [2, 0, 3, 4, 4]
    assert HostPrefill.valid_prefix_lengths(m.bool()) == [2, 0, 3, 4, 4]


def test_custom_ops_have_shape_functions():
    """torch.ops.vc1d.* (what torch.compile sees) infer output shapes, strides and dtypes without a GPU."""
    import viby_model_b200  # noqa: F401
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        x = torch.empty(2, 16, 64, device="cuda", dtype=torch.bfloat16).transpose(1, 2)
        w = torch.empty(64, 4, device="cuda", dtype=torch.bfloat16)
        b = torch.empty(64, device="cuda", dtype=torch.bfloat16)
        y, st = torch.ops.vc1d.prefill(x, w, b, None, None, None, 1, True, True, 4)
        assert y.shape == x.shape and y.stride() == x.stride() and y.dtype == x.dtype
        assert st.shape == (2, 64, 4)
        y2, st2 = torch.ops.vc1d.prefill(x, w, None, None, None, None, 0, False, True, 0)
        assert st2.numel() == 0
        dx, dw, db, dinit = torch.ops.vc1d.prefill_bwd(x, w, b, y, None, None, 1, True)
        assert dinit.numel() == 0
        assert dx.stride() == x.stride() and dw.shape == (64, 4) and dw.dtype == torch.float32 and db.shape == (64,)
        s = torch.empty(2, 64, 4, device="cuda", dtype=torch.bfloat16)
        assert torch.ops.vc1d.update(x[..., 0], s, w, b, None, 1, False).shape == (2, 64)
