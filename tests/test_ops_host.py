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


def test_kept_tile_tables_bookkeeping(monkeypatch):
    """Host side of the tile tables kept between masked launches (ops._class_table_begin/_end): a table is
    offered to a launch only for the same scratch buffer, the same mask memory, layout and torch version
    counter and the same options; what the launch reports (vc1d_last_class_table) updates the record of
    its tile-height place.  No kernel runs: the report is faked."""
    from viby_model_b200 import _cabi, ops

    report = {"value": 0}
    monkeypatch.setattr(_cabi.lib, "vc1d_last_class_table", lambda: report["value"], raising=False)
    monkeypatch.setattr(ops, "_CLASS_TABLES", {})
    a = _cabi.PrefillArgs()
    slot = (0, 1234)
    sc = torch.zeros(16, dtype=torch.int32)
    monkeypatch.setitem(ops._SCRATCH, slot, sc)
    m = torch.ones(4, 8, dtype=torch.bool)
    sig = ("mask", 4, 8, 4, True, False, False, 0)

    def launch(mask, says, signature=sig, scratch=sc):
        version = ops._class_table_begin(a, scratch, slot, mask, signature)
        offered = a.tma_kept_tables
        report["value"] = says
        ops._class_table_end(a, scratch, slot, mask, version, signature)
        assert a.tma_kept_tables == 0  # argument structs are reused
        return offered

    WROTE, READ, FRONT = 1, 2, 3
    assert launch(m, WROTE) == 0  # nothing known yet; the pre-pass wrote place 0
    assert launch(m, READ) == 1
    assert launch(m[:, :], READ) == 1  # a view of the same memory
    assert launch(m, WROTE | (1 << 8), sig[:3] + (4,) + sig[4:]) == 1  # place 1 (another tile height) written
    assert launch(m, READ) == 3
    assert launch(m, 0, sig[:4] + (False,) + sig[5:]) == 0  # other options: not the same classes
    assert launch(m, READ) == 3  # ... and that launch (on a kernel without tables) touched none
    assert launch(m.clone(), 0) == 0  # equal contents elsewhere in memory
    m[0, 0] = False  # torch counts the write
    assert launch(m, WROTE) == 0
    assert launch(m, READ) == 1  # place 1 holds the classes of the old contents and is not offered
    other = torch.zeros(16, dtype=torch.int32)
    assert launch(m, 0, scratch=other) == 0  # not the stream's buffer: a call's own scratch
    assert launch(m, READ) == 1
    assert launch(m, FRONT) == 1  # a buffer with room for one table: whatever was there is gone
    assert launch(m, READ) == 0
    assert launch(m, WROTE) == 0
    with torch.inference_mode():
        untracked = torch.ones(4, 8, dtype=torch.bool)
    assert launch(untracked, WROTE) == 0  # no version counter: never kept
    assert launch(untracked, WROTE) == 0
    assert launch(m, READ) == 0  # and its pre-pass overwrote place 0
    was = ops.reuse_tile_classes(False)
    try:
        assert launch(m, WROTE) == 0
        assert launch(m, WROTE) == 0
    finally:
        ops.reuse_tile_classes(was)
    a.tma_classify = 2  # an explicit choice of the caller
    assert launch(m, 0) == 0
