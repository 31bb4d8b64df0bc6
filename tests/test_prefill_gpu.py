"""Parity of causal_conv1d_fn (CUDA, through the C ABI) with the CPU oracle.

The grid mirrors the reference's own kernel tests (causal-conv1d-mps/test.py:110-146:
dtype x silu x bias x seqlen{1,2,8,...,256} x dim{64,128,256}, batch 2, seed 42; edge shapes
:206-217; mask recipe :177-180), run for both memory layouts and every kernel of the library,
then widens to the golden vectors made by the reference's CanonLayer and to the benchmark
configurations at full size.
"""
import pytest
import torch

import viby_model_b200 as V
from viby_model_b200 import workloads as WL
from conftest import GOLDEN_CASES
from oracle import canon_oracle as O
from parity import assert_close_to_oracle, exact_fraction

pytestmark = pytest.mark.gpu
DEV = "cuda"


def make(B, D, T, W, dtype, has_bias, seed=42, layout="channel_last", wdtype=None):
    g = torch.Generator().manual_seed(seed)
    if layout == "channel_last":
        x = torch.randn(B, T, D, generator=g).to(dtype).transpose(1, 2)  # [B,D,T] view, channel stride 1
    else:
        x = torch.randn(B, D, T, generator=g).to(dtype)
    w = torch.randn(D, W, generator=g).to(wdtype or dtype)
    b = torch.randn(D, generator=g).to(wdtype or dtype) if has_bias else None
    return x, w, b


def dev(t):
    """Move to the GPU keeping the strides (a transposed view stays a transposed view)."""
    if t is None:
        return None
    out = torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device=DEV)
    out.copy_(t)
    return out


def run_both(x, w, b, act, **kw):
    before = V.launch_count()
    y = V.causal_conv1d_fn(dev(x), dev(w), dev(b), activation=act, **kw)
    # one launch, or two when a masked TMA launch runs its tile-classification pre-pass first
    assert V.launch_count() - before in (1, 2), "the CUDA kernel was not launched"
    return y


# ------------------------------------------------------------------------------------------------
# the reference's grid
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("act", [None, "silu"])
@pytest.mark.parametrize("has_bias", [False, True])
@pytest.mark.parametrize("T", [1, 2, 8, 16, 32, 64, 128, 256])
@pytest.mark.parametrize("D", [64, 128, 256])
@pytest.mark.parametrize("layout", ["channel_last", "time_major"])
def test_reference_grid(D, T, has_bias, act, dtype, layout):
    x, w, b = make(2, D, T, 4, dtype, has_bias, layout=layout)
    y = run_both(x, w, b, act)
    ref = O.causal_conv1d_ref(x, w, b, act)
    assert y.stride() == x.stride()
    assert_close_to_oracle(y, ref, f"{layout} D{D} T{T}")
    vec = 4 if dtype == torch.float32 else 8
    if layout == "channel_last":
        assert V.last_kernel() == "channel_last"
    elif T % vec == 0:
        assert V.last_kernel() == "time_major"
    else:
        assert V.last_kernel() == "generic"


@pytest.mark.parametrize("kernel", ["channel_last", "generic", "tma"])
@pytest.mark.parametrize("W", [2, 3, 4])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 2, 3, 4, 5, 7, 9, 31, 33, 100])
def test_widths_and_short_sequences(T, dtype, W, kernel):
    x, w, b = make(3, 40, T, W, dtype, True, seed=7 + T)
    y = run_both(x, w, b, "silu", kernel=kernel)
    assert V.last_kernel() == kernel
    assert_close_to_oracle(y, O.causal_conv1d_ref(x, w, b, "silu"), f"{kernel} W{W} T{T}")


@pytest.mark.parametrize("W", [2, 3, 4])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T", [8, 64, 1000, 4096 + 64])
def test_time_major_kernel(T, dtype, W):
    x, w, b = make(2, 33, T, W, dtype, True, seed=T, layout="time_major")
    y = run_both(x, w, b, "silu", kernel="time_major")
    assert V.last_kernel() == "time_major"
    assert_close_to_oracle(y, O.causal_conv1d_ref(x, w, b, "silu"), f"time_major W{W} T{T}")


def test_edge_shapes_of_the_reference():
    # causal-conv1d-mps/test.py:206-217
    x, w, b = make(1, 1, 1, 4, torch.float32, True, layout="time_major")
    y = run_both(x, w, b, None)
    assert y.shape == (1, 1, 1)
    assert_close_to_oracle(y, O.causal_conv1d_ref(x, w, b, None))
    x, w, b = make(2, 3, 5, 4, torch.float32, False, layout="time_major")
    y = run_both(x, w, None, None)
    assert y.shape == (2, 3, 5)
    assert_close_to_oracle(y, O.causal_conv1d_ref(x, w, None, None))


def test_empty_inputs_launch_nothing():
    before = V.launch_count()
    for shape in ((0, 8, 4), (2, 0, 4), (2, 8, 0)):
        x = torch.empty(shape, device=DEV, dtype=torch.bfloat16)
        w = torch.zeros(shape[1], 4, device=DEV, dtype=torch.bfloat16)
        y = V.causal_conv1d_fn(x, w)
        assert y.shape == x.shape
    assert V.launch_count() == before


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_odd_layouts_take_the_generic_kernel(dtype):
    g = torch.Generator().manual_seed(3)
    base = torch.randn(2, 50, 21, generator=g).to(dtype)  # dim 21: not a multiple of any vector width
    x = base.transpose(1, 2)
    w = torch.randn(21, 4, generator=g).to(dtype)
    y = run_both(x, w, None, "silu")
    assert V.last_kernel() == "generic"
    assert_close_to_oracle(y, O.causal_conv1d_ref(x, w, None, "silu"))
    # sliced (non-dense) input: every second channel and time step of a larger tensor
    big = torch.randn(2, 16, 64, generator=g).to(dtype)
    xs = big[:, ::2, ::2]
    ws = torch.randn(8, 3, generator=g).to(dtype)
    yd = V.causal_conv1d_fn(dev(big)[:, ::2, ::2], dev(ws), activation=None)
    assert V.last_kernel() == "generic"
    assert_close_to_oracle(yd, O.causal_conv1d_ref(xs, ws, None, None))


def test_fp32_weights_with_16bit_activations():
    # the reference's tests keep weight/bias in fp32 while x is bf16/f16 (test.py:133-136)
    x, w, b = make(2, 64, 33, 4, torch.bfloat16, True, wdtype=torch.float32)
    y = run_both(x, w, b, "silu")
    assert_close_to_oracle(y, O.causal_conv1d_ref(x, w, b, "silu"))


def test_non_contiguous_weight_view():
    # CanonLayer passes weight[D,1,K].squeeze(1); also try a strided slice
    g = torch.Generator().manual_seed(5)
    x = torch.randn(2, 20, 64, generator=g).bfloat16().transpose(1, 2)
    w3 = torch.randn(64, 1, 4, generator=g).bfloat16()
    y = run_both(x, w3.squeeze(1), None, None)
    assert_close_to_oracle(y, O.causal_conv1d_ref(x, w3.squeeze(1), None, None))
    wide = torch.randn(64, 8, generator=g).bfloat16()
    wd = dev(wide)[:, 1:8:2]
    y = V.causal_conv1d_fn(dev(x), wd, activation="silu")
    assert_close_to_oracle(y, O.causal_conv1d_ref(x, wide[:, 1:8:2], None, "silu"))


# ------------------------------------------------------------------------------------------------
# fused options
# ------------------------------------------------------------------------------------------------
def right_pad_mask(B, T, seed, dtype=torch.int64):
    g = torch.Generator().manual_seed(seed)
    m = torch.ones(B, T, dtype=dtype)
    for b in range(B):
        valid = int(torch.randint(max(T // 2, 1), max(T, 2), (1,), generator=g))
        m[b, valid:] = 0
    return m


def check_fused_residual(y_fused, xd, wd, bd, md, ref_conv, kernel):
    """residual=True must equal the reference's two-step `x + y` (model/model.py:491) bit for bit:
    the conv output rounded to the I/O dtype, then the sum rounded again.  The conv term itself is
    held to the oracle; the sum is not compared with the oracle directly, because where x and y
    cancel a 1-ulp difference in y is many ulps of the small sum."""
    y_conv = V.causal_conv1d_fn(xd, wd, bd, activation="silu", attention_mask=md, kernel=kernel)
    assert_close_to_oracle(y_conv, ref_conv, f"{kernel} conv term")
    assert torch.equal(y_fused, xd + y_conv)
    # a separate residual tensor takes the other code path and must agree
    r = xd.clone()
    y_sep = V.causal_conv1d_fn(xd, wd, bd, activation="silu", attention_mask=md, residual=r, kernel=kernel)
    assert torch.equal(y_sep, y_fused)


@pytest.mark.parametrize("kernel", ["channel_last", "generic", "tma"])
@pytest.mark.parametrize("mask_dtype", [torch.int64, torch.bool, torch.int32, torch.uint8, torch.bfloat16,
                                        torch.float32])
@pytest.mark.parametrize("skip", [True, False])
def test_mask_dtypes(mask_dtype, skip, kernel):
    B, D, T = 3, 48, 70
    x, w, b = make(B, D, T, 4, torch.bfloat16, True, seed=11)
    m = right_pad_mask(B, T, 12).to(mask_dtype)
    y = run_both(x, w, b, "silu", attention_mask=dev(m), skip_masked_loads=skip, kernel=kernel)
    ref = O.causal_conv1d_ref(x, w, b, "silu", attention_mask=m)
    assert_close_to_oracle(y, ref, f"mask {mask_dtype} skip={skip}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", ["left", "holes", "all_zero", "fraction"])
def test_mask_patterns(kind, dtype):
    B, D, T = 4, 32, 45
    x, w, b = make(B, D, T, 4, dtype, True, seed=21)
    g = torch.Generator().manual_seed(22)
    if kind == "left":
        m = torch.ones(B, T, dtype=torch.int64)
        for i in range(B):
            m[i, : int(torch.randint(0, T // 2, (1,), generator=g))] = 0
    elif kind == "holes":
        m = (torch.rand(B, T, generator=g) > 0.3).to(torch.int64)
    elif kind == "all_zero":
        m = torch.zeros(B, T, dtype=torch.int64)
    else:  # non-binary multiplier, rounded to the I/O dtype like `x * mask`
        m = (torch.rand(B, T, generator=g) * 2).to(dtype)
    for kernel in ("channel_last", "generic", "tma"):
        y = run_both(x, w, b, "silu", attention_mask=dev(m), kernel=kernel)
        assert_close_to_oracle(y, O.causal_conv1d_ref(x, w, b, "silu", attention_mask=m), f"{kind} {kernel}")


@pytest.mark.parametrize("kernel", ["channel_last", "generic", "tma"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,L", [(1, 4), (2, 4), (3, 3), (4, 4), (5, 8), (40, 4), (40, 8), (40, 3), (7, 8)])
def test_final_state_and_residual(T, L, dtype, kernel):
    B, D = 3, 24
    x, w, b = make(B, D, T, 4, dtype, True, seed=31 + T)
    m = right_pad_mask(B, T, 32)
    xd = dev(x)
    y, st = V.causal_conv1d_fn(xd, dev(w), dev(b), activation="silu", attention_mask=dev(m), residual=True,
                               return_final_states=True, state_len=L, kernel=kernel)
    ref_y, ref_s = O.causal_conv1d_ref(x, w, b, "silu", attention_mask=m, state_len=L)
    check_fused_residual(y, xd, dev(w), dev(b), dev(m), ref_y, kernel)
    assert st.shape == (B, D, L) and st.is_contiguous()
    # bit-exact, sign of zero included: masked negative inputs are -0.0 in the reference
    assert torch.equal(st.cpu().view(torch.int16 if dtype != torch.float32 else torch.int32),
                       ref_s.view(torch.int16 if dtype != torch.float32 else torch.int32))


@pytest.mark.parametrize("kernel", ["channel_last", "generic", "tma"])
@pytest.mark.parametrize("W", [2, 3, 4])
@pytest.mark.parametrize("T2", [1, 2, 5, 37])
def test_initial_states_continue_a_sequence(T2, W, kernel):
    B, D, T1 = 2, 32, 19
    x, w, b = make(B, D, T1 + T2, W, torch.bfloat16, True, seed=41)
    xd, wd, bd = dev(x), dev(w), dev(b)
    y_full, s_full = V.causal_conv1d_fn(xd, wd, bd, activation="silu", return_final_states=True, state_len=W,
                                        kernel=kernel)
    y1, s1 = V.causal_conv1d_fn(xd[..., :T1], wd, bd, activation="silu", return_final_states=True, state_len=W,
                                kernel=kernel)
    y2, s2 = V.causal_conv1d_fn(xd[..., T1:], wd, bd, activation="silu", initial_states=s1,
                                return_final_states=True, state_len=W, kernel=kernel)
    assert torch.equal(torch.cat([y1, y2], -1), y_full)  # same kernel arithmetic: bit-identical
    assert torch.equal(s2, s_full)
    ref_y, ref_s = O.causal_conv1d_ref(x[..., T1:], w, b, "silu", initial_states=s1.cpu(), state_len=W)
    assert_close_to_oracle(y2, ref_y)
    assert torch.equal(s2.cpu(), ref_s)


def test_default_final_state_is_width_minus_one_and_out_argument():
    x, w, b = make(2, 16, 12, 4, torch.float32, False)
    xd = dev(x)
    out = torch.empty_like(xd)
    fs = torch.empty(2, 16, 3, device=DEV)
    y, st = V.causal_conv1d_fn(xd, dev(w), None, final_states_out=fs, out=out)
    assert y is out and st is fs
    assert torch.equal(st.cpu(), x[..., -3:].contiguous())


def test_in_place_output_is_refused():
    x, w, b = make(2, 16, 12, 4, torch.float32, False)
    xd = dev(x)
    with pytest.raises(ValueError, match="VC1D_E_ALIAS"):
        V.causal_conv1d_fn(xd, dev(w), out=xd)


def test_kernels_agree_bit_for_bit():
    """All four prefill kernels accumulate in the same order: identical bits for the same input."""
    g = torch.Generator().manual_seed(9)
    xc = torch.randn(2, 64, 96, generator=g).bfloat16()  # [B,D,T] contiguous
    w = torch.randn(64, 4, generator=g).bfloat16()
    b = torch.randn(64, generator=g).bfloat16()
    xd = xc.to(DEV)
    y_tma = V.causal_conv1d_fn(xd.transpose(1, 2).contiguous().transpose(1, 2), w.to(DEV), b.to(DEV),
                               activation="silu", kernel="tma")
    y_tm = V.causal_conv1d_fn(xd, w.to(DEV), b.to(DEV), activation="silu", kernel="time_major")
    y_g = V.causal_conv1d_fn(xd, w.to(DEV), b.to(DEV), activation="silu", kernel="generic")
    x_cl = xd.transpose(1, 2).contiguous().transpose(1, 2)
    y_cl = V.causal_conv1d_fn(x_cl, w.to(DEV), b.to(DEV), activation="silu", kernel="channel_last")
    assert torch.equal(y_tm, y_g)
    assert torch.equal(y_cl, y_g)
    assert torch.equal(y_tma, y_g)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("W", [2, 3, 4])
@pytest.mark.parametrize("B,T,D", [(3, 700, 960), (2, 129, 640), (5, 64, 3456), (1, 2000, 72), (2, 300, 1000)])
def test_tma_kernel_multi_tile(B, T, D, W, dtype):
    """Several row tiles per persistent CTA, partial last tiles in time and in channels, every
    fused option at once; and the ring survives many wraps (expired waits would be counted)."""
    x, w, b = make(B, D, T, W, dtype, True, seed=B * T + W)
    m = right_pad_mask(B, T, 77)
    m[0, :] = 1
    if B > 2:
        m[2, 5:] = 0  # almost everything masked: tiles that request no bytes at all
    xd = dev(x)
    y, st = V.causal_conv1d_fn(xd, dev(w), dev(b), activation="silu", attention_mask=dev(m), residual=True,
                               return_final_states=True, state_len=W, kernel="tma")
    assert V.last_kernel() == "tma"
    ref_y, ref_s = O.causal_conv1d_ref(x, w, b, "silu", attention_mask=m, state_len=W)
    check_fused_residual(y, xd, dev(w), dev(b), dev(m), ref_y, "tma")
    assert torch.equal(st.cpu(), ref_s)
    # without residual the all-masked tiles take the no-load path; forced narrow / wide slabs agree
    y0 = V.causal_conv1d_fn(xd, dev(w), dev(b), activation="silu", attention_mask=dev(m), kernel="tma")
    assert_close_to_oracle(y0, O.causal_conv1d_ref(x, w, b, "silu", attention_mask=m), "tma no residual")
    # every shape of the kernel: slab width, rows per thread, ring depth, grid size
    for slab in (128, 256):
        for rpt, stages, per_sm in ((8, 3, 3), (8, 2, 1), (4, 3, 3), (4, 5, 6), (8, 8, 2)):
            ys = V.causal_conv1d_fn(xd, dev(w), dev(b), activation="silu", attention_mask=dev(m), kernel="tma",
                                    tma=dict(slab_bytes=slab, rows_per_thread=rpt, stages=stages, ctas_per_sm=per_sm))
            assert torch.equal(ys, y0), (slab, rpt, stages, per_sm)
    # dynamic tile claims from scratch counters: same bits, and the counters are left zeroed, so
    # back-to-back launches on one stream keep working
    for _ in range(3):
        yd = V.causal_conv1d_fn(xd, dev(w), dev(b), activation="silu", attention_mask=dev(m), kernel="tma",
                                dynamic_schedule=True)
        assert torch.equal(yd, y0)
    y_cl = V.causal_conv1d_fn(xd, dev(w), dev(b), activation="silu", attention_mask=dev(m), kernel="channel_last")
    assert torch.equal(y_cl, y0)
    torch.cuda.synchronize()
    assert V.tma_timeouts() == 0


def test_tma_scheduler_scratch_survives_changing_shapes():
    """The scheduler's scratch buffer is shared by every launch of a stream.  A masked launch
    writes class bytes into it; they must never land where a later launch with more channel slabs
    keeps its claim counters (a slab whose counter starts non-zero would be skipped)."""
    shapes = [(4, 2048, 128, torch.float32), (3, 700, 960, torch.bfloat16), (2, 300, 4096, torch.bfloat16),
              (6, 1100, 64, torch.float16), (2, 257, 3456, torch.float32)]
    for rounds in range(2):
        for B, T, D, dtype in shapes:
            x, w, b = make(B, D, T, 4, dtype, True, seed=T)
            m = right_pad_mask(B, T, T + rounds)
            xd = dev(x)
            for mask in (dev(m), None):
                y = torch.full_like(xd, float("nan"))
                V.causal_conv1d_fn(xd, dev(w), dev(b), activation="silu", attention_mask=mask, kernel="tma",
                                   dynamic_schedule=True, out=y)
                y_static = V.causal_conv1d_fn(xd, dev(w), dev(b), activation="silu", attention_mask=mask,
                                              kernel="tma", dynamic_schedule=False)
                assert torch.equal(y, y_static), (B, T, D, dtype, mask is None)
    torch.cuda.synchronize()
    assert V.tma_timeouts() == 0


def test_tma_masked_rows_are_never_read():
    x, w, b = make(2, 256, 300, 4, torch.bfloat16, True, seed=5)
    m = right_pad_mask(2, 300, 6)
    xd = dev(x)
    y = V.causal_conv1d_fn(xd, dev(w), dev(b), activation="silu", attention_mask=dev(m), kernel="tma")
    xn = xd.clone()
    xn.transpose(1, 2)[~dev(m).bool()] = float("nan")
    yn = V.causal_conv1d_fn(xn, dev(w), dev(b), activation="silu", attention_mask=dev(m), kernel="tma")
    assert torch.equal(yn, y)
    # with skip_masked_loads off the reference's x * 0 semantics apply: NaN * 0 is NaN
    yk = V.causal_conv1d_fn(xn, dev(w), dev(b), activation="silu", attention_mask=dev(m), kernel="tma",
                            skip_masked_loads=False)
    assert bool(yk.isnan().any())


# ------------------------------------------------------------------------------------------------
# golden vectors made by the reference's CanonLayer
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("c", GOLDEN_CASES, ids=[repr(c) for c in GOLDEN_CASES])
def test_golden_canon_layer_prefill(c):
    """CanonLayer's CUDA branch rebuilt from the kernel (model/model.py:426-491): mask fused,
    state of kernel_size columns, residual; compared with the recorded output of the
    reference's PyTorch branch at the valid positions (the two branches differ at padded
    positions by construction: masked vs unmasked residual)."""
    x = c.get("x")
    w = c.get("weight")
    b = c.get("bias") if c.has("bias") else None
    m = c.get("mask") if c.has("mask") else None
    act = "silu" if c.activation else None
    xd = dev(x)
    y, st = V.causal_conv1d_fn(xd.transpose(1, 2), dev(w), dev(b), activation=act,
                               attention_mask=dev(m), return_final_states=True, state_len=8)
    out = (xd + y.transpose(1, 2)).cpu()
    ref = c.get("prefill_cache_out")
    valid = m.bool().unsqueeze(-1).expand_as(ref) if m is not None else torch.ones_like(ref, dtype=torch.bool)
    if c.dtype == torch.float32:
        assert torch.allclose(out[valid], ref[valid], rtol=1e-5, atol=1e-6)
    else:
        assert torch.allclose(out[valid].float(), ref[valid].float(), rtol=2 ** -6, atol=2 ** -6)
    if c.T > 1:
        assert torch.equal(st.cpu(), c.get("prefill_state"))


# ------------------------------------------------------------------------------------------------
# the benchmark configurations at full size
# ------------------------------------------------------------------------------------------------
def test_config1_canon_b_fp32_both_layouts():
    cfg = WL.CANON_B_FP32
    x_btd = WL.prefill_inputs(cfg)
    w, b = WL.weights(cfg.cfg, cfg.dim, cfg.width, cfg.dtype)
    ref = O.causal_conv1d_ref(x_btd.transpose(1, 2), w, b, None)
    y = V.causal_conv1d_fn(x_btd.to(DEV).transpose(1, 2), w.to(DEV), b.to(DEV))
    assert V.last_kernel() == "tma"
    assert_close_to_oracle(y, ref, "cfg1 channel-last")
    y1 = V.causal_conv1d_fn(x_btd.to(DEV).transpose(1, 2), w.to(DEV), b.to(DEV), kernel="channel_last")
    assert torch.equal(y1, y)
    x_bdt = x_btd.transpose(1, 2).contiguous()
    y2 = V.causal_conv1d_fn(x_bdt.to(DEV), w.to(DEV), b.to(DEV))
    assert V.last_kernel() == "time_major"
    assert_close_to_oracle(y2, ref.contiguous(), "cfg1 contiguous")


@pytest.mark.parametrize("kernel", [None, "channel_last", "tma"])
def test_config2_canon_d_prefill_bf16(kernel):
    cfg = WL.CANON_D_PREFILL
    x_btd = WL.prefill_inputs(cfg)
    m = WL.attention_mask(cfg)
    w, b = WL.weights(cfg.cfg, cfg.dim, cfg.width, cfg.dtype)
    ref, ref_s = O.causal_conv1d_ref(x_btd.transpose(1, 2), w, b, "silu", attention_mask=m, state_len=4)
    xd = x_btd.to(DEV)
    y, st = V.causal_conv1d_fn(xd.transpose(1, 2), w.to(DEV), b.to(DEV), activation="silu",
                               attention_mask=m.to(DEV), return_final_states=True, state_len=4, kernel=kernel)
    assert V.last_kernel() == (kernel or "tma")
    assert_close_to_oracle(y, ref, "cfg2")
    assert exact_fraction(y, ref) > 0.999
    assert torch.equal(st.cpu(), ref_s)
    # unfused flow of the reference's CUDA branch: mask multiply outside, plain kernel call
    y_plain = V.causal_conv1d_fn((xd * m.to(DEV).unsqueeze(-1)).transpose(1, 2), w.to(DEV), b.to(DEV),
                                 activation="silu")
    assert torch.equal(y_plain, y)


def test_config5_ragged_shard_properties():
    """One GPU's share of the ragged sweep at 8 GPUs (64 sequences x 4096 x 3456): sampled
    sequences against the oracle, plus properties that need no oracle at this size."""
    cfg = WL.RAGGED_SWEEP
    rows = list(WL.shard_rows(cfg.batch, 3, 8))
    assert len(rows) == 64
    x = WL.prefill_inputs(cfg, rows, device=DEV, generate_on="cuda")
    m = WL.attention_mask(cfg, rows, device=DEV)
    w, b = WL.weights(cfg.cfg, cfg.dim, cfg.width, cfg.dtype, device=DEV)
    y = V.causal_conv1d_fn(x.transpose(1, 2), w, b, activation="silu", attention_mask=m)
    lens = WL.sequence_lengths(cfg, rows)
    # (1) against the oracle: every sequence of up to 256 valid steps and the 8 longest ones, over their
    # valid steps plus the width-1 steps behind them (what follows is checked as a constant in (2))
    order = sorted(range(len(rows)), key=lambda i: int(lens[i]))
    check = [i for i in order if int(lens[i]) <= 256] + order[-8:]
    assert len(check) >= 20
    wc, bc = w.cpu(), b.cpu()
    for i in check:
        n = min(cfg.seqlen, int(lens[i]) + cfg.width - 1)
        ref = O.causal_conv1d_ref(x[i:i + 1, :n].cpu().transpose(1, 2), wc, bc, "silu",
                                  attention_mask=m[i:i + 1, :n].cpu())
        assert_close_to_oracle(y[i:i + 1, :, :n], ref, f"cfg5 row {rows[i]} len {int(lens[i])}")
    # (2) beyond len+W-1 every output is act(bias): constant along time
    const = torch.nn.functional.silu(b.float()).to(cfg.dtype)
    for i in range(len(rows)):
        n = int(lens[i]) + cfg.width - 1
        if n < cfg.seqlen:
            tail = y[i, :, n:]
            assert bool(((tail.float() - const.float()[:, None]).abs() <= 2 ** -7 * const.float().abs()[:, None]
                         + 1e-6).all())
    # (3) causality: changing the last valid token changes nothing before it
    x2 = x.clone()
    for i in range(len(rows)):
        x2[i, int(lens[i]) - 1] += 1
    y2 = V.causal_conv1d_fn(x2.transpose(1, 2), w, b, activation="silu", attention_mask=m)
    for i in (1, 30, 62):
        n = int(lens[i]) - 1
        assert torch.equal(y2[i, :, :n], y[i, :, :n])
        assert not torch.equal(y2[i, :, n], y[i, :, n])
    # (4) garbage in padded rows is never observed
    x3 = x.clone()
    x3[~m.bool()] = float("nan")
    y3 = V.causal_conv1d_fn(x3.transpose(1, 2), w, b, activation="silu", attention_mask=m)
    assert torch.equal(y3, y)
    # (5) sharding is invisible: a sub-batch gives the same bits
    y_sub = V.causal_conv1d_fn(x[8:24].transpose(1, 2), w, b, activation="silu", attention_mask=m[8:24])
    assert torch.equal(y_sub, y[8:24])


def test_multi_tensor_call_equals_concatenated_call():
    """q | k | v (or gate | up) given as separate tensors: same bits as the reference's cat-conv-split."""
    g = torch.Generator().manual_seed(21)
    B, T = 3, 200
    dims = (640, 160, 160)
    xs = [torch.randn(B, T, d, generator=g).to(torch.bfloat16).to(DEV) for d in dims]
    w = torch.randn(sum(dims), 4, generator=g).to(torch.bfloat16).to(DEV)
    b = torch.randn(sum(dims), generator=g).to(torch.bfloat16).to(DEV)
    m = dev(right_pad_mask(B, T, 3))
    cat = torch.cat(xs, dim=-1)
    ref = V.causal_conv1d_fn(cat.transpose(1, 2), w, b, activation="silu", attention_mask=m, residual=True)
    outs = V.causal_conv1d_fn_multi([x.transpose(1, 2) for x in xs], w, b, activation="silu", attention_mask=m,
                                    residual=True)
    d0 = 0
    for o, d in zip(outs, dims):
        assert torch.equal(o, ref[:, d0:d0 + d])
        d0 += d


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_tma_chunked_continuation_with_masks(dtype):
    """A long prefill cut into chunks that hand their state on (the reference's chunked continuation,
    model/model.py:607-661), several tiles per chunk, masked tails: every chunk through the TMA-staged
    kernel equals the register-window kernel and the oracle, outputs and states."""
    B, D, W, L = 3, 640, 4, 4
    chunks = (200, 1, 130, 77)
    T = sum(chunks)
    x, w, b = make(B, D, T, W, dtype, True, seed=77)
    m = right_pad_mask(B, T, 9)
    m[1, 150:] = 0  # a sequence whose later chunks are entirely masked: first tile still sees history
    xd, wd, bd, md = dev(x), dev(w), dev(b), dev(m)
    states = {"tma": None, "channel_last": None}
    ref_state = None
    t0 = 0
    for n in chunks:
        sl = slice(t0, t0 + n)
        outs = {}
        for kernel in states:
            y, st = V.causal_conv1d_fn(xd[..., sl], wd, bd, activation="silu", attention_mask=md[:, sl],
                                       initial_states=states[kernel], return_final_states=True, state_len=L,
                                       kernel=kernel)
            assert V.last_kernel() == kernel
            outs[kernel] = y
            states[kernel] = st
        assert torch.equal(outs["tma"], outs["channel_last"])
        assert torch.equal(states["tma"], states["channel_last"])
        ref_y, ref_state = O.causal_conv1d_ref(x[..., sl], w, b, "silu", attention_mask=m[:, sl],
                                               initial_states=ref_state, state_len=L)
        assert_close_to_oracle(outs["tma"], ref_y)
        assert torch.equal(states["tma"].cpu(), ref_state)
        t0 += n
    torch.cuda.synchronize()
    assert V.tma_timeouts() == 0


def _mask_of_kind(kind, B, T, seed):
    g = torch.Generator().manual_seed(seed)
    if kind == "right":
        lens = torch.randint(1, T + 1, (B,), generator=g)
        lens[0], lens[1] = T, 3
        return torch.arange(T)[None, :] < lens[:, None]
    if kind == "left":
        lens = torch.randint(1, T + 1, (B,), generator=g)
        return torch.arange(T)[None, :] >= (T - lens)[:, None]
    if kind == "holes":
        m = torch.rand(B, T, generator=g) > 0.02
        m[2, 100:400] = False  # a stretch long enough to hold tiles without any live tap
        return m
    if kind == "zeros":
        return torch.zeros(B, T, dtype=torch.bool)
    return torch.ones(B, T, dtype=torch.bool)


@pytest.mark.parametrize("tma", [dict(empty_store=1), dict(empty_store=2), dict(classify=1), dict(classify=2), dict(static_first=3),
                                 dict(classify=1, empty_store=1),
                                 dict(claim_chunk=2), dict(claim_chunk=4, empty_store=1),
                                 dict(classify=2, static_first=2, pdl=2), dict(rows_per_thread=4, empty_store=2)],
                         ids=lambda d: ",".join(f"{k}={v}" for k, v in d.items()))
@pytest.mark.parametrize("mask_kind", ["right", "left", "holes", "zeros", "ones"])
@pytest.mark.parametrize("mask_dtype,D", [(torch.bool, 1160), (torch.int64, 1160), (torch.bool, 960)])
def test_tma_scheduling_variants_agree(mask_dtype, D, mask_kind, tma):
    """Every way the TMA-staged kernel can hand out, classify and store its tiles gives the bits of the
    register-window kernel: bulk-stored or consumer-stored constant tiles, tiles handed out from the
    pre-pass's list ordered by cost (the default at this size) or in their natural order with a class byte
    each, classes worked out inside the kernel, chunked claims, unclaimed first tiles.  The second and third
    launch of each case use the list or table that the first one left.  The shapes have a
    last time tile that is not full and either a last 256-byte channel slab that is half outside the
    tensor (1160 channels) or 128-byte slabs and 128-row tiles (960 channels, the Canon-B width)."""
    B, T, W = 20, 1008, 4
    x = O.seeded((B, T, D), 77, "normal", torch.bfloat16)
    w = O.seeded((D, W), 78, "uniform", torch.bfloat16)
    b = O.seeded((D,), 79, "uniform", torch.bfloat16)
    m = _mask_of_kind(mask_kind, B, T, 80).to(mask_dtype)
    xd, wd, bd, md = dev(x).transpose(1, 2), dev(w), dev(b), dev(m)
    ref = V.causal_conv1d_fn(xd, wd, bd, activation="silu", attention_mask=md, kernel="channel_last")
    before = V.launch_count()
    y = V.causal_conv1d_fn(xd, wd, bd, activation="silu", attention_mask=md, kernel="tma", tma=tma,
                           dynamic_schedule=True)
    assert V.last_kernel() == "tma"
    if tma.get("classify") == 2 and mask_dtype == torch.bool:
        assert V.launch_count() - before == 1, "the kernel classifies its tiles itself: no pre-pass launch"
    assert torch.equal(y, ref)
    # twice more on the same stream: the scratch counters were left zeroed
    for _ in range(2):
        y2 = V.causal_conv1d_fn(xd, wd, bd, activation="silu", attention_mask=md, kernel="tma", tma=tma,
                                dynamic_schedule=True)
        assert torch.equal(y2, ref)
    torch.cuda.synchronize()
    assert V.tma_timeouts() == 0


@pytest.mark.parametrize("B", [64, 65, 300])
def test_tma_class_table_of_a_very_long_batch(B):
    """The three forms in which a CTA holds the pre-pass's result: the ordered tile list (up to 4096 tiles:
    batch 64 here is exactly that many), a class byte per tile (4160 tiles), and, beyond the 16384 bytes a
    CTA spends on that, two bits per tile (19200 tiles).  Against the register-window kernel."""
    T, D = 4096, 256
    g = torch.Generator(device=DEV).manual_seed(3)
    x = torch.randn(B, T, D, generator=g, device=DEV).bfloat16()
    w = dev(O.seeded((D, 4), 5, "uniform", torch.bfloat16))
    b = dev(O.seeded((D,), 6, "uniform", torch.bfloat16))
    lens = torch.randint(1, T + 1, (B,), generator=torch.Generator().manual_seed(4))
    m = (torch.arange(T)[None, :] < lens[:, None]).to(DEV)
    m[5, 50:700] = False
    ref = V.causal_conv1d_fn(x.transpose(1, 2), w, b, activation="silu", attention_mask=m, kernel="channel_last")
    before = V.launch_count()
    y = V.causal_conv1d_fn(x.transpose(1, 2), w, b, activation="silu", attention_mask=m, kernel="tma")
    assert V.launch_count() - before == 2 and V.last_kernel() == "tma"
    assert torch.equal(y, ref)
    torch.cuda.synchronize()
    assert V.tma_timeouts() == 0


def test_tile_classes_are_kept_while_the_mask_is_unchanged():
    """Consecutive masked launches on one stream share their tile classes: the pre-pass runs for the first
    of them and again as soon as anything the classes depend on differs (mask written in place, another
    mask of equal contents, another sequence length, a backward launch in between), not when only the
    channel count differs (a model's Canon calls A-D share the mask; each tile height has its own table).  Every result bit-equal to a launch
    with the sharing switched off."""
    B, T, W = 64, 1024, 4  # enough tiles per CTA for dynamic claims, which is what the class table serves
    g = torch.Generator(device=DEV).manual_seed(11)
    xs = {D: torch.randn(B, T, D, generator=g, device=DEV).bfloat16() for D in (640, 960)}
    ws = {D: dev(O.seeded((D, W), D, "uniform", torch.bfloat16)) for D in xs}
    bs = {D: dev(O.seeded((D,), D + 1, "uniform", torch.bfloat16)) for D in xs}
    lens = torch.randint(1, T + 1, (B,), generator=torch.Generator().manual_seed(12))
    m = (torch.arange(T)[None, :] < lens[:, None]).to(DEV)

    def run(D, mask, **kw):
        before = V.launch_count()
        y = V.causal_conv1d_fn(xs[D].transpose(1, 2), ws[D], bs[D], activation="silu", attention_mask=mask, **kw)
        assert V.last_kernel() == "tma"
        return y, V.launch_count() - before

    def fresh(D, mask):
        was = V.reuse_tile_classes(False)
        try:
            y, n = run(D, mask)
        finally:
            V.reuse_tile_classes(was)
        assert n == 2
        return y

    want = {D: fresh(D, m) for D in xs}
    y, n = run(640, m)
    assert n == 2 and torch.equal(y, want[640])  # pre-pass + main kernel
    y, n = run(960, m)
    assert n == 2 and torch.equal(y, want[960])  # 128-byte channel slabs, tiles twice as high: a table of its own
    for D in (640, 960, 640, 960):
        y, n = run(D, m)
        assert n == 1 and torch.equal(y, want[D]), D  # the classes that an earlier launch left
    # the mask written in place: torch counts it, the classes are worked out again
    m[3, :] = False
    m[4, 100:900] = False
    want = {D: fresh(D, m) for D in xs}
    y, n = run(960, m)
    assert n == 2 and torch.equal(y, want[960])
    y, n = run(960, m)
    assert n == 1 and torch.equal(y, want[960])
    # a view of the same memory is the same mask; another tensor of equal contents is not
    y, n = run(640, m)
    assert n == 2 and torch.equal(y, want[640])
    y, n = run(640, m[:, :])
    assert n == 1 and torch.equal(y, want[640])
    m2 = m.clone()
    y, n = run(640, m2)
    assert n == 2 and torch.equal(y, want[640])
    # a mask that dies and one of other contents that may take its place in memory
    del m2
    m3 = ~m
    m3[:, 0] = True
    want3 = fresh(640, m3)
    y, n = run(640, m3)
    assert n == 2 and torch.equal(y, want3)
    # other options that the classes depend on
    y, n = run(640, m3)
    assert n == 1
    y, n = run(640, m3, residual=True)
    assert n == 2 and torch.equal(y, V.causal_conv1d_fn(xs[640].transpose(1, 2), ws[640], bs[640], activation="silu",
                                                        attention_mask=m3, residual=True, kernel="channel_last"))
    # a backward launch between two forward launches writes its own classes to the same scratch memory
    y, n = run(640, m3)
    assert n == 2
    V.causal_conv1d_bwd(xs[640].transpose(1, 2), ws[640], bs[640], torch.ones_like(xs[640]).transpose(1, 2), "silu",
                        attention_mask=m3, kernel="tma")
    y, n = run(640, m3)
    assert n == 2 and torch.equal(y, want3)
    # a shorter batch with a mask at the same address and version: another number of tiles
    xs_short = xs[640][:, :512]
    before = V.launch_count()
    y = V.causal_conv1d_fn(xs_short.transpose(1, 2), ws[640], bs[640], activation="silu", attention_mask=m3[:, :512])
    assert V.launch_count() - before == 2
    assert torch.equal(y, V.causal_conv1d_fn(xs_short.transpose(1, 2), ws[640], bs[640], activation="silu",
                                             attention_mask=m3[:, :512], kernel="channel_last"))
    torch.cuda.synchronize()
    assert V.tma_timeouts() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("mask_dtype", [torch.bool, torch.int64, torch.float32])
def test_ordered_tile_list_in_the_other_dtypes(dtype, mask_dtype):
    """The ordered tile list and its reuse for fp32 and fp16 tensors (other channel counts per slab) and for
    masks of other types: pre-pass on the first launch only, results bit-equal to the register-window kernel."""
    B, T, D, W = 48, 1000, 520, 4
    g = torch.Generator(device=DEV).manual_seed(17)
    x = torch.randn(B, T, D, generator=g, device=DEV).to(dtype)
    w = dev(O.seeded((D, W), 18, "uniform", dtype))
    b = dev(O.seeded((D,), 19, "uniform", dtype))
    m = dev(_mask_of_kind("right", B, T, 20).to(mask_dtype))
    ref = V.causal_conv1d_fn(x.transpose(1, 2), w, b, activation="silu", attention_mask=m, kernel="channel_last")
    counts = []
    for _ in range(3):
        before = V.launch_count()
        y = V.causal_conv1d_fn(x.transpose(1, 2), w, b, activation="silu", attention_mask=m, kernel="tma")
        counts.append(V.launch_count() - before)
        assert V.last_kernel() == "tma" and torch.equal(y, ref)
    assert counts == [2, 1, 1]
    torch.cuda.synchronize()
    assert V.tma_timeouts() == 0


def test_kept_tile_classes_and_cuda_graphs():
    """A captured launch never relies on classes from outside its graph: replays stay correct after eager
    launches with other masks have used the stream's scratch memory."""
    B, T, D = 64, 1024, 640
    g = torch.Generator(device=DEV).manual_seed(13)
    x = torch.randn(B, T, D, generator=g, device=DEV).bfloat16()
    w = dev(O.seeded((D, 4), 5, "uniform", torch.bfloat16))
    lens = torch.randint(1, T + 1, (B,), generator=torch.Generator().manual_seed(14))
    m = (torch.arange(T)[None, :] < lens[:, None]).to(DEV)
    other = ~m
    want = V.causal_conv1d_fn(x.transpose(1, 2), w, None, activation="silu", attention_mask=m, kernel="channel_last")
    want_other = V.causal_conv1d_fn(x.transpose(1, 2), w, None, activation="silu", attention_mask=other, kernel="channel_last")
    y = torch.empty_like(x)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        V.causal_conv1d_fn(x.transpose(1, 2), w, None, activation="silu", attention_mask=m, out=y.transpose(1, 2))
        V.causal_conv1d_fn(x.transpose(1, 2), w, None, activation="silu", attention_mask=m, out=y.transpose(1, 2))
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            V.causal_conv1d_fn(x.transpose(1, 2), w, None, activation="silu", attention_mask=m, out=y.transpose(1, 2))
            V.causal_conv1d_fn(x.transpose(1, 2), w, None, activation="silu", attention_mask=m, out=y.transpose(1, 2))
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(2):
        with torch.cuda.stream(side):
            z = V.causal_conv1d_fn(x.transpose(1, 2), w, None, activation="silu", attention_mask=other)
            assert torch.equal(z, want_other)
            side.synchronize()
        y.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(y.transpose(1, 2), want)
        with torch.cuda.stream(side):
            z = V.causal_conv1d_fn(x.transpose(1, 2), w, None, activation="silu", attention_mask=m)
            assert torch.equal(z, want)
    assert V.tma_timeouts() == 0


def test_kept_tile_classes_on_two_streams():
    """Two streams with a mask each, launches interleaved from one host thread: every stream has its own
    scratch memory and its own record of kept tables, so neither sees the other's classes."""
    B, T, D = 64, 1024, 640
    g = torch.Generator(device=DEV).manual_seed(21)
    x = torch.randn(B, T, D, generator=g, device=DEV).bfloat16()
    w = dev(O.seeded((D, 4), 5, "uniform", torch.bfloat16))
    b = dev(O.seeded((D,), 6, "uniform", torch.bfloat16))
    lens = torch.randint(1, T + 1, (B,), generator=torch.Generator().manual_seed(22))
    masks = [(torch.arange(T)[None, :] < lens[:, None]).to(DEV), (torch.arange(T)[None, :] >= (T - lens)[:, None]).to(DEV)]
    want = [V.causal_conv1d_fn(x.transpose(1, 2), w, b, activation="silu", attention_mask=m, kernel="channel_last") for m in masks]
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    outs = [[], []]
    counts = [[], []]
    for it in range(6):
        for k in (0, 1):
            with torch.cuda.stream(streams[k]):
                before = V.launch_count()
                outs[k].append(V.causal_conv1d_fn(x.transpose(1, 2), w, b, activation="silu", attention_mask=masks[k]))
                counts[k].append(V.launch_count() - before)
    torch.cuda.synchronize()
    for k in (0, 1):
        assert counts[k] == [2, 1, 1, 1, 1, 1], counts[k]
        for y in outs[k]:
            assert torch.equal(y, want[k])
    assert V.tma_timeouts() == 0


def test_bounded_waits_expire_and_report():
    """Failure detection of the TMA-staged kernel, provoked without faulting anything: with the
    self-test switch every producer warp withholds its first tile and every wait polls only 4096 times,
    so the consumers' wait for that tile (and then the producer's wait for the slot) runs out.  The
    kernel must come back normally, the device counter read by tma_timeouts() must have grown, and
    the next ordinary launch must be clean and correct.  Runs in a child process: the counter is
    cumulative, and every other test asserts that it is still zero."""
    import subprocess
    import sys

    code = r'''
import torch
import viby_model_b200 as V
dev = "cuda"
g = torch.Generator().manual_seed(1)
x = torch.randn(8, 512, 1152, generator=g).bfloat16().to(dev)
w = (torch.rand(1152, 4, generator=g) - 0.5).bfloat16().to(dev)
m = (torch.arange(512)[None, :] < torch.randint(1, 513, (8,), generator=g)[:, None]).to(dev)
ref = V.causal_conv1d_fn(x.transpose(1, 2), w, None, activation="silu", attention_mask=m, kernel="channel_last")
assert V.tma_timeouts() == 0
V.causal_conv1d_fn(x.transpose(1, 2), w, None, activation="silu", attention_mask=m, kernel="tma", tma=dict(test_expire=1))
torch.cuda.synchronize()          # the launch returns: nothing hangs, nothing traps
expired = V.tma_timeouts()
assert expired > 0, "the expired waits were not reported"
y = V.causal_conv1d_fn(x.transpose(1, 2), w, None, activation="silu", attention_mask=m, kernel="tma")
torch.cuda.synchronize()
assert V.tma_timeouts() == expired, "an ordinary launch after the self-test reported expired waits"
assert torch.equal(y, ref)
print("EXPIRED", expired)
'''
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300,
                       cwd=str(__import__("conftest").ROOT))
    assert r.returncode == 0, r.stdout + r.stderr
    assert "EXPIRED" in r.stdout


def test_config5_full_batch_addresses_beyond_32_bits():
    """The whole ragged configuration on one GPU: 512 x 4096 x 3456 bf16 = 14.5 GB in, 14.5 GB out, so byte
    offsets pass 2^32 and the launch has 32768 tiles per channel slab (two-bit class table).  Sequences from
    the start, the middle and the end of the batch must equal the same sequences launched on their own
    (small offsets, byte-per-tile table), and the packed launch of the whole batch must agree with both."""
    cfg = WL.RAGGED_SWEEP
    free, _ = torch.cuda.mem_get_info()
    if free < 40 * 2 ** 30:
        pytest.skip("needs 40 GB of free device memory")
    lens = WL.sequence_lengths(cfg).tolist()
    x = WL.prefill_inputs(cfg, device=DEV, generate_on="cuda")
    m = WL.attention_mask(cfg, device=DEV, dtype=torch.bool)
    w, b = WL.weights(cfg.cfg, cfg.dim, cfg.width, cfg.dtype, device=DEV)
    assert x.numel() * x.element_size() > 2 ** 33
    before = V.launch_count()
    y = V.causal_conv1d_fn(x.transpose(1, 2), w, b, activation="silu", attention_mask=m)
    assert V.launch_count() - before == 2 and V.last_kernel() == "tma"
    for i in (0, 1, 255, 256, 300, 510, 511):
        yi = V.causal_conv1d_fn(x[i:i + 1].transpose(1, 2), w, b, activation="silu", attention_mask=m[i:i + 1])
        assert torch.equal(yi, y[i:i + 1]), f"sequence {i}"
    y = y.transpose(1, 2)  # [B, T, D]
    xp = torch.cat([x[i, :n] for i, n in enumerate(lens)], 0).unsqueeze(0)
    ids = V.seq_idx_from_lengths(lens, device=DEV)
    yp = V.causal_conv1d_fn(xp.transpose(1, 2), w, b, activation="silu", seq_idx=ids).transpose(1, 2)
    at = 0
    for i, n in enumerate(lens):
        if i % 37 == 0 or i > 505:
            assert torch.equal(yp[0, at:at + n], y[i, :n]), f"packed sequence {i}"
        at += n
    torch.cuda.synchronize()
    assert V.tma_timeouts() == 0
