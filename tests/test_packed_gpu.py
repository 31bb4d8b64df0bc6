"""Packed variable-length prefill (``seq_idx``; signature causal-conv1d-mps/causal_conv1d_mps/
autograd.py:501-510) on the GPU, through the C ABI: sequences laid end to end in one row must give
what a right-padded batch gives at its valid positions (the reference's prefill,
model/model.py:454-466), and what the CPU oracle gives for each sequence on its own.
"""
import pytest
import torch

import viby_model_b200 as V
from viby_model_b200 import workloads as WL
from conftest import GOLDEN_CASES
from oracle import canon_oracle as O
from parity import assert_close_to_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


def pack(x_btd, lens):
    rows = [x_btd[b, :n] for b, n in enumerate(lens)]
    return torch.cat(rows, 0).unsqueeze(0).contiguous()


@pytest.mark.parametrize("kernel", [None, "generic", "tma"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("W", [2, 3, 4])
def test_packed_rows_against_oracle(W, dtype, kernel):
    """Lengths that put sequence starts at every position of a thread's rows, at tile edges, one or
    two steps apart, and right at the end of the row."""
    D = 256 if dtype != torch.float32 else 128
    lens = [1, 1, 2, 3, 64, 1, 63, 65, 5, 128, 7, 8, 9, 190, 2, 1, 66, 1]
    x = O.seeded((1, sum(lens), D), 21, "normal", dtype)
    w = O.seeded((D, W), 22, "uniform", dtype)
    b = O.seeded((D,), 23, "uniform", dtype)
    ids = V.seq_idx_from_lengths(lens)
    before = V.launch_count()
    y = V.causal_conv1d_fn(x.to(DEV).transpose(1, 2), w.to(DEV), b.to(DEV), seq_idx=ids.to(DEV), activation="silu",
                           kernel=kernel)
    assert V.launch_count() > before
    if kernel is not None:
        assert V.last_kernel() == kernel
    ref = O.causal_conv1d_packed_ref(x.transpose(1, 2), w, b, "silu", seq_idx=ids)
    assert_close_to_oracle(y, ref, f"packed W{W} {dtype} {kernel}")
    torch.cuda.synchronize()
    assert V.tma_timeouts() == 0


@pytest.mark.parametrize("dynamic", [False, True])
def test_packed_equals_padded_batch_bit_for_bit(dynamic):
    """The same sequences as a right-padded masked batch and as one packed row: equal bits at every
    valid position (both through the TMA-staged kernel)."""
    B, T, D, W = 24, 512, 1152, 4
    g = torch.Generator().manual_seed(5)
    lens = torch.randint(1, T + 1, (B,), generator=g).tolist()
    lens[3], lens[7] = T, 1
    x = O.seeded((B, T, D), 31, "normal", torch.bfloat16)
    w = O.seeded((D, W), 32, "uniform", torch.bfloat16).to(DEV)
    b = O.seeded((D,), 33, "uniform", torch.bfloat16).to(DEV)
    m = (torch.arange(T)[None, :] < torch.tensor(lens)[:, None])
    y_pad = V.causal_conv1d_fn(x.to(DEV).transpose(1, 2), w, b, activation="silu", attention_mask=m.to(DEV),
                               kernel="tma", dynamic_schedule=dynamic).transpose(1, 2)
    xp = pack(x, lens)
    ids = V.seq_idx_from_lengths(lens, device=DEV)
    y_pk = V.causal_conv1d_fn(xp.to(DEV).transpose(1, 2), w, b, activation="silu", seq_idx=ids, kernel="tma",
                              dynamic_schedule=dynamic).transpose(1, 2)
    assert V.last_kernel() == "tma"
    at = 0
    for bi, n in enumerate(lens):
        assert torch.equal(y_pk[0, at:at + n], y_pad[bi, :n]), f"sequence {bi} (length {n})"
        at += n
    ref = O.causal_conv1d_packed_ref(xp.transpose(1, 2), w.cpu(), b.cpu(), "silu", seq_idx=ids.cpu())
    assert_close_to_oracle(y_pk.transpose(1, 2), ref, "packed vs oracle")


RIGHT_PADDED = [c for c in GOLDEN_CASES if c.has("mask") and c.mask == "right"]


@pytest.mark.parametrize("c", RIGHT_PADDED, ids=[repr(c) for c in RIGHT_PADDED])
def test_packed_golden_cases(c):
    """The right-padded golden cases of the reference's CanonLayer, packed: the conv term plus the
    input reproduces the reference's prefill output at the valid positions."""
    x, w = c.get("x"), c.get("weight")
    b = c.get("bias") if c.has("bias") else None
    m = c.get("mask")
    act = "silu" if c.activation else None
    lens = [int(v) for v in (m != 0).sum(1)]
    if sum(lens) == 0:
        pytest.skip("no valid position")
    xp = pack(x, lens)
    ids = V.seq_idx_from_lengths(lens, device=DEV)
    y = V.causal_conv1d_fn(xp.to(DEV).transpose(1, 2), w.to(DEV), None if b is None else b.to(DEV), seq_idx=ids,
                           activation=act).transpose(1, 2).cpu()
    ref = c.get("prefill_out")
    at = 0
    for bi, n in enumerate(lens):
        out = x[bi, :n] + y[0, at:at + n]
        if c.dtype == torch.float32:
            assert torch.allclose(out, ref[bi, :n], rtol=1e-5, atol=1e-6)
        else:
            assert torch.allclose(out.float(), ref[bi, :n].float(), rtol=2 ** -6, atol=2 ** -6)
        at += n


def test_packed_shard_of_the_ragged_sweep():
    """One GPU's share (64 sequences) of the ragged large-batch configuration, packed: 1/5 of the
    padded rows.  Every sequence up to 256 steps and 8 long ones against the oracle; all of them
    against the padded launch."""
    cfg = WL.RAGGED_SWEEP
    rows = list(WL.shard_rows(cfg.batch, 3, 8))
    lens = WL.sequence_lengths(cfg, rows).tolist()
    x = WL.prefill_inputs(cfg, rows, device=DEV, generate_on="cuda")
    m = WL.attention_mask(cfg, rows, device=DEV, dtype=torch.bool)
    w, b = WL.weights(cfg.cfg, cfg.dim, cfg.width, cfg.dtype, device=DEV)
    y_pad = V.causal_conv1d_fn(x.transpose(1, 2), w, b, activation="silu", attention_mask=m).transpose(1, 2)
    xp = torch.cat([x[i, :n] for i, n in enumerate(lens)], 0).unsqueeze(0)
    ids = V.seq_idx_from_lengths(lens, device=DEV)
    y_pk = V.causal_conv1d_fn(xp.transpose(1, 2), w, b, activation="silu", seq_idx=ids).transpose(1, 2)
    assert V.last_kernel() == "tma"
    at, starts = 0, []
    for i, n in enumerate(lens):
        assert torch.equal(y_pk[0, at:at + n], y_pad[i, :n]), f"sequence {rows[i]}"
        starts.append(at)
        at += n
    order = sorted(range(len(lens)), key=lambda i: lens[i])
    check = [i for i in order if lens[i] <= 256] + order[-8:]
    wc, bc = w.cpu(), b.cpu()
    for i in check:
        n = lens[i]
        ref = O.causal_conv1d_ref(x[i, :n].cpu().unsqueeze(0).transpose(1, 2), wc, bc, "silu")
        assert_close_to_oracle(y_pk[:, starts[i]:starts[i] + n].transpose(1, 2), ref, f"sequence {rows[i]}")
    torch.cuda.synchronize()
    assert V.tma_timeouts() == 0


def test_packed_argument_errors():
    x = torch.zeros(1, 40, 64, device=DEV).transpose(1, 2)
    w = torch.zeros(64, 4, device=DEV)
    ids = torch.zeros(1, 40, dtype=torch.int32, device=DEV)
    with pytest.raises(ValueError, match="does not match"):
        V.causal_conv1d_fn(x, w, seq_idx=ids[:, :39])
    with pytest.raises(ValueError, match="cannot be combined"):
        V.causal_conv1d_fn(x, w, seq_idx=ids, attention_mask=torch.ones(1, 40, device=DEV))
    with pytest.raises(ValueError, match="cannot be combined"):
        V.causal_conv1d_fn(x, w, seq_idx=ids, return_final_states=True)


@pytest.mark.parametrize("kernel", ["generic", "tma"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W", [2, 3, 4])
@pytest.mark.parametrize("act", [None, "silu"])
def test_packed_backward_against_oracle(act, W, dtype, kernel):
    """Gradients on packed rows: dx, dweight, dbias against the float64 oracle (each run of equal ids
    differentiated on its own), sequence starts at every offset of a thread's rows and at tile and
    chunk edges, in the scalar and in the TMA-staged kernel."""
    D = 72 if kernel == "generic" else 256
    lens = [1, 2, 3, 125, 1, 130, 4, 127, 128, 129, 64, 5, 7, 8, 9, 1, 1, 63, 65, 16, 15, 17, 2]
    x = O.seeded((1, sum(lens), D), 41, "normal", dtype)
    dy = O.seeded((1, sum(lens), D), 42, "normal", dtype)
    w = O.seeded((D, W), 43, "uniform", dtype)
    b = O.seeded((D,), 44, "uniform", dtype)
    ids = V.seq_idx_from_lengths(lens)
    for residual in (False, True):
        before = V.launch_count()
        dx, dw, db = V.causal_conv1d_bwd(x.to(DEV).transpose(1, 2), w.to(DEV), b.to(DEV), dy.to(DEV).transpose(1, 2), act,
                                         residual=residual, seq_idx=ids.to(DEV), kernel=kernel)
        assert V.launch_count() - before in (1, 2) and V.last_kernel() == "bwd_" + kernel
        rdx, rdw, rdb = O.causal_conv1d_packed_bwd_ref(x.transpose(1, 2), w, b, dy.transpose(1, 2), act, seq_idx=ids,
                                                       residual=residual)
        sdx, _, _ = O.causal_conv1d_packed_bwd_ref(x.abs().transpose(1, 2), w.abs(), None, dy.abs().transpose(1, 2), None,
                                                   seq_idx=ids, residual=residual)
        ulp = 2.0 ** -23 if dtype == torch.float32 else 2.0 ** -7
        bound = 1.1 * sdx.double() * (ulp * 1.01 + 4e-6) + 1e-7
        assert bool(((dx.cpu().double() - rdx.double()).abs() <= bound).all())
        n = sum(lens)
        assert torch.allclose(dw.cpu().double(), rdw, rtol=2e-4, atol=2e-5 * (float(rdw.abs().max()) + 1e-3) * n ** 0.5)
        assert torch.allclose(db.cpu().double(), rdb, rtol=2e-4, atol=2e-5 * (float(rdb.abs().max()) + 1e-3) * n ** 0.5)


def test_packed_autograd_equals_padded_autograd():
    """Training on packed rows: gradients of a loss over the valid positions equal those of the padded,
    masked batch (whose backward runs on the TMA-staged kernel) -- dx bit for bit at the valid positions."""
    B, T, D, W = 6, 300, 512, 4  # large enough for both backward passes to take the TMA-staged kernel
    g = torch.Generator().manual_seed(9)
    lens = [300, 1, 77, 128, 129, 250]
    x = torch.randn(B, T, D, generator=g).bfloat16()
    coef = torch.randn(B, T, D, generator=g).bfloat16()
    m = torch.arange(T)[None, :] < torch.tensor(lens)[:, None]
    w0 = (torch.rand(D, W, generator=g) - 0.5).bfloat16()
    b0 = (torch.rand(D, generator=g) - 0.5).bfloat16()

    xd = x.to(DEV).requires_grad_(True)
    wd, bd = w0.to(DEV).requires_grad_(True), b0.to(DEV).requires_grad_(True)
    y = V.causal_conv1d_fn(xd.transpose(1, 2), wd, bd, activation="silu", attention_mask=m.to(DEV)).transpose(1, 2)
    (y * (coef * m.unsqueeze(-1)).to(DEV)).sum().backward()

    xp = pack(x, lens).to(DEV).requires_grad_(True)
    cp = pack(coef, lens).to(DEV)
    wp, bp = w0.to(DEV).requires_grad_(True), b0.to(DEV).requires_grad_(True)
    ids = V.seq_idx_from_lengths(lens, device=DEV)
    yp = V.causal_conv1d_fn(xp.transpose(1, 2), wp, bp, activation="silu", seq_idx=ids).transpose(1, 2)
    (yp * cp).sum().backward()
    at = 0
    for i, n in enumerate(lens):
        assert torch.equal(xp.grad[0, at:at + n], xd.grad[i, :n]), f"sequence {i}"
        at += n
    assert torch.allclose(wp.grad.float(), wd.grad.float(), rtol=2e-2, atol=2e-2 * float(wd.grad.float().abs().max()))
    assert torch.allclose(bp.grad.float(), bd.grad.float(), rtol=2e-2, atol=2e-2 * float(bd.grad.float().abs().max()))


def test_packed_ids_that_repeat_are_separate_sequences():
    """Sequences are runs of equal ids: an id that comes back later in the row names a new sequence
    (every kernel and the oracle agree on that)."""
    D, W = 128, 4
    ids = torch.tensor([[3, 3, 7, 3, 3, 3, 7, 7] * 40], dtype=torch.int32)
    T = ids.shape[1]
    x = O.seeded((1, T, D), 51, "normal", torch.float32)
    w = O.seeded((D, W), 52, "uniform", torch.float32)
    ref = O.causal_conv1d_packed_ref(x.transpose(1, 2), w, None, "silu", seq_idx=ids)
    for kernel in ("generic", "tma"):
        y = V.causal_conv1d_fn(x.to(DEV).transpose(1, 2), w.to(DEV), None, seq_idx=ids.to(DEV), activation="silu",
                               kernel=kernel)
        assert_close_to_oracle(y, ref, kernel)
    dy = O.seeded((1, T, D), 53, "normal", torch.float32)
    rdx, rdw, _ = O.causal_conv1d_packed_bwd_ref(x.transpose(1, 2), w, None, dy.transpose(1, 2), "silu", seq_idx=ids)
    for kernel in ("generic", "tma"):
        dx, dw, _ = V.causal_conv1d_bwd(x.to(DEV).transpose(1, 2), w.to(DEV), None, dy.to(DEV).transpose(1, 2), "silu",
                                        seq_idx=ids.to(DEV), kernel=kernel)
        assert torch.allclose(dx.cpu(), rdx, rtol=1e-4, atol=1e-5), kernel
        assert torch.allclose(dw.cpu().double(), rdw, rtol=1e-4, atol=1e-4), kernel
