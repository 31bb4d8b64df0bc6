#!/usr/bin/env python
"""Benchmark of the Canon depthwise causal conv1d hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the prefill kernel over one Canon-D batch: 32 sequences x 1024
tokens x 3456 channels, bf16, width 4, bias, SiLU, right-padded with valid lengths uniform in
[128, 1024] and the attention mask applied inside the kernel (synthetic, seeded).  With N > 1
(launched by torch.distributed.run, one process per GPU) every rank runs its own 32 sequences
-- weak scaling, sharded by sequence, no collective on the data path; NCCL is used only for
the barrier around the timed region and the max-over-ranks of the device time.

The single JSON line printed by rank 0 carries:
  value / ms_per_step   padded tokens per second over all ranks, inputs resident in HBM, timed
                        with CUDA events on the launching stream;
  e2e                   the same metric through HostPrefill: pinned host input, host-to-device
                        copy, kernel, device-to-host copy of the result, every step;
  roofline              algorithmic HBM bytes of one launch / its average duration, against the
                        measured copy bandwidth of this GPU pool;
  cpu_baseline          the reference's CPU arithmetic for the same workload on the host cores;
  decode                the decode configuration (batch 256, dim 960, state 3, 1024 steps) as a
                        CUDA graph, and a decode shape large enough to be bandwidth-bound;
  clocks                SM clock and throttle reasons sampled while the timed regions ran.

--impl reference times only the CPU path (the reference has no CUDA kernel of its own for this
operator and its Metal kernels cannot run here).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "prefill_tokens_per_s"
UNIT = "tokens/s"

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the ncu
# capture summarised under profiles/ (None until a capture of the current kernel exists).
NCU_TRAFFIC_BYTES = {"canon_d_prefill_bf16": 320_200_000}


def measured_peak_gbs():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs."""

    def __init__(self, index: int, period_s: float = 0.02):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {
            "sm_mhz": statistics.median(self.samples),
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


def nvml_index_for_local_device(dev_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[dev_index])
        except Exception:
            return dev_index
    return dev_index


# --------------------------------------------------------------------------------------------------
# CPU path of the reference (timed as the baseline / the reference arm)
# --------------------------------------------------------------------------------------------------
def cpu_reference_step(x_btd, weight, bias, mask):
    """What the reference's CanonLayer does for this operator on a CPU, in the model dtype
    (model/model.py:590-620, 664-670): mask multiply, causal left-pad, F.conv1d(groups=D), SiLU."""
    import torch.nn.functional as F

    x = x_btd * mask.unsqueeze(-1)
    xin = F.pad(x.transpose(1, 2), (weight.shape[1] - 1, 0))
    y = F.conv1d(xin, weight.unsqueeze(1), bias=bias, groups=weight.shape[0])
    return F.silu(y)


def time_cpu_reference(cfg, rows, steps, warmup):
    from viby_model_b200 import workloads as WL

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x = WL.prefill_inputs(cfg, rows)
    m = WL.attention_mask(cfg, rows, dtype=torch.bool)
    w, b = WL.weights(cfg.cfg, cfg.dim, cfg.width, cfg.dtype)
    with torch.no_grad():
        for _ in range(warmup):
            cpu_reference_step(x, w, b, m)
        times = []
        for _ in range(steps):
            t0 = time.perf_counter()
            cpu_reference_step(x, w, b, m)
            times.append(time.perf_counter() - t0)
    tokens = len(rows) * cfg.seqlen
    return tokens, times, cores


def run_reference_arm(args):
    """--impl reference: the reference's own CPU arithmetic on the host cores; rank 0 only."""
    from viby_model_b200 import workloads as WL

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = WL.CANON_D_PREFILL
    rows = list(range(8))  # bounded sample: 8 of the 32 sequences per step
    steps, warmup = max(1, args.steps), max(1, min(args.warmup, 3))
    tokens, times, cores = time_cpu_reference(cfg, rows, min(steps, 10), warmup)
    mean_s = sum(times) / len(times)
    value = tokens / mean_s
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": args.gpus,
        "steps": len(times),
        "warmup": warmup,
        "ms_per_step": mean_s * 1e3,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "config": workload_config(cfg, args.gpus),
        "cpu_baseline": {
            "value": value,
            "unit": UNIT,
            "cores": cores,
            "kind": "port",
            "sample": f"{len(rows)} of {cfg.batch} sequences x {cfg.seqlen} tokens per step, mean of {len(times)} steps",
        },
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(cfg, n_gpus):
    return {
        "workload": cfg.name,
        "batch_per_gpu": cfg.batch,
        "global_batch": cfg.batch * n_gpus,
        "seq_len": cfg.seqlen,
        "channels": cfg.dim,
        "width": cfg.width,
        "activation": cfg.activation,
        "bias": True,
        "mask": "bool [B,T], right-padded, valid length uniform in [128,1024], applied in-kernel",
        "layout": "channel-last [B,T,D] viewed as [B,D,T]",
        "parallelism": f"sequence-sharded x{n_gpus}, no collective",
        "l2": "inputs larger than L2 (226 MB read + 226 MB written per step vs 126 MB)",
    }


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--kernel", default=None, help="force a prefill kernel (channel_last | tma)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--no-backward", action="store_true")
    ap.add_argument("--decode-saturating-only", action="store_true",
                    help="run only the bandwidth-bound decode shape and print its figures (for profiling)")
    args = ap.parse_args()

    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch.distributed as dist

    import viby_model_b200 as V
    from viby_model_b200 import workloads as WL
    from viby_model_b200.host_io import HostPrefill

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operators have no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # Keep stdout for the one JSON line: NCCL prints its version banner (and, with NCCL_DEBUG
        # set, its logs) straight to file descriptor 1, so fd 1 is pointed at stderr for the run and
        # the result is written to a private copy of the original stdout.
        sys.stdout.flush()
        result_out = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)
        dist.init_process_group("nccl", device_id=dev)
    else:
        result_out = sys.stdout
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    # one process per GPU: keep this rank's pinned buffers and copy threads on the GPU's NUMA node
    from viby_model_b200.host_io import bind_to_gpu_numa_node
    numa_node = bind_to_gpu_numa_node(local_rank) if world > 1 else None

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    if args.decode_saturating_only:
        res = bench_decode_saturating(V, WL, dev, world, barrier, max_over_ranks)
        if rank == 0:
            print(json.dumps({"decode_saturating": res}), file=result_out, flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- workload: this rank's 32 sequences ---------------------------------------------------
    cfg = WL.CANON_D_PREFILL
    rows = [rank * cfg.batch + i for i in range(cfg.batch)]
    x_host = WL.prefill_inputs(cfg, rows).pin_memory()
    # bool, as the reference's trainer builds it: attn_mask = (X != pad)  (trainer/base_trainer.py:204)
    m_host = WL.attention_mask(cfg, rows, dtype=torch.bool).pin_memory()
    lens = WL.sequence_lengths(cfg, rows)
    w, b = WL.weights(cfg.cfg, cfg.dim, cfg.width, cfg.dtype, device=dev)
    x = x_host.to(dev, non_blocking=True)
    m = m_host.to(dev, non_blocking=True)
    y = torch.empty_like(x)
    xv, yv = x.transpose(1, 2), y.transpose(1, 2)
    valid_tokens = int(lens.sum())
    padded_tokens = cfg.batch * cfg.seqlen

    def step():
        V.causal_conv1d_fn(xv, w, b, activation=cfg.activation, attention_mask=m, out=yv, kernel=args.kernel)

    sampler = ClockSampler(nvml_index_for_local_device(local_rank))
    launches0 = V.launch_count()

    # ---- device-resident timing ------------------------------------------------------------------
    for _ in range(warmup):
        step()
    barrier()
    with sampler:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches_before = V.launch_count()
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        barrier()
        timed_launches = V.launch_count() - launches_before
        ms_total = max_over_ranks(e0.elapsed_time(e1))
        kernel_name = V.last_kernel()

        # ---- end to end: pinned host in, pinned host out, every step -------------------------
        y_host = torch.empty_like(x_host).pin_memory()
        e2e_steps = max(3, min(steps, 20))

        def time_e2e(send_masked_rows):
            pipe = HostPrefill(cfg.batch, cfg.seqlen, cfg.dim, cfg.dtype, device=dev, chunk_batch=4,
                               mask_dtype=torch.bool, send_masked_rows=send_masked_rows)
            for _ in range(3):
                pipe.run(x_host, w, b, cfg.activation, m_host, y_host)
            barrier()
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record()
            for _ in range(e2e_steps):
                # consecutive batches pipeline into each other; every one is copied in and read back
                pipe.run(x_host, w, b, cfg.activation, m_host, y_host, join=False)
            pipe.join()
            f1.record()
            barrier()
            return pipe, max_over_ranks(f0.elapsed_time(f1))

        _, e2e_full_ms_total = time_e2e(True)   # every input row crosses PCIe
        pipe, e2e_ms_total = time_e2e(False)    # rows no kernel reads stay on the host

        # ---- backward of the same workload (training step of the Canon-D layer) ------------------
        backward = None
        if not args.no_backward:
            backward = bench_backward(V, cfg, xv, w, b, m, valid_tokens, padded_tokens, world, barrier,
                                      max_over_ranks)

        # ---- decode ---------------------------------------------------------------------------
        decode = None
        if not args.no_decode:
            decode = bench_decode(V, WL, dev, rank, world, barrier, max_over_ranks)
    e2e_ok = bool(torch.equal(y_host.to(dev), y))

    ms_per_step = ms_total / steps
    value = world * padded_tokens / (ms_per_step * 1e-3)
    valid_total = sum_over_ranks(float(valid_tokens))
    e2e_ms = e2e_ms_total / e2e_steps
    e2e_value = world * padded_tokens / (e2e_ms * 1e-3)

    # ---- roofline of the dominant kernel -------------------------------------------------------
    peak, peak_kind = measured_peak_gbs()
    elem = 2
    mask_bytes = m.numel() * m.element_size()
    alg_bytes = WL.prefill_bytes(cfg.batch, cfg.dim, cfg.seqlen, cfg.width, elem, valid_tokens=valid_tokens,
                                 mask_bytes=mask_bytes)
    dense_bytes = WL.prefill_bytes(cfg.batch, cfg.dim, cfg.seqlen, cfg.width, elem, mask_bytes=mask_bytes)
    launch_s = ms_per_step * 1e-3
    achieved = alg_bytes / launch_s / 1e9
    roofline = {
        "bound": "hbm",
        "kernel": kernel_name,
        "achieved": achieved,
        "peak": peak,
        "peak_kind": peak_kind,
        "unit": "GB/s",
        "frac": achieved / peak,
        "frac_of_nominal_8000": achieved / 8000.0,
        "algorithmic_bytes_per_launch": alg_bytes,
        "dense_bytes_per_launch": dense_bytes,
        "dense_equiv_gbs": dense_bytes / launch_s / 1e9,
        "traffic": NCU_TRAFFIC_BYTES.get(cfg.name),
    }

    clocks = sampler.summary()
    line = {
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": world,
        "steps": steps,
        "warmup": warmup,
        "ms_per_step": ms_per_step,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "config": workload_config(cfg, world),
        "valid_tokens_per_s": valid_total / (ms_per_step * 1e-3),
        "e2e": {
            "value": e2e_value,
            "unit": UNIT,
            "h2d_bytes_per_step": pipe.h2d_bytes,
            "d2h_bytes_per_step": pipe.d2h_bytes,
            "ms_per_step": e2e_ms,
            "steps": e2e_steps,
            "matches_device_result": e2e_ok,
            "numa_node": numa_node,
            "note": "rows behind each sequence's last valid position are never read by the kernel and are not sent",
        },
        "e2e_all_rows_sent": {
            "value": world * padded_tokens / (e2e_full_ms_total / e2e_steps * 1e-3),
            "unit": UNIT,
            "h2d_bytes_per_step": cfg.batch * cfg.seqlen * (cfg.dim * 2 + 1),
            "d2h_bytes_per_step": pipe.d2h_bytes,
            "ms_per_step": e2e_full_ms_total / e2e_steps,
            "note": "the same pipeline copying all of x, masked rows included",
        },
        "gpu_launches": timed_launches,
        "roofline": roofline,
        "clocks": clocks,
    }
    if backward is not None:
        line["backward"] = backward
    if decode is not None:
        line["decode"] = decode
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sample_rows = list(range(8))
        tokens, times, cores = time_cpu_reference(cfg, sample_rows, 5, 1)
        best = min(times)
        line["cpu_baseline"] = {
            "value": tokens / best,
            "unit": UNIT,
            "cores": cores,
            "kind": "port",
            "sample": f"{len(sample_rows)} of {cfg.batch} sequences x {cfg.seqlen} tokens, best of {len(times)} "
                      f"after 1 warm-up, reference arithmetic (bf16 F.conv1d + SiLU) in torch",
            "ms": best * 1e3,
        }
    if rank == 0:
        print(json.dumps(line), file=result_out, flush=True)
    if world > 1:
        dist.destroy_process_group()


def bench_backward(V, cfg, xv, w, b, m, valid_tokens, padded_tokens, world, barrier, max_over_ranks):
    """Gradients (dx, dweight, dbias) of the bench workload: one causal_conv1d_bwd launch per step,
    device-resident.  Algorithmic bytes: x read where valid + dy read + dx written."""
    g = torch.Generator(device=xv.device).manual_seed(11)
    dy = torch.randn(xv.shape[0], xv.shape[2], xv.shape[1], generator=g, device=xv.device).to(cfg.dtype).transpose(1, 2)
    def step():
        return V.causal_conv1d_bwd(xv, w, b, dy, cfg.activation, attention_mask=m)
    for _ in range(5):
        step()
    barrier()
    n = 50
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        step()
    e1.record()
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1)) / n
    elem = 2
    nbytes = (valid_tokens + 2 * padded_tokens) * cfg.dim * elem
    peak, _ = measured_peak_gbs()
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {
        "kernel": V.last_kernel(),
        "ms_per_step": ms,
        "tokens_per_s": world * padded_tokens / (ms * 1e-3),
        "algorithmic_bytes_per_launch": nbytes,
        "achieved_gbs": gbs,
        "frac_of_measured_peak": gbs / peak,
        "note": "includes the zeroing of the fp32 dweight/dbias accumulators and the tile-classification pre-pass",
    }


def bench_decode(V, WL, dev, rank, world, barrier, max_over_ranks):
    """Decode configuration: 1024 successive causal_conv1d_update steps on a [256, 960, 3] state
    seeded from a 512-token prefill, replayed as one CUDA graph; plus one bandwidth-bound shape."""
    cfg = WL.DECODE_CANON_B
    rows = [rank * cfg.batch + i for i in range(cfg.batch)]
    w, b = WL.weights(cfg.cfg, cfg.dim, cfg.width, cfg.dtype, device=dev)
    pre = WL.decode_prefill(cfg, rows, device=dev)
    _, state0 = V.causal_conv1d_fn(pre.transpose(1, 2), w, b, return_final_states=True, state_len=cfg.state_len)
    g = torch.Generator(device=dev).manual_seed(7 + rank)
    toks = torch.randn(cfg.steps, cfg.batch, cfg.dim, generator=g, device=dev).to(cfg.dtype)
    ys = torch.empty_like(toks)
    state = state0.clone()

    def eager():
        for s in range(cfg.steps):
            V.causal_conv1d_update(toks[s], state, w, b, out=ys[s])

    # eager launches
    eager()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    eager()
    e1.record()
    barrier()
    eager_ms = max_over_ranks(e0.elapsed_time(e1))

    # the same 1024 launches captured once and replayed
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        eager()
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            eager()
    torch.cuda.current_stream(dev).wait_stream(side)
    for _ in range(3):
        graph.replay()
    barrier()
    reps = 5
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    barrier()
    graph_ms = max_over_ranks(e0.elapsed_time(e1)) / reps
    step_bytes = WL.decode_bytes(cfg.batch, cfg.dim, cfg.width, cfg.state_len, 2)

    saturating = bench_decode_saturating(V, WL, dev, world, barrier, max_over_ranks)
    return {
        "config": {"workload": cfg.name, "batch_per_gpu": cfg.batch, "channels": cfg.dim, "state_len": cfg.state_len,
                   "width": cfg.width, "steps": cfg.steps, "prefill_len": cfg.prefill_len},
        "tokens_per_s_graph": world * cfg.batch * cfg.steps / (graph_ms * 1e-3),
        "us_per_step_graph": graph_ms * 1e3 / cfg.steps,
        "tokens_per_s_eager": world * cfg.batch * cfg.steps / (eager_ms * 1e-3),
        "us_per_step_eager": eager_ms * 1e3 / cfg.steps,
        "bytes_per_step": step_bytes,
        "gbs_graph": step_bytes * cfg.steps / (graph_ms * 1e-3) / 1e9,
        "saturating": saturating,
    }


def bench_decode_saturating(V, WL, dev, world, barrier, max_over_ranks):
    """Bandwidth-bound decode shape: as many (sequence, channel) rows as one Canon-D prefill batch."""
    cfg = WL.DECODE_CANON_B
    Bs, Ds, Ls = 32768, 3456, cfg.state_len
    ws, bs = WL.weights(cfg.cfg, Ds, cfg.width, cfg.dtype, device=dev)
    xs = torch.randn(Bs, Ds, device=dev).to(cfg.dtype)
    ss = torch.randn(Bs, Ds, Ls, device=dev).to(cfg.dtype)
    yo = torch.empty_like(xs)
    for _ in range(5):
        V.causal_conv1d_update(xs, ss, ws, bs, activation="silu", out=yo)
    barrier()
    n = 20
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        V.causal_conv1d_update(xs, ss, ws, bs, activation="silu", out=yo)
    e1.record()
    barrier()
    sat_ms = max_over_ranks(e0.elapsed_time(e1)) / n
    sat_bytes = WL.decode_bytes(Bs, Ds, cfg.width, Ls, 2)
    peak, _ = measured_peak_gbs()
    return {
        "batch": Bs, "channels": Ds, "state_len": Ls, "activation": "silu",
        "ms_per_step": sat_ms, "bytes_per_step": sat_bytes,
        "achieved_gbs": sat_bytes / (sat_ms * 1e-3) / 1e9,
        "frac_of_measured_peak": sat_bytes / (sat_ms * 1e-3) / 1e9 / peak,
        "tokens_per_s": world * Bs / (sat_ms * 1e-3),
    }


if __name__ == "__main__":
    main()
