#!/usr/bin/env python
"""Benchmark of the Canon depthwise causal conv1d hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the prefill kernel over one Canon-D batch: 32 sequences x 1024
tokens x 3456 channels, bf16, width 4, bias, SiLU, right-padded with valid lengths uniform in
[128, 1024] and the attention mask applied inside the kernel (synthetic, seeded).  With N > 1
(launched by torch.distributed.run, one process per GPU) every rank runs its own 32 sequences
-- weak scaling, sharded by sequence, no collective on the data path; NCCL is used only for
the barrier around the timed regions and the reductions of the device times.

The single JSON line printed by rank 0 carries:
  value / ms_per_step   padded tokens per second over all ranks, inputs resident in HBM, timed
                        with CUDA events on the launching stream (K steps per round, several
                        rounds back to back, the median round reported; max over ranks);
  e2e                   the same metric through HostPrefill: pinned host input, host-to-device
                        copy, kernel, device-to-host copy of the result, every step; with the
                        plain copy rate of the same bytes over the same link beside it;
  roofline              algorithmic HBM bytes of one launch / its average duration, against the
                        measured copy bandwidth of this GPU pool;
  ragged_sweep          the ragged large-batch configuration (512 sequences, up to 4096 tokens,
                        lengths log-uniform) sharded over the N ranks -- strong scaling;
  shapes                the Canon A/B/C/D shapes of the whole-model configuration and a dense batch;
  backward, decode, model_decode_step
                        gradient kernel of the step; the decode configuration as a CUDA graph,
                        bandwidth-bound decode shapes; the 72 decode calls of one model step;
  cpu_baseline          the reference's CPU arithmetic for the same workload on the host cores;
  clocks                SM clock and throttle reasons sampled while the timed regions ran.

--impl reference times only the CPU path, in a process that never loads the CUDA library (the
reference has no CUDA kernel of its own for this operator and its Metal kernels cannot run here).
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent

METRIC = "prefill_tokens_per_s"
UNIT = "tokens/s"

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the ncu
# capture summarised under profiles/ (None until a capture of the current kernel exists).
NCU_TRAFFIC_BYTES = {"canon_d_prefill_bf16": 317_200_000}


def load_workloads():
    """The seeded input generators, loaded by file path: importing the package would load the CUDA
    library, which the reference arm must not do."""
    spec = importlib.util.spec_from_file_location("vc1d_workloads", ROOT / "viby_model_b200" / "workloads.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules["vc1d_workloads"] = mod  # dataclasses look their module up by name
    spec.loader.exec_module(mod)
    return mod


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


def find_reference_tree():
    """A checkout of the reference, where one exists on this machine (never on the GPU boxes)."""
    for cand in (os.environ.get("VIBY_REFERENCE"), "/root/reference", str(ROOT / "baseline" / "_ref")):
        if cand and (Path(cand) / "model" / "model.py").exists():
            return Path(cand)
    return None


def reference_canon_layer(tree: Path, cfg, weight, bias):
    """The reference's own CanonLayer (model/model.py:201-675), imported unmodified with both optional
    kernel packages made unimportable, so that its forward takes the PyTorch branch (:587-675)."""
    sys.modules["causal_conv1d"] = None      # model/model.py:20-30 then sets HAS_CAUSAL_CONV1D_CUDA = False
    sys.modules["causal_conv1d_mps"] = None  # model/model.py:12-18
    sys.dont_write_bytecode = True
    sys.path.insert(0, str(tree))
    from model.model import CanonLayer, VibyConfig  # noqa: E402

    conf = VibyConfig(canon_bias=bias is not None, canon_activation=cfg.activation is not None,
                      canon_kernel=cfg.width)
    layer = CanonLayer(cfg.dim, conf, "d").to(cfg.dtype)
    with torch.no_grad():
        layer.weight.copy_(weight.unsqueeze(1))
        if bias is not None:
            layer.bias_param.copy_(bias)
    return layer.eval()


def time_cpu_reference(WL, cfg, rows, steps, warmup, want_tree=True):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x = WL.prefill_inputs(cfg, rows)
    m = WL.attention_mask(cfg, rows, dtype=torch.bool)
    w, b = WL.weights(cfg.cfg, cfg.dim, cfg.width, cfg.dtype)
    kind, step = "port", (lambda: cpu_reference_step(x, w, b, m))
    tree = find_reference_tree() if want_tree else None
    if tree is not None:
        try:
            layer = reference_canon_layer(tree, cfg, w, b)
            kind, step = "reference", (lambda: layer(x, attention_mask=m))
        except Exception as e:  # an incomplete tree: fall back to the restated calls
            print(f"reference tree at {tree} not usable ({type(e).__name__}: {e}); timing the port", file=sys.stderr)
    with torch.no_grad():
        for _ in range(warmup):
            step()
        times = []
        for _ in range(steps):
            t0 = time.perf_counter()
            step()
            times.append(time.perf_counter() - t0)
    tokens = len(rows) * cfg.seqlen
    return tokens, times, cores, kind


def run_reference_arm(args):
    """--impl reference: the reference's own CPU code path on the host cores, one process (rank 0)
    whatever N is.  Nothing of viby_model_b200 is imported, so no CUDA library is loaded."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    WL = load_workloads()
    cfg = WL.CANON_D_PREFILL
    rows = list(range(8))  # bounded sample: 8 of the 32 sequences per step
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    tokens, times, cores, kind = time_cpu_reference(WL, cfg, rows, steps, warmup)
    mean_s = sum(times) / len(times)
    value = tokens / mean_s
    what = ("the reference's CanonLayer.forward, PyTorch branch (model/model.py:587-675), imported unmodified"
            if kind == "reference" else
            "the reference's CPU arithmetic restated in torch (model/model.py:590-620, 664-670): no reference tree on this machine")
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": args.gpus,
        "steps": steps,
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
            "kind": kind,
            "what": what,
            "processes": 1,
            "sample": f"{len(rows)} of {cfg.batch} sequences x {cfg.seqlen} tokens per step, mean of {steps} steps; "
                      f"one host process on rank 0 at every N",
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
class Ctx:
    """What every section of the GPU arm needs: the device, the rank layout and the reductions."""

    def __init__(self, V, WL, dev, rank, world):
        import torch.distributed as dist

        self.V, self.WL, self.dev, self.rank, self.world, self.dist = V, WL, dev, rank, world, dist
        self.peak, self.peak_kind = measured_peak_gbs()

    def barrier(self):
        torch.cuda.synchronize(self.dev)
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize(self.dev)

    def gather(self, v: float):
        """The value of every rank, in rank order."""
        if self.world == 1:
            return [float(v)]
        t = torch.tensor([float(v)], dtype=torch.float64, device=self.dev)
        out = [torch.empty_like(t) for _ in range(self.world)]
        self.dist.all_gather(out, t)
        return [float(o.item()) for o in out]

    def max_over_ranks(self, v: float) -> float:
        return max(self.gather(v))

    def sum_over_ranks(self, v: float) -> float:
        return sum(self.gather(v))

    def time_loop(self, fn, steps, warmup=3):
        """steps calls of fn between two events on the current stream, barriers on both sides.
        Returns (this rank's ms for all steps, host seconds the loop took to enqueue)."""
        for _ in range(warmup):
            fn()
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        t0 = time.perf_counter()
        for _ in range(steps):
            fn()
        host_s = time.perf_counter() - t0
        e1.record()
        self.barrier()
        return e0.elapsed_time(e1), host_s


def spread(values):
    return {"min": min(values), "median": statistics.median(values), "max": max(values)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--kernel", default=None, help="force a prefill kernel (channel_last | tma)")
    ap.add_argument("--rounds", type=int, default=5, help="timed rounds of --steps steps each; the median is reported")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--no-backward", action="store_true")
    ap.add_argument("--no-ragged", action="store_true")
    ap.add_argument("--no-shapes", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--only", default=None, choices=["headline", "decode_saturating", "ragged", "backward", "model_prefill", "model_decode", "shapes"],
                    help="run one section and print its figures (for profiling: few launches, small footprint)")
    ap.add_argument("--state-len", type=int, default=3, help="state length of --only decode_saturating")
    ap.add_argument("--circular", action="store_true", help="circular state for --only decode_saturating")
    args = ap.parse_args()

    if args.impl == "reference":
        run_reference_arm(args)
        return

    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist

    import viby_model_b200 as V
    from viby_model_b200 import workloads as WL
    from viby_model_b200.host_io import NUMA_STATUS, HostPrefill, bind_to_gpu_numa_node

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
    ctx = Ctx(V, WL, dev, rank, world)
    # host threads of this rank (the launcher sets OMP_NUM_THREADS=1): an equal share of the cores, for the
    # host-side part of the end-to-end path
    host_threads = max(1, (os.cpu_count() or 1) // world)
    torch.set_num_threads(host_threads)
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    # one process per GPU: keep this rank's pinned buffers and copy threads on the GPU's NUMA node
    numa_node = bind_to_gpu_numa_node(local_rank) if world > 1 else None
    numa_note = NUMA_STATUS.get(local_rank, "one process: not bound")

    def emit(obj):
        if rank == 0:
            print(json.dumps(obj), file=result_out, flush=True)
        if world > 1:
            dist.destroy_process_group()

    if args.only == "decode_saturating":
        emit({"decode_saturating": bench_decode_saturating(ctx, args.state_len, circular=args.circular,
                                                           steps=min(steps, 20))})
        return
    if args.only == "ragged":
        emit({"ragged_sweep": bench_ragged(ctx, steps=min(steps, 10))})
        return
    if args.only == "model_prefill":
        emit({"model_prefill_step": bench_model_prefill_step(ctx)})
        return
    if args.only == "shapes":
        emit({"shapes": bench_shapes(ctx)})
        return
    if args.only == "model_decode":
        emit({"model_decode_step": bench_model_decode_step(ctx)})
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

    if args.only == "backward":
        emit({"backward": bench_backward(ctx, cfg, xv, w, b, m, valid_tokens, padded_tokens, steps=min(steps, 50))})
        return

    sampler = ClockSampler(nvml_index_for_local_device(local_rank))

    # ---- device-resident timing: R rounds of K steps back to back, each between its own events ----
    rounds = 1 if args.only == "headline" else max(1, args.rounds)
    for _ in range(warmup):
        step()
    ctx.barrier()
    with sampler:
        events = [torch.cuda.Event(enable_timing=True) for _ in range(rounds + 1)]
        launches_before = V.launch_count()
        host_t0 = time.perf_counter()
        events[0].record()
        for r in range(rounds):
            for _ in range(steps):
                step()
            events[r + 1].record()
        host_s = time.perf_counter() - host_t0
        ctx.barrier()
        timed_launches = (V.launch_count() - launches_before) // rounds
        kernel_name = V.last_kernel()
        my_rounds = [events[r].elapsed_time(events[r + 1]) for r in range(rounds)]
        # per round: every rank's time; the round counts with its slowest rank
        per_round = [ctx.gather(t) for t in my_rounds]
        round_ms = [max(v) for v in per_round]
        order = sorted(range(rounds), key=lambda r: round_ms[r])
        mid = order[(rounds - 1) // 2]
        ms_total = round_ms[mid]
        # The same loop with the tile classes worked out on every call (what the first call with a mask
        # costs; in the timed loop above they are kept while the mask tensor is unchanged, as they are
        # across the 72 Canon calls of one forward pass of the reference's network).
        was = V.reuse_tile_classes(False)
        try:
            fresh_launches = V.launch_count()
            fresh_ms = max(ctx.gather(ctx.time_loop(step, steps, warmup=3)[0])) / steps
            fresh_launches = (V.launch_count() - fresh_launches) // (steps + 3)
        finally:
            V.reuse_tile_classes(was)
        if args.only == "headline":
            emit({"ms_per_step": ms_total / steps, "kernel": kernel_name, "launches_per_round": timed_launches,
                  "ms_per_step_classified_every_call": fresh_ms})
            return

        # ---- end to end: pinned host in, pinned host out, every step -------------------------
        e2e = None
        if not args.no_e2e:
            e2e = bench_e2e(ctx, HostPrefill, cfg, x_host, m_host, w, b, x, y, steps, padded_tokens, host_threads)
            e2e["main"]["numa_node"] = numa_node
            e2e["main"]["numa_note"] = numa_note
            e2e["main"]["host_threads_per_rank"] = host_threads

        backward = None if args.no_backward else bench_backward(ctx, cfg, xv, w, b, m, valid_tokens, padded_tokens)
        decode = None if args.no_decode else bench_decode(ctx)
        model_step = None if args.no_decode else bench_model_decode_step(ctx)
        shapes = None if args.no_shapes else bench_shapes(ctx)
        model_prefill = None if args.no_shapes else bench_model_prefill_step(ctx)
        del x_host
        ragged = None if args.no_ragged else bench_ragged(ctx, steps=10)

    ms_per_step = ms_total / steps
    value = world * padded_tokens / (ms_per_step * 1e-3)
    valid_total = ctx.sum_over_ranks(float(valid_tokens))

    # ---- roofline of the dominant kernel -------------------------------------------------------
    peak, peak_kind = ctx.peak, ctx.peak_kind
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
        "timing": {
            "rounds": rounds,
            "steps_per_round": steps,
            "reported": "median round (by its slowest rank)",
            "ms_per_step_rounds": [t / steps for t in round_ms],
            "ms_per_step_first_round": round_ms[0] / steps,
            "per_rank_ms_per_step": spread([t / steps for t in per_round[mid]]),
            "slowest_rank": max(range(world), key=lambda r: per_round[mid][r]),
            "host_enqueue_us_per_step": host_s / (rounds * steps) * 1e6,
        },
        "gpu_launches": timed_launches,
        "tile_classes": {
            "kept_while_mask_unchanged": True,
            "note": "the classes of the mask's tiles (all valid / mixed / all padding) depend on the mask alone; "
                    "a launch whose mask tensor is the one of the launch before it on the stream (same memory, "
                    "same torch version counter) reads the class table that launch left and runs no pre-pass",
            "ms_per_step_classified_every_call": fresh_ms,
            "frac_classified_every_call": alg_bytes / (fresh_ms * 1e-3) / 1e9 / peak,
            "launches_per_step_classified_every_call": fresh_launches,
        },
        "roofline": roofline,
        "clocks": sampler.summary(),
    }
    if e2e is not None:
        line["e2e"] = e2e["main"]
        line["e2e_variants"] = e2e["variants"]
    if backward is not None:
        line["backward"] = backward
    if decode is not None:
        line["decode"] = decode
    if model_step is not None:
        line["model_decode_step"] = model_step
    if shapes is not None:
        line["shapes"] = shapes
    if model_prefill is not None:
        line["model_prefill_step"] = model_prefill
    if ragged is not None:
        line["ragged_sweep"] = ragged
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sample_rows = list(range(8))
        tokens, times, cores, kind = time_cpu_reference(WL, cfg, sample_rows, 5, 1, want_tree=False)
        best = min(times)
        line["cpu_baseline"] = {
            "value": tokens / best,
            "unit": UNIT,
            "cores": cores,
            "kind": kind,
            "sample": f"{len(sample_rows)} of {cfg.batch} sequences x {cfg.seqlen} tokens, best of {len(times)} "
                      f"after 1 warm-up, reference arithmetic (bf16 F.conv1d + SiLU) in torch",
            "ms": best * 1e3,
        }
    emit(line)


# --------------------------------------------------------------------------------------------------
# sections
# --------------------------------------------------------------------------------------------------
def bench_e2e(ctx, HostPrefill, cfg, x_host, m_host, w, b, x_dev, y_dev, steps, padded_tokens, host_threads):
    """The step through HostPrefill, host buffers in and out, in three variants; and the plain copy
    rate of the same byte counts over the same link (two streams, no kernel) for comparison."""
    dev, world = ctx.dev, ctx.world
    y_host = torch.empty_like(x_host).pin_memory()
    e2e_steps = max(3, min(steps, 20))

    def run(**kw):
        pipe = HostPrefill(cfg.batch, cfg.seqlen, cfg.dim, cfg.dtype, device=dev, chunk_batch=4,
                           mask_dtype=torch.bool, fill_workers=max(1, min(8, host_threads // 2)), **kw)
        y_host.fill_(0)
        for _ in range(3):
            pipe.run(x_host, w, b, cfg.activation, m_host, y_host)
        ctx.barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(e2e_steps):
            # consecutive batches pipeline into each other; every one is copied in and read back
            pipe.run(x_host, w, b, cfg.activation, m_host, y_host, join=False)
        pipe.join()
        f1.record()
        ctx.barrier()
        per_rank = ctx.gather(f0.elapsed_time(f1) / e2e_steps)
        ok = bool(torch.equal(y_host.to(dev), y_dev))
        ms = max(per_rank)
        return {
            "value": world * padded_tokens / (ms * 1e-3),
            "unit": UNIT,
            "h2d_bytes_per_step": pipe.h2d_bytes,
            "d2h_bytes_per_step": pipe.d2h_bytes,
            "ms_per_step": ms,
            "per_rank_ms_per_step": spread(per_rank),
            "steps": e2e_steps,
            "matches_device_result": ok,
        }

    full = run(send_masked_rows=True)
    full["note"] = "every row of x sent, every row of y copied back"
    lean_in = run()
    lean_in["note"] = "rows behind each sequence's last valid position are never read by the kernel and are not sent"
    lean = run(skip_constant_rows=True)
    lean["note"] = ("as above, and output rows whose taps are all masked (the constant act(bias)) are not copied "
                    "back: the host writes them into y_host from one [channels] vector inside the timed region")

    # plain copies of the same byte counts: what the link gives with no kernel and no pipeline logic
    def link(h2d_bytes, d2h_bytes):
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        xin = x_host.view(-1).view(torch.uint8)
        xd = x_dev.view(-1).view(torch.uint8)
        yd = y_dev.view(-1).view(torch.uint8)
        yout = y_host.view(-1).view(torch.uint8)
        n_in, n_out = min(h2d_bytes, xin.numel()), min(d2h_bytes, yout.numel())
        scratch_dev = torch.empty(n_in, dtype=torch.uint8, device=dev)

        def once():
            with torch.cuda.stream(s_in):
                scratch_dev.copy_(xin[:n_in], non_blocking=True)
            with torch.cuda.stream(s_out):
                yout[:n_out].copy_(yd[:n_out], non_blocking=True)

        for _ in range(2):
            once()
        ctx.barrier()
        main = torch.cuda.current_stream(dev)
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        reps = 5
        for _ in range(reps):
            once()
        main.wait_stream(s_in)
        main.wait_stream(s_out)
        f1.record()
        ctx.barrier()
        del xd
        per_rank = ctx.gather(f0.elapsed_time(f1) / reps)
        ms = max(per_rank)
        return {"ms": ms, "gbs_per_rank_both_directions": (n_in + n_out) / (ms * 1e-3) / 1e9,
                "d2h_gbs_per_rank": n_out / (ms * 1e-3) / 1e9, "per_rank_ms": spread(per_rank)}

    for v in (full, lean_in, lean):
        lk = link(v["h2d_bytes_per_step"], v["d2h_bytes_per_step"])
        v["link_ms_same_bytes"] = lk["ms"]
        v["link_gbs"] = lk["gbs_per_rank_both_directions"]
        v["frac_of_link"] = lk["ms"] / v["ms_per_step"]
    # Headline: y_host holds the same bytes in all three plans; a caller picks the one that is fastest on
    # its host (filling the constant rows costs host threads, copying them costs link time), and so does
    # this line.  All three stay in the record.
    plans = {"all_rows_both_ways": full, "valid_rows_in_all_rows_out": lean_in,
             "valid_rows_in_non_constant_rows_out": lean}
    best = min(("valid_rows_in_non_constant_rows_out", "valid_rows_in_all_rows_out"),
               key=lambda k: plans[k]["ms_per_step"])
    main = dict(plans[best])
    main["plan"] = best
    return {"main": main, "variants": plans}


def bench_backward(ctx, cfg, xv, w, b, m, valid_tokens, padded_tokens, steps=50):
    """Gradients (dx, dweight, dbias) of the bench workload: one causal_conv1d_bwd launch per step,
    device-resident.  Algorithmic bytes: x read where valid + dy read + dx written."""
    V = ctx.V
    g = torch.Generator(device=xv.device).manual_seed(11)
    dy = torch.randn(xv.shape[0], xv.shape[2], xv.shape[1], generator=g, device=xv.device).to(cfg.dtype).transpose(1, 2)

    def step():
        return V.causal_conv1d_bwd(xv, w, b, dy, cfg.activation, attention_mask=m)

    n = steps
    ms_rank, host_s = ctx.time_loop(step, n, warmup=min(5, max(3, steps)))
    ms = ctx.max_over_ranks(ms_rank) / n
    elem = 2
    nbytes = (valid_tokens + 2 * padded_tokens) * cfg.dim * elem
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {
        "kernel": V.last_kernel(),
        "ms_per_step": ms,
        "tokens_per_s": ctx.world * padded_tokens / (ms * 1e-3),
        "algorithmic_bytes_per_launch": nbytes,
        "achieved_gbs": gbs,
        "frac_of_measured_peak": gbs / ctx.peak,
        "host_enqueue_us_per_step": host_s / n * 1e6,
        "note": "one call = the tile-classification pre-pass (which also clears the fp32 dweight/dbias accumulators) "
                "and the main kernel",
    }


def bench_decode(ctx):
    """Decode configuration: 1024 successive causal_conv1d_update steps on a [256, 960, 3] state
    seeded from a 512-token prefill, replayed as one CUDA graph; plus bandwidth-bound shapes."""
    V, WL, dev, rank, world = ctx.V, ctx.WL, ctx.dev, ctx.rank, ctx.world
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

    eager_rank, _ = ctx.time_loop(eager, 1, warmup=1)
    eager_ms = ctx.max_over_ranks(eager_rank)

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
    reps = 5
    graph_rank, _ = ctx.time_loop(graph.replay, reps, warmup=3)
    graph_ms = ctx.max_over_ranks(graph_rank) / reps
    step_bytes = WL.decode_bytes(cfg.batch, cfg.dim, cfg.width, cfg.state_len, 2)
    return {
        "config": {"workload": cfg.name, "batch_per_gpu": cfg.batch, "channels": cfg.dim, "state_len": cfg.state_len,
                   "width": cfg.width, "steps": cfg.steps, "prefill_len": cfg.prefill_len},
        "bound": "launch",
        "bound_note": "3.9 MB per step is under 1 us of HBM time and the 1.5 MB state stays in L2: a step costs its "
                      "launch; bandwidth-bound decode figures are under 'saturating'",
        "tokens_per_s_graph": world * cfg.batch * cfg.steps / (graph_ms * 1e-3),
        "us_per_step_graph": graph_ms * 1e3 / cfg.steps,
        "tokens_per_s_eager": world * cfg.batch * cfg.steps / (eager_ms * 1e-3),
        "us_per_step_eager": eager_ms * 1e3 / cfg.steps,
        "bytes_per_step": step_bytes,
        "gbs_graph": step_bytes * cfg.steps / (graph_ms * 1e-3) / 1e9,
        "saturating": bench_decode_saturating(ctx, cfg.state_len),
        "saturating_state_len_4": bench_decode_saturating(ctx, 4),
        "saturating_state_len_8": bench_decode_saturating(ctx, 8),
        "saturating_circular_state_len_8": bench_decode_saturating(ctx, 8, circular=True),
    }


def bench_decode_saturating(ctx, state_len, circular=False, steps=20):
    """Bandwidth-bound decode shape: as many (sequence, channel) rows as one Canon-D prefill batch."""
    V, WL, dev = ctx.V, ctx.WL, ctx.dev
    cfg = WL.DECODE_CANON_B
    Bs, Ds, Ls = 32768, 3456, state_len
    ws, bs = WL.weights(cfg.cfg, Ds, cfg.width, cfg.dtype, device=dev)
    xs = torch.randn(Bs, Ds, device=dev).to(cfg.dtype)
    ss = torch.randn(Bs, Ds, Ls, device=dev).to(cfg.dtype)
    yo = torch.empty_like(xs)
    seqlens = torch.arange(Bs, dtype=torch.int32, device=dev) if circular else None

    def step():
        V.causal_conv1d_update(xs, ss, ws, bs, "silu", seqlens, out=yo)

    n = steps
    ms_rank, _ = ctx.time_loop(step, n, warmup=min(5, max(3, steps)))
    sat_ms = ctx.max_over_ranks(ms_rank) / n
    kernel = V.last_kernel()
    # x + y + the state row read + the state row written.  (The circular state keeps its columns in place
    # and needs only width-1 of them, but a channel's whole row -- 16 bytes at state_len 8 -- is half a
    # DRAM sector: it moves whole either way, so the row is counted whole.)
    sat_bytes = WL.decode_bytes(Bs, Ds, cfg.width, Ls, 2) + (Bs * 4 if circular else 0)
    return {
        "batch": Bs, "channels": Ds, "state_len": Ls, "activation": "silu", "circular": circular, "kernel": kernel,
        "ms_per_step": sat_ms, "bytes_per_step": sat_bytes,
        "achieved_gbs": sat_bytes / (sat_ms * 1e-3) / 1e9,
        "frac_of_measured_peak": sat_bytes / (sat_ms * 1e-3) / 1e9 / ctx.peak,
        "tokens_per_s": ctx.world * Bs / (sat_ms * 1e-3),
    }


def bench_model_decode_step(ctx):
    """The Canon work of ONE decode step of the whole-model configuration: 18 layers x (A 640, B 960,
    C 640, D 3456 channels) = 72 causal_conv1d_update calls at batch 64 with the [B, D, 4] states the
    reference's CUDA branch keeps (model/model.py:299-313), bf16, no bias, no activation (the
    reference's defaults).  Eager with programmatic dependent launch on and off, and as one CUDA graph."""
    V, dev = ctx.V, ctx.dev
    B, L, W, layers = 64, 4, 4, 18
    dims = (640, 960, 640, 3456)
    g = torch.Generator(device=dev).manual_seed(3)
    calls = []
    for _ in range(layers):
        for D in dims:
            calls.append((torch.randn(B, D, generator=g, device=dev).bfloat16(),
                          torch.randn(B, D, L, generator=g, device=dev).bfloat16(),
                          (torch.rand(D, W, generator=g, device=dev) - 0.5).bfloat16(),
                          torch.empty(B, D, device=dev, dtype=torch.bfloat16)))

    def model_step():
        for xt, st, wt, out in calls:
            V.causal_conv1d_update(xt, st, wt, None, None, out=out)

    nbytes = sum(B * D * 2 * (2 + 2 * L) + D * W * 2 for D in dims) * layers
    res = {"calls_per_step": len(calls), "batch": B, "state_len": L, "channels": list(dims), "layers": layers,
           "bytes_per_step": nbytes}
    n = 20
    for name, pdl in (("eager_pdl_on", True), ("eager_pdl_off", False)):
        before = V.set_pdl(pdl)
        ms_rank, host_s = ctx.time_loop(model_step, n, warmup=3)
        V.set_pdl(None)
        ms = ctx.max_over_ranks(ms_rank) / n
        res[name] = {"us_per_step": ms * 1e3, "us_per_call": ms * 1e3 / len(calls), "gbs": nbytes / (ms * 1e-3) / 1e9,
                     "host_enqueue_us_per_step": host_s / n * 1e6}
        del before
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        model_step()
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            model_step()
    torch.cuda.current_stream(dev).wait_stream(side)
    ms_rank, _ = ctx.time_loop(graph.replay, n, warmup=3)
    ms = ctx.max_over_ranks(ms_rank) / n
    res["graph"] = {"us_per_step": ms * 1e3, "us_per_call": ms * 1e3 / len(calls), "gbs": nbytes / (ms * 1e-3) / 1e9}
    # The same 72 problems as ONE launch (vc1d_update_multi).  Inside one network they depend on each other and
    # cannot be batched like this; the figure is what a table of independent steps (several requests, beams or
    # networks decoded side by side) costs against a launch each.
    xs, states, ws, outs = ([c[k] for c in calls] for k in (0, 1, 2, 3))

    table = V.UpdateTable(xs, states, ws, None, None, outs=outs)
    ms_rank, host_s = ctx.time_loop(table.launch, n, warmup=3)
    ms = ctx.max_over_ranks(ms_rank) / n
    res["independent_steps_in_one_launch"] = {
        "us_per_step": ms * 1e3, "us_per_call": ms * 1e3 / len(calls), "gbs": nbytes / (ms * 1e-3) / 1e9,
        "frac_of_measured_peak": nbytes / (ms * 1e-3) / 1e9 / ctx.peak, "kernel": V.last_kernel(),
        "host_enqueue_us_per_step": host_s / n * 1e6}
    res["bound"] = "launch"
    return res


def bench_shapes(ctx):
    """Device-resident prefill at the shapes of the whole-model configuration (batch 64 x 1024 tokens;
    Canon A/C 640, B 960, D 3456 channels; bf16; no bias, no activation, no mask: what the reference's
    layer passes by default) and one dense Canon-D batch of 128 sequences with bias and SiLU."""
    V, WL, dev = ctx.V, ctx.WL, ctx.dev
    out = {}
    g = torch.Generator(device=dev).manual_seed(5)
    specs = [("canon_a_c_b64", 64, 640, None, False), ("canon_b_b64", 64, 960, None, False),
             ("canon_d_b64", 64, 3456, None, False), ("canon_d_dense_b128_silu", 128, 3456, "silu", True)]
    for name, B, D, act, has_bias in specs:
        T, W = 1024, 4
        x = torch.randn(B, T, D, generator=g, device=dev).bfloat16()
        y = torch.empty_like(x)
        wt = (torch.rand(D, W, generator=g, device=dev) - 0.5).bfloat16()
        bt = (torch.rand(D, generator=g, device=dev) - 0.5).bfloat16() if has_bias else None
        xv, yv = x.transpose(1, 2), y.transpose(1, 2)

        def step():
            V.causal_conv1d_fn(xv, wt, bt, activation=act, out=yv)

        n = 20
        ms_rank, _ = ctx.time_loop(step, n, warmup=3)
        ms = ctx.max_over_ranks(ms_rank) / n
        nbytes = 2 * x.numel() * 2
        out[name] = {"batch": B, "seq_len": T, "channels": D, "activation": act, "bias": has_bias,
                     "kernel": V.last_kernel(), "us_per_launch": ms * 1e3, "bytes_per_launch": nbytes,
                     "achieved_gbs": nbytes / (ms * 1e-3) / 1e9,
                     "frac_of_measured_peak": nbytes / (ms * 1e-3) / 1e9 / ctx.peak,
                     "tokens_per_s": ctx.world * B * T / (ms * 1e-3)}
        del x, y
    return out


def bench_model_prefill_step(ctx):
    """The 72 Canon prefill calls of one forward pass of the whole-model configuration (18 blocks x Canon
    A, B, C, D at 640 / 960 / 640 / 3456 channels; batch 64 x 1024 tokens, bf16, no bias, no activation:
    the reference's defaults) with the padding mask applied inside the kernel, every call handed the same
    mask tensor as the reference's network does (model/model.py:1021-1055).  Tile classes are worked
    out once per tile height and kept for the other calls; the second figure does it on every call; the
    third is the dense call pattern of the reference's own layer (mask multiplied in beforehand)."""
    V, WL, dev = ctx.V, ctx.WL, ctx.dev
    B, T, W, layers = 64, 1024, 4, 18
    dims = [640, 960, 640, 3456]
    g = torch.Generator(device=dev).manual_seed(6)
    xs = {D: torch.randn(B, T, D, generator=g, device=dev).bfloat16() for D in set(dims)}
    ys = {D: torch.empty_like(x) for D, x in xs.items()}
    ws = {D: (torch.rand(D, W, generator=g, device=dev) - 0.5).bfloat16() for D in set(dims)}
    lens = torch.randint(128, T + 1, (B,), generator=torch.Generator().manual_seed(7))
    mask = (torch.arange(T)[None, :] < lens[:, None]).to(dev)
    valid = int(lens.sum())
    nbytes = layers * sum((valid + B * T) * D * 2 for D in dims)
    dense_bytes = layers * sum(2 * B * T * D * 2 for D in dims)

    def step(m):
        for _ in range(layers):
            for D in dims:
                V.causal_conv1d_fn(xs[D].transpose(1, 2), ws[D], None, attention_mask=m, out=ys[D].transpose(1, 2))

    out = {"calls_per_step": 4 * layers, "batch": B, "seq_len": T, "channels": dims, "layers": layers,
           "valid_tokens": valid, "bytes_per_step": nbytes, "dense_bytes_per_step": dense_bytes}
    for name, m, keep, nb in (("masked_classes_kept", mask, True, nbytes), ("masked_classified_every_call", mask, False, nbytes),
                              ("dense", None, True, dense_bytes)):
        was = V.reuse_tile_classes(keep)
        try:
            before = V.launch_count()
            ms_rank, host_s = ctx.time_loop(lambda: step(m), 5, warmup=2)
            launches = (V.launch_count() - before) // 7
        finally:
            V.reuse_tile_classes(was)
        ms = ctx.max_over_ranks(ms_rank) / 5
        out[name] = {"ms_per_step": ms, "us_per_call": ms * 1e3 / (4 * layers), "launches_per_step": launches,
                     "achieved_gbs": nb / (ms * 1e-3) / 1e9, "frac_of_measured_peak": nb / (ms * 1e-3) / 1e9 / ctx.peak,
                     "tokens_per_s": ctx.world * B * T / (ms * 1e-3), "host_enqueue_us_per_step": host_s / 5 * 1e6}
    return out


def bench_ragged(ctx, steps=10):
    """The ragged large-batch configuration: 512 sequences x up to 4096 tokens x 3456 channels, bf16,
    SiLU, lengths log-uniform in [16, 4096], right-padded and masked.  STRONG scaling: the 512
    sequences are split over the N ranks, once by cost (longest-processing-time on the bytes a
    sequence moves) and once as contiguous equal-count slices; no rank talks to another.  A third
    figure runs the by-cost shards as packed rows (seq_idx), which neither read nor write padding."""
    V, WL, dev, rank, world = ctx.V, ctx.WL, ctx.dev, ctx.rank, ctx.world
    from viby_model_b200.dist_util import shard_by_cost, shard_range

    cfg = WL.RAGGED_SWEEP
    lens_all = WL.sequence_lengths(cfg).tolist()
    w, b = WL.weights(cfg.cfg, cfg.dim, cfg.width, cfg.dtype, device=dev)
    elem = 2
    row_bytes = cfg.dim * elem

    def run(rows, packed):
        lens = [lens_all[i] for i in rows]
        x = WL.prefill_inputs(cfg, rows, device=dev, generate_on="cuda")
        if packed:
            xp = torch.cat([x[i, :n] for i, n in enumerate(lens)], 0).unsqueeze(0)
            del x
            yp = torch.empty_like(xp)
            ids = V.seq_idx_from_lengths(lens, device=dev)
            xv, yv = xp.transpose(1, 2), yp.transpose(1, 2)

            def step():
                V.causal_conv1d_fn(xv, w, b, activation=cfg.activation, seq_idx=ids, out=yv)

            my_bytes = 2 * sum(lens) * row_bytes
        else:
            m = WL.attention_mask(cfg, rows, device=dev, dtype=torch.bool)
            y = torch.empty_like(x)
            xv, yv = x.transpose(1, 2), y.transpose(1, 2)

            def step():
                V.causal_conv1d_fn(xv, w, b, activation=cfg.activation, attention_mask=m, out=yv)

            my_bytes = (sum(lens) + len(rows) * cfg.seqlen) * row_bytes
        ms_rank, _ = ctx.time_loop(step, steps, warmup=3)
        kernel = V.last_kernel()
        per_rank = [t / steps for t in ctx.gather(ms_rank)]
        bytes_rank = ctx.gather(float(my_bytes))
        ms = max(per_rank)
        total_bytes = sum(bytes_rank)
        gbs = total_bytes / (ms * 1e-3) / 1e9
        return {
            "kernel": kernel,
            "ms_per_step": ms,
            "per_rank_ms": spread(per_rank),
            "imbalance_max_over_mean": ms / (sum(per_rank) / len(per_rank)),
            "bytes_imbalance_max_over_mean": max(bytes_rank) / (total_bytes / len(bytes_rank)),
            "padded_tokens_per_s": cfg.batch * cfg.seqlen / (ms * 1e-3),
            "valid_tokens_per_s": sum(lens_all) / (ms * 1e-3),
            "algorithmic_bytes": total_bytes,
            "achieved_gbs_all_ranks": gbs,
            "frac_of_measured_peak_per_gpu": gbs / world / ctx.peak,
        }

    costs = [n + cfg.seqlen for n in lens_all]  # rows read + rows written
    by_cost = shard_by_cost(costs, world)[rank]
    contiguous = list(shard_range(cfg.batch, rank, world))
    res = {
        "config": {"workload": cfg.name, "global_batch": cfg.batch, "max_seq_len": cfg.seqlen, "channels": cfg.dim,
                   "lengths": "log-uniform in [16, 4096]", "valid_tokens": sum(lens_all),
                   "padded_tokens": cfg.batch * cfg.seqlen},
        "scaling": "strong",
        "n_gpus": world,
        "steps": steps,
        "sharded_by_cost": run(by_cost, False),
    }
    torch.cuda.empty_cache()
    res["sharded_contiguous"] = res["sharded_by_cost"] if world == 1 else run(contiguous, False)
    torch.cuda.empty_cache()
    packed_rows = shard_by_cost(lens_all, world)[rank]
    res["packed_rows_by_cost"] = run(packed_rows, True)
    torch.cuda.empty_cache()
    return res


if __name__ == "__main__":
    main()
