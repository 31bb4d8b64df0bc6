"""Prefill for callers whose tensors live in host memory.

``HostPrefill`` streams a pinned-host batch through the GPU in batch chunks on three CUDA
streams -- host-to-device copy, kernel, device-to-host copy -- so the copies of one chunk
overlap the kernel of the next and the two PCIe directions run concurrently.  The device
buffers are allocated once, in the constructor; ``run`` allocates nothing on the device.

Two things keep the PCIe link, which bounds this path, busy with useful bytes only:
  * rows behind a sequence's last valid position are never read by the kernels (masked loads are
    skipped), so they are not sent: only ``x[b, :last_valid_b]`` crosses the link;
  * with ``join=False`` consecutive ``run`` calls pipeline into each other (the copy-in of the next
    batch overlaps the copy-out of the previous one); buffer reuse is ordered by events per chunk;
  * with ``skip_constant_rows`` output rows that lie ``width - 1`` or more steps behind a sequence's last
    valid position are not copied back either: every tap of such a row is masked, so the row is the
    per-channel constant ``act(bias)``, which the host writes into ``y_host`` itself from one ``[dim]``
    vector while the copies run.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np
from concurrent.futures import ThreadPoolExecutor
from typing import Optional

import torch

from .ops import causal_conv1d_fn


NUMA_STATUS = {}  # device index -> why bind_to_gpu_numa_node returned what it did


def bind_to_gpu_numa_node(device_index: int) -> Optional[int]:
    """Pin the calling process to the CPUs of the NUMA node the GPU hangs off, so that pinned host
    buffers allocated afterwards (first touch) and the copy threads sit next to its PCIe root.
    With one process per GPU on a multi-socket host this keeps host<->device copies off the
    inter-socket link.  Returns the node, or None when the topology cannot be read (nothing is
    changed then); ``NUMA_STATUS[device_index]`` says which."""
    node = _bind_to_gpu_numa_node(device_index)
    NUMA_STATUS.setdefault(device_index, f"bound to node {node}")
    return node


def _nvml_cpu_set(device_index: int):
    """CPUs NVML considers local to the GPU (its NUMA node), or None.  Works where sysfs does not
    expose the PCI device's node, as inside some containers."""
    try:
        import os

        import pynvml

        pynvml.nvmlInit()
        props = torch.cuda.get_device_properties(device_index)
        uuid = str(props.uuid)
        h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
        words = (max(os.sched_getaffinity(0)) // 64) + 1
        try:
            mask = pynvml.nvmlDeviceGetCpuAffinityWithinScope(h, words, pynvml.NVML_AFFINITY_SCOPE_NODE)
        except Exception:
            mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * i + bit for i, word in enumerate(mask) for bit in range(64) if (int(word) >> bit) & 1}
        return cpus or None
    except Exception:
        return None


def _bind_to_gpu_numa_node(device_index: int) -> Optional[int]:
    import os

    try:
        props = torch.cuda.get_device_properties(device_index)
        if hasattr(props, "pci_bus_id"):
            bus = f"{getattr(props, 'pci_domain_id', 0):04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        else:
            import pynvml

            pynvml.nvmlInit()
            uuid = str(props.uuid)
            h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
            bus = pynvml.nvmlDeviceGetPciInfo(h).busId
            bus = (bus.decode() if isinstance(bus, bytes) else bus).lower()[-12:]
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            cpus = _nvml_cpu_set(device_index)
            allowed = (cpus or set()) & os.sched_getaffinity(0)
            if allowed and len(allowed) < len(os.sched_getaffinity(0)):
                os.sched_setaffinity(0, allowed)
                NUMA_STATUS[device_index] = (f"sysfs reports numa_node = {node}; bound to the {len(allowed)} CPUs NVML "
                                             f"lists as local to the GPU")
                return -1
            NUMA_STATUS[device_index] = (f"/sys/bus/pci/devices/{bus}/numa_node = {node} and NVML names no smaller "
                                         f"CPU set: the host exposes no NUMA topology")
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            NUMA_STATUS[device_index] = f"node {node}: none of its CPUs is in this process's affinity mask"
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except Exception as e:
        NUMA_STATUS[device_index] = f"topology not readable: {type(e).__name__}: {e}"
        return None


class HostPrefill:
    def __init__(self, batch: int, seqlen: int, dim: int, dtype: torch.dtype, device="cuda",
                 chunk_batch: int = 4, masked: bool = True, mask_dtype: torch.dtype = torch.int64,
                 send_masked_rows: bool = False, skip_constant_rows: bool = False, copy_streams: int = 1,
                 fill_workers: Optional[int] = None):
        self.device = torch.device(device)
        self.batch, self.seqlen, self.dim, self.dtype = batch, seqlen, dim, dtype
        self.chunk = max(1, min(chunk_batch, batch))
        self.send_masked_rows = send_masked_rows  # True: copy all of x, also the rows no kernel reads
        self.skip_constant_rows = skip_constant_rows and masked  # True: act(bias) rows are written by the host
        self.const_dev = torch.empty(1, 1, dim, dtype=dtype, device=self.device)
        self.const_host = torch.empty(1, 1, dim, dtype=dtype).pin_memory()
        self.zero_in = torch.zeros(1, 1, dim, dtype=dtype, device=self.device)
        self.zero_mask = torch.zeros(1, 1, dtype=mask_dtype, device=self.device) if masked else None
        self.last_d2h_bytes = 0
        self._fill = True  # (timing experiments switch the host-side fill off; results are then incomplete)
        # the host-side fill: plain memory copies out of a block of constant rows, on a few worker threads
        self._fill_workers = (max(1, int(fill_workers)) if fill_workers is not None
                              else max(1, min(8, (os.cpu_count() or 2) // 2)))
        self._pool = ThreadPoolExecutor(max_workers=self._fill_workers) if self.skip_constant_rows else None
        self._fill_futures = []
        self._const_blocks = ([torch.empty(256, dim, dtype=dtype) for _ in range(2)]
                              if self.skip_constant_rows else None)
        self._runs = 0
        self.x_dev = torch.empty(batch, seqlen, dim, dtype=dtype, device=self.device)
        self.y_dev = torch.empty_like(self.x_dev)
        self.m_dev = torch.empty(batch, seqlen, dtype=mask_dtype, device=self.device) if masked else None
        # copies of consecutive chunks can alternate between copy_streams streams per direction (measured on
        # one B200: 1 to 4 streams and chunks of 2 to 8 sequences all give the same rate, the link's)
        k = max(1, int(copy_streams))
        self.s_h2d_all = [torch.cuda.Stream(self.device) for _ in range(k)]
        self.s_d2h_all = [torch.cuda.Stream(self.device) for _ in range(k)]
        self.s_run = torch.cuda.Stream(self.device)
        self.s_const = torch.cuda.Stream(self.device)  # the constant row: must not queue behind earlier batches
        n = (batch + self.chunk - 1) // self.chunk
        self.ev_in = [torch.cuda.Event() for _ in range(n)]
        self.ev_run = [torch.cuda.Event() for _ in range(n)]
        self.ev_out = [torch.cuda.Event() for _ in range(n)]
        self.last_h2d_bytes = 0  # bytes the most recent run() sent to the device

    @property
    def h2d_bytes(self) -> int:
        """Bytes the most recent run() copied to the device (all of x and the mask before any run)."""
        if self.last_h2d_bytes:
            return self.last_h2d_bytes
        n = self.x_dev.numel() * self.x_dev.element_size()
        if self.m_dev is not None:
            n += self.m_dev.numel() * self.m_dev.element_size()
        return n

    @property
    def d2h_bytes(self) -> int:
        """Bytes the most recent run() copied back to the host (all of y before any run)."""
        if self.last_d2h_bytes:
            return self.last_d2h_bytes
        return self.y_dev.numel() * self.y_dev.element_size()

    @staticmethod
    def valid_prefix_lengths(mask_host: torch.Tensor) -> list:
        """Per sequence, the index after its last non-zero mask entry (0 when all are zero)."""
        # (numpy on purpose: a parallel region of the tensor library here would leave its worker threads
        # spinning on the cores that the copy and fill threads of this class need)
        m = mask_host.view(torch.uint8).numpy() if mask_host.dtype == torch.bool else mask_host.float().numpy()
        nz = m != 0
        T = nz.shape[1]
        last = T - np.argmax(nz[:, ::-1], axis=1)
        return np.where(nz.any(axis=1), last, 0).tolist()

    def run(self, x_host: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], activation,
            mask_host: Optional[torch.Tensor], y_host: torch.Tensor, *, join: bool = True) -> torch.Tensor:
        """x_host, y_host: pinned ``[batch, seqlen, dim]``; mask_host: pinned ``[batch, seqlen]`` or None.
        Returns y_host.  With ``join=True`` all work has been ordered into the caller's current stream on
        return; with ``join=False`` call ``join()`` (or wait on ``ev_out[-1]``) before reading y_host."""
        main = torch.cuda.current_stream(self.device)
        for s in self.s_h2d_all:
            s.wait_stream(main)  # the inputs may come from work queued on the caller's stream
        masked = self.m_dev is not None and mask_host is not None
        lens = self.valid_prefix_lengths(mask_host) if masked else None
        if self.send_masked_rows and lens is not None:
            lens = [self.seqlen] * self.batch
        row_bytes = self.dim * self.x_dev.element_size()
        sent = 0
        received = 0
        out_rows = None
        if self.skip_constant_rows and masked:
            # rows from out_rows[b] on have every tap masked: they equal act(bias) in every sequence.
            # One masked single-step launch computes that row; the host fills it in while the copies run.
            width = weight.shape[1]
            out_rows = [min(self.seqlen, n + width - 1) for n in self.valid_prefix_lengths(mask_host)]
            with torch.cuda.stream(self.s_const):
                self.s_const.wait_stream(main)
                causal_conv1d_fn(self.zero_in.transpose(1, 2), weight, bias, activation=activation,
                                 attention_mask=self.zero_mask, out=self.const_dev.transpose(1, 2))
                self.const_host.copy_(self.const_dev, non_blocking=True)
                const_ready = torch.cuda.Event()
                const_ready.record(self.s_const)
            received += row_bytes
        for i, b0 in enumerate(range(0, self.batch, self.chunk)):
            b1 = min(b0 + self.chunk, self.batch)
            s_h2d = self.s_h2d_all[i % len(self.s_h2d_all)]
            s_d2h = self.s_d2h_all[i % len(self.s_d2h_all)]
            with torch.cuda.stream(s_h2d):
                s_h2d.wait_event(self.ev_run[i])  # the previous batch's kernel has read this chunk
                if masked:
                    for b in range(b0, b1):
                        if lens[b] > 0:
                            self.x_dev[b, : lens[b]].copy_(x_host[b, : lens[b]], non_blocking=True)
                            sent += lens[b] * row_bytes
                    self.m_dev[b0:b1].copy_(mask_host[b0:b1], non_blocking=True)
                    sent += (b1 - b0) * self.seqlen * self.m_dev.element_size()
                else:
                    self.x_dev[b0:b1].copy_(x_host[b0:b1], non_blocking=True)
                    sent += (b1 - b0) * self.seqlen * row_bytes
                self.ev_in[i].record(s_h2d)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(self.ev_in[i])
                self.s_run.wait_event(self.ev_out[i])  # the previous batch's result has left this chunk
                causal_conv1d_fn(
                    self.x_dev[b0:b1].transpose(1, 2), weight, bias, activation=activation,
                    attention_mask=self.m_dev[b0:b1] if masked else None,
                    out=self.y_dev[b0:b1].transpose(1, 2),
                )
                self.ev_run[i].record(self.s_run)
            with torch.cuda.stream(s_d2h):
                s_d2h.wait_event(self.ev_run[i])
                if out_rows is None:
                    y_host[b0:b1].copy_(self.y_dev[b0:b1], non_blocking=True)
                    received += (b1 - b0) * self.seqlen * row_bytes
                else:
                    for b in range(b0, b1):
                        if out_rows[b] > 0:
                            y_host[b, : out_rows[b]].copy_(self.y_dev[b, : out_rows[b]], non_blocking=True)
                            received += out_rows[b] * row_bytes
                self.ev_out[i].record(s_d2h)
        if out_rows is not None and self._fill:
            # the host writes the constant rows on a worker thread while this thread goes on enqueueing (the
            # fill of a Canon-D batch takes a few milliseconds of host time: about as long as the copies)
            self._wait_fill(keep=1)  # the fill of the batch before the previous one has long finished
            const_ready.synchronize()  # a [dim] vector on a stream of its own: a few tens of microseconds
            blk = self._const_blocks[self._runs % 2]  # (the previous batch's fill may still be reading the other)
            self._runs += 1
            for r in range(blk.shape[0]):  # plain copies: no parallel region of the tensor library on this path
                ctypes.memmove(blk[r].data_ptr(), self.const_host.data_ptr(), row_bytes)
            src, block_bytes = blk.data_ptr(), blk.numel() * blk.element_size()
            pieces = []  # (destination address, bytes): at most const_block rows each
            for b in range(self.batch):
                at = y_host[b, out_rows[b]:].data_ptr() if out_rows[b] < self.seqlen else 0
                left = (self.seqlen - out_rows[b]) * row_bytes
                while left > 0:
                    n = min(left, block_bytes)
                    pieces.append((at, n))
                    at += n
                    left -= n
            k = self._fill_workers

            def fill(part):
                for dst, n in part:
                    ctypes.memmove(dst, src, n)  # releases the GIL

            self._fill_futures.append([self._pool.submit(fill, pieces[i::k]) for i in range(k)])
        self.last_h2d_bytes = sent
        self.last_d2h_bytes = received
        if join:
            self.join()
        return y_host

    def _wait_fill(self, keep: int = 0) -> None:
        """Wait for the host-side fills of all but the ``keep`` most recent run() calls."""
        while len(self._fill_futures) > keep:
            for f in self._fill_futures.pop(0):
                f.result()

    def join(self) -> None:
        """Order everything queued so far into the caller's current stream (and wait for the host-side
        fill of the constant rows, when there is one)."""
        self._wait_fill()
        main = torch.cuda.current_stream(self.device)
        for s in self.s_d2h_all + [self.s_run, self.s_const] + self.s_h2d_all:
            main.wait_stream(s)
