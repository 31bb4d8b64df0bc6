"""Prefill for callers whose tensors live in host memory.

``HostPrefill`` streams a pinned-host batch through the GPU in batch chunks on three CUDA
streams -- host-to-device copy, kernel, device-to-host copy -- so the copies of one chunk
overlap the kernel of the next and the two PCIe directions run concurrently.  The device
buffers are allocated once, in the constructor; ``run`` allocates nothing.
"""
from __future__ import annotations

from typing import Optional

import torch

from .ops import causal_conv1d_fn


class HostPrefill:
    def __init__(self, batch: int, seqlen: int, dim: int, dtype: torch.dtype, device="cuda",
                 chunk_batch: int = 4, masked: bool = True, mask_dtype: torch.dtype = torch.int64):
        self.device = torch.device(device)
        self.batch, self.seqlen, self.dim, self.dtype = batch, seqlen, dim, dtype
        self.chunk = max(1, min(chunk_batch, batch))
        self.x_dev = torch.empty(batch, seqlen, dim, dtype=dtype, device=self.device)
        self.y_dev = torch.empty_like(self.x_dev)
        self.m_dev = torch.empty(batch, seqlen, dtype=mask_dtype, device=self.device) if masked else None
        self.s_h2d = torch.cuda.Stream(self.device)
        self.s_run = torch.cuda.Stream(self.device)
        self.s_d2h = torch.cuda.Stream(self.device)
        n = (batch + self.chunk - 1) // self.chunk
        self.ev_in = [torch.cuda.Event() for _ in range(n)]
        self.ev_run = [torch.cuda.Event() for _ in range(n)]

    @property
    def h2d_bytes(self) -> int:
        n = self.x_dev.numel() * self.x_dev.element_size()
        if self.m_dev is not None:
            n += self.m_dev.numel() * self.m_dev.element_size()
        return n

    @property
    def d2h_bytes(self) -> int:
        return self.y_dev.numel() * self.y_dev.element_size()

    def run(self, x_host: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], activation,
            mask_host: Optional[torch.Tensor], y_host: torch.Tensor) -> torch.Tensor:
        """x_host, y_host: pinned ``[batch, seqlen, dim]``; mask_host: pinned ``[batch, seqlen]`` or None.
        Returns y_host; on return all work has been ordered into the caller's current stream."""
        main = torch.cuda.current_stream(self.device)
        for s in (self.s_h2d, self.s_run, self.s_d2h):
            s.wait_stream(main)
        for i, b0 in enumerate(range(0, self.batch, self.chunk)):
            b1 = min(b0 + self.chunk, self.batch)
            with torch.cuda.stream(self.s_h2d):
                self.x_dev[b0:b1].copy_(x_host[b0:b1], non_blocking=True)
                if self.m_dev is not None and mask_host is not None:
                    self.m_dev[b0:b1].copy_(mask_host[b0:b1], non_blocking=True)
                self.ev_in[i].record(self.s_h2d)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(self.ev_in[i])
                causal_conv1d_fn(
                    self.x_dev[b0:b1].transpose(1, 2), weight, bias, activation=activation,
                    attention_mask=self.m_dev[b0:b1] if (self.m_dev is not None and mask_host is not None) else None,
                    out=self.y_dev[b0:b1].transpose(1, 2),
                )
                self.ev_run[i].record(self.s_run)
            with torch.cuda.stream(self.s_d2h):
                self.s_d2h.wait_event(self.ev_run[i])
                y_host[b0:b1].copy_(self.y_dev[b0:b1], non_blocking=True)
        main.wait_stream(self.s_d2h)
        main.wait_stream(self.s_run)
        main.wait_stream(self.s_h2d)
        return y_host
