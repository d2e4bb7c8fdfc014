"""Host-buffer front end of the bf16-in / bf16-out path: activations arrive in pinned host memory, outputs go
back to pinned host memory, weights stay resident on the device.

`HostFp8Linear.submit(a_host, out_host)` enqueues  host->device copy, quantize (1x128), FP8 GEMM, device->host copy
on three streams with `depth` rotating device buffers, so the copies of one call overlap the kernels of its
neighbours; `wait()` blocks until everything submitted so far has landed in `out_host`.  The reference has no host
path (its operators take device tensors only, yan/jit_kernels/cute_gemm.py:21-31); this is the call a user with
host-resident activations makes.
"""
from __future__ import annotations

from typing import Tuple

import torch

from .gemm import gemm_fp8_fp8_bf16_nt
from .quant import per_token_cast_to_fp8


class HostFp8Linear:
    def __init__(self, rhs: Tuple[torch.Tensor, torch.Tensor], m: int, depth: int = 2) -> None:
        rhs_q, rhs_scales = rhs
        assert rhs_q.is_cuda and rhs_q.dtype == torch.float8_e4m3fn
        self.rhs = (rhs_q, rhs_scales)
        self.n, self.k = rhs_q.shape
        self.m = m
        self.depth = depth
        dev = rhs_q.device
        self.copy_in, self.compute, self.copy_out = (torch.cuda.Stream(dev) for _ in range(3))
        self.a_dev = [torch.empty((m, self.k), dtype=torch.bfloat16, device=dev) for _ in range(depth)]
        self.lhs = [(torch.empty((m, self.k), dtype=torch.float8_e4m3fn, device=dev),
                     torch.empty((self.k // 128, m), dtype=torch.float32, device=dev).t()) for _ in range(depth)]
        self.out_dev = [torch.empty((m, self.n), dtype=torch.bfloat16, device=dev) for _ in range(depth)]
        self.in_ready = [torch.cuda.Event() for _ in range(depth)]
        self.computed = [torch.cuda.Event() for _ in range(depth)]
        self.out_done = [torch.cuda.Event() for _ in range(depth)]
        self.calls = 0

    def submit(self, a_host: torch.Tensor, out_host: torch.Tensor) -> None:
        """a_host: pinned bf16 [M, K]; out_host: pinned bf16 [M, N].  Returns at once; see wait()."""
        assert a_host.is_pinned() and out_host.is_pinned()
        assert a_host.shape == (self.m, self.k) and out_host.shape == (self.m, self.n)
        s = self.calls % self.depth
        caller = torch.cuda.current_stream()
        self.copy_in.wait_stream(caller)
        with torch.cuda.stream(self.copy_in):
            if self.calls >= self.depth:
                self.copy_in.wait_event(self.computed[s])     # the kernels that read this slot are done
            self.a_dev[s].copy_(a_host, non_blocking=True)
            self.in_ready[s].record(self.copy_in)
        with torch.cuda.stream(self.compute):
            self.compute.wait_event(self.in_ready[s])
            if self.calls >= self.depth:
                self.compute.wait_event(self.out_done[s])     # the previous output of this slot has left the device
            per_token_cast_to_fp8(self.a_dev[s], out=self.lhs[s])
            gemm_fp8_fp8_bf16_nt(self.lhs[s], self.rhs, self.out_dev[s])
            self.computed[s].record(self.compute)
        with torch.cuda.stream(self.copy_out):
            self.copy_out.wait_event(self.computed[s])
            out_host.copy_(self.out_dev[s], non_blocking=True)
            self.out_done[s].record(self.copy_out)
        self.calls += 1

    def wait(self) -> None:
        """Makes the caller's stream wait for every submitted call, then blocks the host until they are done."""
        caller = torch.cuda.current_stream()
        caller.wait_stream(self.copy_out)
        caller.wait_stream(self.compute)
        caller.wait_stream(self.copy_in)
        caller.synchronize()
