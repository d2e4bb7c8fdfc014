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
    """rhs: this rank's weights (e4m3 [N_local, K], scales).  m: rows of the activation matrix.

    group / shard_input: with several ranks that all hold the same activations in host memory (the column-parallel
    form: A replicated, B sharded along N), every rank would pull all of A over its host link.  With shard_input=True
    rank r copies and quantizes only rows [r*M/g, (r+1)*M/g) and the ranks exchange the quantized rows (e4m3 codes and
    scales, half the bytes of the bf16 rows) with one all-gather over NVLink; the GEMM then sees the same operand,
    bit for bit, as if the rank had quantized all of A itself (the quantizer works row by row)."""

    def __init__(self, rhs: Tuple[torch.Tensor, torch.Tensor], m: int, depth: int = 2, group=None,
                 shard_input: bool = False) -> None:
        rhs_q, rhs_scales = rhs
        assert rhs_q.is_cuda and rhs_q.dtype == torch.float8_e4m3fn
        self.rhs = (rhs_q, rhs_scales)
        self.n, self.k = rhs_q.shape
        self.m = m
        self.depth = depth
        self.group = group
        self.world, self.rank = 1, 0
        if shard_input:
            import torch.distributed as dist
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.shard_input = shard_input and self.world > 1
        assert m % self.world == 0, "the rows are dealt out evenly"
        self.m_local = m // self.world
        dev = rhs_q.device
        kb = self.k // 128
        self.copy_in, self.compute, self.copy_out = (torch.cuda.Stream(dev) for _ in range(3))
        self.a_dev = [torch.empty((self.m_local, self.k), dtype=torch.bfloat16, device=dev) for _ in range(depth)]
        self.lhs = [(torch.empty((m, self.k), dtype=torch.float8_e4m3fn, device=dev),
                     torch.empty((kb, m), dtype=torch.float32, device=dev).t()) for _ in range(depth)]
        if self.shard_input:
            # this rank's quantized rows, and the scales of all ranks as they arrive: [rank][k-block][row]
            self.lhs_local = [(torch.empty((self.m_local, self.k), dtype=torch.float8_e4m3fn, device=dev),
                               torch.empty((kb, self.m_local), dtype=torch.float32, device=dev).t()) for _ in range(depth)]
            self.scales_gathered = [torch.empty((self.world, kb, self.m_local), dtype=torch.float32, device=dev)
                                    for _ in range(depth)]
        self.out_dev = [torch.empty((m, self.n), dtype=torch.bfloat16, device=dev) for _ in range(depth)]
        self.in_ready = [torch.cuda.Event() for _ in range(depth)]
        self.computed = [torch.cuda.Event() for _ in range(depth)]
        self.out_done = [torch.cuda.Event() for _ in range(depth)]
        self.calls = 0

    def h2d_bytes_per_call(self) -> int:
        return self.m_local * self.k * 2

    def _quantize(self, s: int) -> None:
        """Fills self.lhs[s] (all M rows) from self.a_dev[s] (this rank's rows)."""
        if not self.shard_input:
            per_token_cast_to_fp8(self.a_dev[s], out=self.lhs[s])
            return
        import torch.distributed as dist
        q_local, s_local = self.lhs_local[s]
        per_token_cast_to_fp8(self.a_dev[s], out=(q_local, s_local))
        q_full, s_full = self.lhs[s]
        dist.all_gather_into_tensor(q_full.view(torch.uint8), q_local.view(torch.uint8), group=self.group)
        dist.all_gather_into_tensor(self.scales_gathered[s], s_local.t(), group=self.group)
        # [rank][k-block][row] -> k-block-major over all M rows
        kb = self.k // 128
        s_full.t().view(kb, self.world, self.m_local).copy_(self.scales_gathered[s].permute(1, 0, 2))

    def submit(self, a_host: torch.Tensor, out_host: torch.Tensor) -> None:
        """a_host: pinned bf16 [M, K] (with shard_input only this rank's rows are read); out_host: pinned bf16
        [M, N_local].  Returns at once; see wait()."""
        assert a_host.is_pinned() and out_host.is_pinned()
        assert a_host.shape == (self.m, self.k) and out_host.shape == (self.m, self.n)
        s = self.calls % self.depth
        caller = torch.cuda.current_stream()
        self.copy_in.wait_stream(caller)
        rows = a_host[self.rank * self.m_local:(self.rank + 1) * self.m_local]
        with torch.cuda.stream(self.copy_in):
            if self.calls >= self.depth:
                self.copy_in.wait_event(self.computed[s])     # the kernels that read this slot are done
            self.a_dev[s].copy_(rows, non_blocking=True)
            self.in_ready[s].record(self.copy_in)
        with torch.cuda.stream(self.compute):
            self.compute.wait_event(self.in_ready[s])
            if self.calls >= self.depth:
                self.compute.wait_event(self.out_done[s])     # the previous output of this slot has left the device
            self._quantize(s)
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
