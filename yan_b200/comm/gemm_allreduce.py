"""The two sharded forms of the FP8 GEMM inside one NVSwitch box, one process per GPU.

They replace the reference's `comm/gemm_allreduce.cu:276-411`, which fuses a per-tile NVSHMEM NVLS allreduce
into a CUTLASS fp16 GEMM epilogue (row-parallel: every PE computes a full-size partial D, `:211-213,339-401`):

* N-split (column-parallel): rank r owns rows [r*N/g, (r+1)*N/g) of B and of its scales; A is replicated; each rank
  writes its own N/g output columns.  No communication.
* K-split (row-parallel): rank r owns columns [r*K/g, (r+1)*K/g) of A and B (cuts on multiples of 128, so
  quantizing a shard gives exactly the shard of the quantized tensor); each rank computes a full [M, N] partial
  and the partials are summed with an allreduce over NCCL (NVLink 5 / NVSwitch).  The rows are processed in
  chunks so that the allreduce of chunk i runs on a second stream while the GEMM of chunk i+1 computes.

* K-split with the two-shot peer-memory allreduce (`gemm_k_split_two_shot`): the GEMM writes its partial into a
  buffer the other ranks have mapped (peer_memory.TwoShotAllreduce) and one kernel per rank sums the ranks' buffers in
  place with plain peer loads and stores -- no NCCL call on the data path.

The GEMM itself never reads remote memory; TMA and MMA operands are always local.
`gemm_fn` lets host-side tests substitute the arithmetic; the default is the CUDA GEMM.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

Operand = Tuple[torch.Tensor, torch.Tensor]


def shard_n(rhs: Operand, rank: int, world: int) -> Operand:
    """Rows [rank*N/world, (rank+1)*N/world) of (e4m3 [N,K], scales [N/128, K/128]).  N/world must be a multiple of 128."""
    q, s = rhs
    n = q.shape[0]
    assert n % (128 * world) == 0, "each N shard must hold whole 128-row scale blocks"
    ns = n // world
    return q[rank * ns:(rank + 1) * ns], s[rank * ns // 128:(rank + 1) * ns // 128]


def shard_k(op: Operand, rank: int, world: int) -> Operand:
    """Columns [rank*K/world, (rank+1)*K/world) of an operand and the matching k-block columns of its scales
    (works for lhs = (e4m3 [M,K], [M,K/128]) and rhs = (e4m3 [N,K], [N/128,K/128]) alike)."""
    q, s = op
    k = q.shape[1]
    assert k % (128 * world) == 0, "each K shard must hold whole 128-wide k-blocks"
    ks = k // world
    return q[:, rank * ks:(rank + 1) * ks], s[:, rank * ks // 128:(rank + 1) * ks // 128]


def _default_gemm(out_dtype: torch.dtype) -> Callable:
    from ..jit_kernels.gemm import gemm_fp8_fp8_bf16_nt, gemm_fp8_fp8_f32_nt
    return gemm_fp8_fp8_bf16_nt if out_dtype == torch.bfloat16 else gemm_fp8_fp8_f32_nt


def gemm_n_split(lhs: Operand, rhs_shard: Operand, out: torch.Tensor, rank: int, world: int,
                 gemm_fn: Optional[Callable] = None) -> torch.Tensor:
    """out[:, rank*N/world : (rank+1)*N/world] = lhs . rhs_shard^T.

    `out` is either this rank's own [M, N/world] tensor or the full [M, N] buffer, of which only this rank's
    column slice is written (the kernel takes the row stride of the slice)."""
    m = lhs[0].shape[0]
    ns = rhs_shard[0].shape[0]
    if out.shape == (m, ns):
        target = out
    else:
        assert out.shape == (m, ns * world), "out must be [M, N/world] or [M, N]"
        target = out[:, rank * ns:(rank + 1) * ns]
    (gemm_fn or _default_gemm(torch.bfloat16))(lhs, rhs_shard, target)
    return target


def gemm_k_split_allreduce(lhs_shard: Operand, rhs_shard: Operand, out: torch.Tensor,
                           group: Optional[dist.ProcessGroup] = None, partial_dtype: torch.dtype = torch.bfloat16,
                           num_chunks: int = 1, gemm_fn: Optional[Callable] = None,
                           comm_stream: Optional["torch.cuda.Stream"] = None,
                           partial: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, N] (bf16) = sum over ranks of lhs_shard . rhs_shard^T.

    partial_dtype = bfloat16: each rank's partial is rounded to bf16 and the allreduce sums bf16 in place in `out`
    (the arithmetic the workload specifies).  partial_dtype = float32: partials stay fp32 (twice the bytes on the
    wire), are summed in fp32 and rounded to bf16 once.
    num_chunks > 1 splits the rows into chunks of whole 128-row tiles and overlaps chunk i's allreduce with chunk
    i+1's GEMM (CUDA tensors only)."""
    m = lhs_shard[0].shape[0]
    n = rhs_shard[0].shape[0]
    assert out.shape == (m, n) and out.dtype == torch.bfloat16
    assert partial_dtype in (torch.bfloat16, torch.float32)
    gemm = gemm_fn or _default_gemm(partial_dtype)
    if partial_dtype == torch.bfloat16:
        buf = out
    else:
        buf = partial if partial is not None else torch.empty((m, n), dtype=torch.float32, device=out.device)
        assert buf.shape == (m, n) and buf.dtype == torch.float32

    rows_per_chunk = max(128, -(-m // max(1, num_chunks)) // 128 * 128) if num_chunks > 1 else m
    bounds = [(r0, min(m, r0 + rows_per_chunk)) for r0 in range(0, m, rows_per_chunk)]
    qa, sa = lhs_shard
    overlap = out.is_cuda and len(bounds) > 1
    if overlap:
        comm_stream = comm_stream or torch.cuda.Stream(device=out.device)
        main = torch.cuda.current_stream(out.device)
        done = []
    for (r0, r1) in bounds:
        gemm((qa[r0:r1], sa[r0:r1]), rhs_shard, buf[r0:r1])
        if overlap:
            ready = torch.cuda.Event()
            ready.record(main)
            with torch.cuda.stream(comm_stream):
                comm_stream.wait_event(ready)
                dist.all_reduce(buf[r0:r1], op=dist.ReduceOp.SUM, group=group)
                if buf is not out:
                    out[r0:r1].copy_(buf[r0:r1])
                ev = torch.cuda.Event()
                ev.record(comm_stream)
                done.append(ev)
        else:
            dist.all_reduce(buf[r0:r1], op=dist.ReduceOp.SUM, group=group)
            if buf is not out:
                out[r0:r1].copy_(buf[r0:r1])
    if overlap:
        for ev in done:
            main.wait_event(ev)
    return out


def gemm_k_split_two_shot(lhs_shard: Operand, rhs_shard: Operand, comm, num_chunks: int = 1, comm_sms: int = 24,
                          gemm_fn: Optional[Callable] = None,
                          comm_stream: Optional["torch.cuda.Stream"] = None) -> torch.Tensor:
    """K-split GEMM whose partials are summed by the two-shot peer-memory kernel instead of NCCL.

    `comm` is a peer_memory.TwoShotAllreduce for [M, N]; the GEMM writes its bf16 partial straight into `comm.buffer`
    (peer-mapped memory), the kernel sums the ranks' buffers in place (fp32 sum, one rounding) and the result is
    returned in `comm.buffer` on every rank.  With num_chunks > 1 the rows go in chunks of whole 128-row tiles: the
    GEMM of chunk i+1 runs on all but `comm_sms` SMs while the allreduce of chunk i uses those on a second stream.
    Calls may follow one another on the same stream: a rank's allreduce kernel stores nothing before every rank has
    entered the same call, which each rank does only after its own earlier work on the buffer (stream order)."""
    from ..jit_kernels.utils import get_num_sms, set_num_sms
    m, n = comm.m, comm.n
    assert lhs_shard[0].shape[0] == m and rhs_shard[0].shape[0] == n
    gemm = gemm_fn or _default_gemm(torch.bfloat16)
    buf = comm.buffer
    qa, sa = lhs_shard
    if num_chunks <= 1:
        gemm(lhs_shard, rhs_shard, buf)
        comm.reduce_rows(0, m)
        return buf
    rows_per_chunk = max(128, -(-m // num_chunks) // 128 * 128)
    bounds = [(r0, min(m, r0 + rows_per_chunk)) for r0 in range(0, m, rows_per_chunk)]
    comm_stream = comm_stream or torch.cuda.Stream(device=buf.device)
    main = torch.cuda.current_stream(buf.device)
    all_sms = get_num_sms()
    try:
        for i, (r0, r1) in enumerate(bounds):
            # the first chunk has the GPU to itself; later ones share it with the allreduce of the chunk before
            set_num_sms(all_sms if i == 0 else max(1, all_sms - comm_sms))
            gemm((qa[r0:r1], sa[r0:r1]), rhs_shard, buf[r0:r1])
            ready = torch.cuda.Event()
            ready.record(main)
            with torch.cuda.stream(comm_stream):
                comm_stream.wait_event(ready)
                last = i + 1 == len(bounds)
                comm.reduce_rows(r0, r1, num_ctas=None if last else comm_sms, exclusive_sms=not last)
    finally:
        set_num_sms(all_sms)
    done = torch.cuda.Event()
    done.record(comm_stream)
    main.wait_event(done)
    return buf
