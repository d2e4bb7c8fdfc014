"""Peer-mapped device memory and the two-shot allreduce kernel for the ranks of one NVSwitch box.

The reference keeps its partial tiles in an NVSHMEM symmetric heap and reduces them with NVLS multimem loads inside
the GEMM epilogue (comm/gemm_allreduce.cu:57-60,238-259,339-401).  This module gets the same effect -- a buffer every
rank of the box can load from and store to -- with CUDA IPC handles exchanged through the process group, and sums the
K-split partials with one kernel per rank over plain peer pointers (include/comm/peer_allreduce.cuh).
One process per GPU; all ranks must be on the same machine.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import _lib

SIGNAL_BYTES = 128  # one PeerSignals block (include/comm/peer_allreduce.cuh)

# (pid of the exporter, handle bytes) -> [mapped base address, reference count]: an allocation is mapped once per process
_opened: Dict[Tuple[int, bytes], List[int]] = {}


def slice_bounds(count: int, world: int, rank: int) -> Tuple[int, int]:
    """The part of `count` 16-byte vectors that `rank` reduces: ceil(count/world) vectors from rank*ceil(count/world),
    clipped to the range (the last ranks of a short range may own nothing).  Mirrors the kernel's arithmetic."""
    per = -(-count // world)
    first = min(count, rank * per)
    return first, min(count, first + per)


class PeerSharedTensor:
    """`local` is this rank's tensor; `ptrs[r]` is the address of rank r's tensor in this process."""

    def __init__(self, shape, dtype: torch.dtype, group: Optional[dist.ProcessGroup] = None, device: str = "cuda"):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.local = torch.zeros(shape, dtype=dtype, device=device)  # `device` exists for host-side tests of the hand-shake
        # Every step that can fail on one rank only is followed by an exchange of the outcome, so that all ranks raise
        # together instead of one leaving the others inside a collective.
        try:
            handle = (ctypes.c_ubyte * 64)()
            offset = ctypes.c_ulonglong(0)
            _lib.call("yan_b200_ipc_export", ctypes.c_void_p(self.local.data_ptr()), handle, ctypes.byref(offset))
            mine = (os.getpid(), bytes(handle), int(offset.value), None)
        except Exception as e:  # noqa: BLE001 - reported to every rank below
            mine = (os.getpid(), b"", 0, f"rank {self.rank}: {type(e).__name__}: {e}")
        everyone: list = [None] * self.world
        dist.all_gather_object(everyone, mine, group=group)
        errors = [e[3] for e in everyone if e[3] is not None]
        if errors:
            raise RuntimeError("peer memory export failed: " + "; ".join(errors))
        self._keys: List[Tuple[int, bytes]] = []
        self.ptrs: List[int] = []
        failure = None
        for r, (pid, h, off, _err) in enumerate(everyone):
            if r == self.rank:
                self.ptrs.append(self.local.data_ptr())
                continue
            key = (pid, h)
            try:
                if key not in _opened:
                    base = ctypes.c_void_p(0)
                    buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                    _lib.call("yan_b200_ipc_open", buf, ctypes.byref(base))
                    _opened[key] = [int(base.value), 0]
                _opened[key][1] += 1
                self._keys.append(key)
                self.ptrs.append(_opened[key][0] + off)
            except Exception as e:  # noqa: BLE001
                failure = f"rank {self.rank} mapping rank {r}: {type(e).__name__}: {e}"
                break
        outcomes: list = [None] * self.world
        dist.all_gather_object(outcomes, failure, group=group)
        if any(o is not None for o in outcomes):
            self._unmap()
            raise RuntimeError("peer memory mapping failed: " + "; ".join(o for o in outcomes if o is not None))
        if self.local.is_cuda:
            torch.cuda.synchronize()
        dist.barrier(group=group)  # every rank has mapped every buffer (and zeroed its own) before anyone uses them

    def ptr_array(self):
        return (ctypes.c_void_p * self.world)(*self.ptrs)

    def _unmap(self) -> None:
        for key in self._keys:
            entry = _opened[key]
            entry[1] -= 1
            if entry[1] == 0:
                _lib.call("yan_b200_ipc_close", ctypes.c_void_p(entry[0]))
                del _opened[key]
        self._keys = []

    def close(self) -> None:
        """Unmaps the peers' buffers.  Collective: no rank may still be using this rank's buffer."""
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self._unmap()


class MulticastSharedTensor:
    """Like PeerSharedTensor, with the ranks' tensors additionally bound to one NVSwitch multicast object:
    `multicast_ptr` addresses all copies at once (multimem instructions).  The allocation and the handle exchange are
    PyTorch's (torch.distributed._symmetric_memory); this class only reads the addresses."""

    def __init__(self, shape, dtype: torch.dtype, group: Optional[dist.ProcessGroup] = None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.local = symm_mem.empty(shape, dtype=dtype, device="cuda")
        self._handle = symm_mem.rendezvous(self.local, group if group is not None else dist.group.WORLD)
        self.ptrs = [int(p) for p in self._handle.buffer_ptrs]
        self.multicast_ptr = int(self._handle.multicast_ptr)
        if self.multicast_ptr == 0:
            raise RuntimeError("this allocation has no multicast mapping (no NVSwitch multicast support)")
        self.local.zero_()
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def ptr_array(self):
        return (ctypes.c_void_p * self.world)(*self.ptrs)

    def close(self) -> None:
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self._handle = None


class CollectiveClock:
    """Host half of the allreduce kernels' ordering state: the epoch the next launch announces to its peers and the
    value this rank's CTA counter reaches when that launch's last CTA is through.  The device half lives in the
    signal block (`PeerSignals` in include/comm/peer_allreduce.cuh).  Every launch advances both halves by the same
    amounts whether its waits ran out or not, so one timed-out call does not poison the next; `reset` starts over
    after the signal block has been zeroed."""

    def __init__(self) -> None:
        self.epoch = 0
        self.cta_count = 0

    def next_launch(self, ctas: int):
        """(epoch, counter_target) of a launch with `ctas` CTAs."""
        assert ctas > 0
        self.epoch = (self.epoch + 1) & 0xFFFFFFFF or 1  # 0 means "the caller orders the ranks"
        self.cta_count = (self.cta_count + ctas) & 0xFFFFFFFF
        return self.epoch, self.cta_count

    def reset(self) -> None:
        self.epoch = 0
        self.cta_count = 0


class TwoShotAllreduce:
    """In-place sum over the ranks of a peer-shared bf16 matrix [M, N] (`buffer`): the GEMM writes its partial product
    into `buffer`, `reduce_rows` leaves the sum of all ranks' partials there on every rank.

    device_barriers=True : the kernel orders the ranks itself with epoch flags in peer memory (bounded waits).
    device_barriers=False: the ranks are ordered by a one-element NCCL allreduce before and after the kernel.
    in_switch=False: each rank loads its slice from every buffer, adds, and stores the sum to every buffer.
    in_switch=True : the buffers are bound to an NVSwitch multicast object and the sum is formed in the switch
                     (multimem.ld_reduce / multimem.st); less NVLink traffic per GPU, needs multicast support.
    """

    def __init__(self, m: int, n: int, group: Optional[dist.ProcessGroup] = None, device_barriers: bool = True,
                 num_ctas: Optional[int] = None, in_switch: bool = False):
        assert n % 8 == 0, "rows are moved in 16-byte vectors"
        self.group = group
        self.m, self.n = m, n
        self.in_switch = in_switch
        # one allocation: the matrix, then the signal block
        arena_type = MulticastSharedTensor if in_switch else PeerSharedTensor
        self._arena = arena_type((m * n * 2 + SIGNAL_BYTES,), torch.uint8, group)
        self.rank, self.world = self._arena.rank, self._arena.world
        assert 2 <= self.world <= 8
        self.buffer = self._arena.local[: m * n * 2].view(torch.bfloat16).view(m, n)
        self._data = self._arena.ptr_array()
        self._signals = (ctypes.c_void_p * self.world)(*[p + m * n * 2 for p in self._arena.ptrs])
        self.device_barriers = device_barriers
        sms = torch.cuda.get_device_properties(self.buffer.device).multi_processor_count
        self.num_ctas = num_ctas or sms  # one CTA per SM saturates the links (measured)
        self._clock = CollectiveClock()
        self._token = torch.zeros(1, dtype=torch.float32, device="cuda")

    def reduce_rows(self, row_begin: int = 0, row_end: Optional[int] = None, num_ctas: Optional[int] = None,
                    exclusive_sms: bool = False) -> None:
        """Allreduce of rows [row_begin, row_end) on the current stream.  Every rank makes the same calls in the same
        order.  exclusive_sms: the kernel's CTAs fill one SM each, so it occupies exactly `num_ctas` SMs (for running
        beside a GEMM that was given the other SMs)."""
        row_end = self.m if row_end is None else row_end
        assert 0 <= row_begin < row_end <= self.m
        ctas = num_ctas or self.num_ctas
        stream = _lib.current_stream_ptr()
        begin, count = row_begin * self.n, (row_end - row_begin) * self.n
        if self.in_switch:
            name, target = "yan_b200_allreduce_bf16_in_switch", ctypes.c_void_p(self._arena.multicast_ptr)
        else:
            name, target = "yan_b200_allreduce_bf16_two_shot", self._data
        if self.device_barriers:
            epoch, counter_target = self._clock.next_launch(ctas)
            _lib.call(name, target, self._signals, self.world, self.rank, begin, count, epoch, counter_target,
                      ctas, int(exclusive_sms), stream)
        else:
            dist.all_reduce(self._token, group=self.group)  # every rank's partial is complete
            _lib.call(name, target, None, self.world, self.rank, begin, count, 0, 0, ctas, int(exclusive_sms), stream)
            dist.all_reduce(self._token, group=self.group)  # every rank's stores have landed

    def reset(self) -> None:
        """Collective: every rank calls it after a reported wait expiry (or whenever the ranks want a clean slate).
        Waits for all ranks' work, zeroes every signal block and restarts the epochs."""
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self._arena.local[self.m * self.n * 2:].zero_()
        self._clock.reset()
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    def close(self) -> None:
        self._arena.close()


class TileFusedAllreduce:
    """The K-split GEMM fused with its allreduce, tile by tile (the shape of the reference's epilogue,
    comm/gemm_allreduce.cu:339-410, without NVSHMEM).

    `gemm_and_reduce(lhs_shard, rhs_shard)` runs this rank's K shard of the GEMM; the epilogue stores every finished bf16
    tile into the staging array of the rank that owns its m-block (`stage`, [world, M, N], peer-mapped) while the MMAs of
    the next tiles run -- the reduce-scatter half of the allreduce costs no time of its own.  A second kernel then sums,
    on every rank, the `world` staged copies of the rows it owns (fp32 in rank order, one rounding: bit-identical to
    TwoShotAllreduce) and stores them into all ranks' `buffer` -- the all-gather half.  Every rank makes the same calls in
    the same order."""

    def __init__(self, m: int, n: int, group: Optional[dist.ProcessGroup] = None, num_ctas: Optional[int] = None):
        assert n % 8 == 0 and m % 128 == 0
        self.group = group
        self.m, self.n = m, n
        world = dist.get_world_size(group)
        assert 2 <= world <= 8
        tensor_bytes = m * n * 2
        stage_offset = -(-(tensor_bytes + SIGNAL_BYTES) // 256) * 256
        self._arena = PeerSharedTensor((stage_offset + world * tensor_bytes,), torch.uint8, group)
        self.rank, self.world = self._arena.rank, self._arena.world
        self.buffer = self._arena.local[:tensor_bytes].view(torch.bfloat16).view(m, n)
        self.stage = self._arena.local[stage_offset:].view(torch.bfloat16).view(world, m, n)
        self._data = self._arena.ptr_array()
        self._signals = (ctypes.c_void_p * self.world)(*[p + tensor_bytes for p in self._arena.ptrs])
        self._stage = (ctypes.c_void_p * self.world)(*[p + stage_offset for p in self._arena.ptrs])
        sms = torch.cuda.get_device_properties(self.buffer.device).multi_processor_count
        self.num_ctas = num_ctas or sms
        self._clock = CollectiveClock()

    def gemm_and_reduce(self, lhs_shard, rhs_shard, block_n: int = 0) -> torch.Tensor:
        """Both halves on the current stream; returns `buffer` (valid once the stream has run the second kernel)."""
        self.scatter_gemm(lhs_shard, rhs_shard, block_n)
        return self.gather()

    def scatter_gemm(self, lhs_shard, rhs_shard, block_n: int = 0) -> None:
        """First half: this rank's K shard of the GEMM, every finished tile stored into its owner's staging array."""
        from ..jit_kernels.utils import get_col_major_tensor, get_num_sms
        lhs_q, lhs_scales = lhs_shard
        rhs_q, rhs_scales = rhs_shard
        m, k = lhs_q.shape
        assert (m, rhs_q.shape[0]) == (self.m, self.n) and rhs_q.shape[1] == k and k % 128 == 0
        assert lhs_q.dtype == torch.float8_e4m3fn and rhs_q.dtype == torch.float8_e4m3fn
        assert lhs_q.is_contiguous() and rhs_q.is_contiguous() and rhs_scales.is_contiguous()
        lhs_scales = get_col_major_tensor(lhs_scales)
        if lhs_scales.stride(1) != m:
            lhs_scales = lhs_scales.t().contiguous().t()
        stream = _lib.current_stream_ptr()
        _lib.call("yan_b200_gemm_fp8_fp8_bf16_nt_scatter", lhs_q.data_ptr(), lhs_scales.data_ptr(), rhs_q.data_ptr(),
                  rhs_scales.data_ptr(), self._stage, self.world, self.rank, m, self.n, k, self.n, stream, get_num_sms(),
                  block_n)

    def gather(self) -> torch.Tensor:
        """Second half: waits (on the device, bounded) until every rank's scatter has landed, sums the staged copies of
        the rows this rank owns and stores the sums into every rank's `buffer`."""
        stream = _lib.current_stream_ptr()
        epoch, counter_target = self._clock.next_launch(self.num_ctas)
        _lib.call("yan_b200_allreduce_bf16_gather_staged", ctypes.c_void_p(self.stage.data_ptr()), self._data, self._signals,
                  self.world, self.rank, self.m, self.n, epoch, counter_target, self.num_ctas, stream)
        return self.buffer

    def reset(self) -> None:
        """Collective; after a reported wait expiry: zero the signal blocks and restart the epochs."""
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        tensor_bytes = self.m * self.n * 2
        self._arena.local[tensor_bytes:tensor_bytes + SIGNAL_BYTES].zero_()
        self._clock.reset()
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    def close(self) -> None:
        self._arena.close()
