"""Measurement helpers with the reference's names and meaning (yan/utils.py:50-121)."""
from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist


class empty_suppress:
    def __enter__(self):
        return self

    def __exit__(self, *_):
        pass


class suppress_stdout_stderr:
    """Redirects the process-level stdout/stderr to /dev/null (yan/utils.py:14-46)."""

    def __enter__(self):
        self.null = [open(os.devnull, "w"), open(os.devnull, "w")]
        self.fds = [sys.stdout.fileno(), sys.stderr.fileno()]
        self.saved = [os.dup(fd) for fd in self.fds]
        self.py = (sys.stdout, sys.stderr)
        for f, fd in zip(self.null, self.fds):
            os.dup2(f.fileno(), fd)
        sys.stdout, sys.stderr = self.null
        return self

    def __exit__(self, *_):
        sys.stdout, sys.stderr = self.py
        for saved, fd in zip(self.saved, self.fds):
            os.dup2(saved, fd)
            os.close(saved)
        for f in self.null:
            f.close()


def l2_flush_bytes() -> int:
    """Bytes to overwrite so nothing of the previous launch stays in L2: twice the device's L2
    (the reference's fixed 128 MB, yan/utils.py:71-72, is smaller than B200's 126 MB L2 plus slack)."""
    l2 = torch.cuda.get_device_properties(torch.cuda.current_device()).L2_cache_size
    return 2 * max(int(l2), 64 << 20)


def bench_kineto(fn, kernel_names, num_tests: int = 30, suppress_kineto_output: bool = False,
                 trace_path: str = None, barrier_comm_profiling: bool = False, flush_l2: bool = False):
    """Average device time (seconds) of the kernels whose profiler row contains `kernel_names`
    (a string or a tuple of strings; each must match exactly one row).  Same procedure as
    yan/utils.py:50-107: one warm call, a torch.profiler pass over 2 x num_tests calls, optional L2
    flush before each call, optional large matmul + all-reduce to line ranks up, table parsing."""
    using_nsys = os.environ.get("YAN_NSYS_PROFILING", False)
    fn()
    flush = torch.empty(l2_flush_bytes() // 4, dtype=torch.int, device="cuda") if flush_l2 else None
    suppress = suppress_stdout_stderr if suppress_kineto_output and not using_nsys else empty_suppress
    with suppress():
        schedule = torch.profiler.schedule(wait=0, warmup=1, active=1, repeat=1) if not using_nsys else None
        profiler = (torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA], schedule=schedule)
                    if not using_nsys else empty_suppress())
        with profiler:
            for _ in range(2):
                if barrier_comm_profiling:
                    lhs = torch.randn((4096, 4096), dtype=torch.float, device="cuda")
                    rhs = torch.randn((4096, 4096), dtype=torch.float, device="cuda")
                    lhs @ rhs
                    dist.all_reduce(torch.ones(1, dtype=torch.float, device="cuda"))
                for _ in range(num_tests):
                    if flush is not None:
                        flush.zero_()
                    fn()
                if not using_nsys:
                    profiler.step()
    if using_nsys:
        return 1
    assert isinstance(kernel_names, (str, tuple))
    is_tupled = isinstance(kernel_names, tuple)
    lines = profiler.key_averages().table(sort_by="cuda_time_total", max_name_column_width=300).split("\n")
    names = (kernel_names,) if isinstance(kernel_names, str) else kernel_names
    for name in names:
        assert sum(name in line for line in lines) == 1, f"Errors of the kernel {name} in the profiling table: {lines}"
    if trace_path is not None:
        profiler.export_chrome_trace(trace_path)
    units = {"ms": 1e3, "us": 1e6}
    times = []
    for name in names:
        for line in lines:
            if name in line:
                t = line.split()[-2]
                for unit, scale in units.items():
                    if unit in t:
                        times.append(float(t.replace(unit, "")) / scale)
                        break
                break
    return tuple(times) if is_tupled else times[0]


def bench_events(fn, num_tests: int = 20, warmup: int = 3, flush_l2: bool = True) -> float:
    """Average device time (seconds) of `fn` measured with CUDA events on the current stream, one
    event pair per call so the optional L2 flush between calls is not counted."""
    flush = torch.empty(l2_flush_bytes() // 4, dtype=torch.int, device="cuda") if flush_l2 else None
    for _ in range(warmup):
        fn()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(num_tests)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(num_tests)]
    torch.cuda.synchronize()
    for s, e in zip(starts, ends):
        if flush is not None:
            flush.zero_()
        s.record()
        fn()
        e.record()
    torch.cuda.synchronize()
    return sum(s.elapsed_time(e) for s, e in zip(starts, ends)) / num_tests / 1e3


def calc_diff(x: torch.Tensor, y: torch.Tensor):
    """1 - 2<x,y>/(|x|^2 + |y|^2)  (yan/utils.py:109-113)."""
    x, y = x.double(), y.double()
    denominator = (x * x + y * y).sum()
    sim = 2 * (x * y).sum() / denominator
    return 1 - sim


def count_bytes(tensors) -> int:
    total = 0
    for t in tensors:
        if isinstance(t, tuple):
            total += count_bytes(t)
        else:
            total += t.numel() * t.element_size()
    return total
