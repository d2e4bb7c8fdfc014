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


def _line_up_ranks() -> None:
    """A large matmul and a one-element all-reduce: every rank reaches the profiled calls at about the same time."""
    x = torch.randn((4096, 4096), dtype=torch.float, device="cuda")
    torch.mm(x, x)
    dist.all_reduce(torch.ones(1, dtype=torch.float, device="cuda"))


def _kernel_seconds(events, wanted: str) -> float:
    """Mean device time of the one profiled kernel whose name contains `wanted`."""
    hits = [e for e in events if wanted in e.key]
    if len(hits) != 1:
        found = sorted(e.key for e in events)
        raise AssertionError(f"'{wanted}' must name exactly one profiled kernel, it matches {len(hits)} of {found}")
    event = hits[0]
    total_us = getattr(event, "device_time_total", None)
    if total_us is None:  # older profiler builds
        total_us = event.cuda_time_total
    return float(total_us) / max(int(event.count), 1) / 1e6


def bench_kineto(fn, kernel_names, num_tests: int = 30, suppress_kineto_output: bool = False,
                 trace_path: str = None, barrier_comm_profiling: bool = False, flush_l2: bool = False):
    """Mean device time in seconds of the kernel(s) named by `kernel_names` while `fn` runs under the profiler.

    Keeps the contract of the reference's helper (yan/utils.py:50-107): `kernel_names` is a substring or a tuple of
    substrings, each of which has to match exactly one profiled kernel; a tuple in gives a tuple out; `fn` is called
    once to warm up and then 2 x `num_tests` times, of which the second batch is the one recorded;
    `barrier_comm_profiling` lines the ranks up before each batch; `trace_path` writes a chrome trace;
    YAN_NSYS_PROFILING=1 runs the calls without the profiler (for an outer tool) and returns 1.
    Here the times come from the profiler's event records (name, total device time, count) and, with `flush_l2`,
    a buffer of twice the L2 size is overwritten before every call."""
    if not isinstance(kernel_names, (str, tuple)):
        raise AssertionError("kernel_names is a string or a tuple of strings")
    outer_tool = bool(os.environ.get("YAN_NSYS_PROFILING", False))
    scrub = torch.empty(l2_flush_bytes() // 4, dtype=torch.int, device="cuda") if flush_l2 else None

    def batch():
        if barrier_comm_profiling:
            _line_up_ranks()
        for _ in range(num_tests):
            if scrub is not None:
                scrub.zero_()
            fn()

    fn()
    if outer_tool:
        batch()
        batch()
        return 1
    quiet = suppress_stdout_stderr if suppress_kineto_output else empty_suppress
    with quiet():
        plan = torch.profiler.schedule(wait=0, warmup=1, active=1, repeat=1)
        with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA], schedule=plan) as prof:
            for _ in range(2):
                batch()
                prof.step()
    if trace_path is not None:
        prof.export_chrome_trace(trace_path)
    events = list(prof.key_averages())
    if isinstance(kernel_names, str):
        return _kernel_seconds(events, kernel_names)
    return tuple(_kernel_seconds(events, name) for name in kernel_names)


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


def perf_log(record: dict, path: str = None) -> None:
    """Appends one JSON line (shape, configuration, microseconds, TFLOP/s or GB/s, roofline fraction, error figures:
    whatever the caller measured) to the file named by `path` or by the YAN_PERF_LOG environment variable; a no-op
    when neither is set.  Tables of measurements are generated from this log rather than copied by hand."""
    import json
    import time
    path = path or os.environ.get("YAN_PERF_LOG")
    if not path:
        return
    line = dict(record)
    line.setdefault("unix_time", round(time.time(), 3))
    if torch.cuda.is_available():
        line.setdefault("device", torch.cuda.get_device_name())
    with open(path, "a") as f:
        f.write(json.dumps(line, sort_keys=True) + "\n")


def calc_diff(x: torch.Tensor, y: torch.Tensor):
    """Dissimilarity 1 - 2<x,y> / (|x|^2 + |y|^2) in float64: 0 for equal tensors, the reference's acceptance
    metric (`< 1e-3`, yan/utils.py:109-113)."""
    xd, yd = x.double().flatten(), y.double().flatten()
    return 1 - 2 * torch.dot(xd, yd) / (torch.dot(xd, xd) + torch.dot(yd, yd))


def count_bytes(tensors) -> int:
    """Bytes held by a (possibly nested) tuple of tensors."""
    return sum(count_bytes(t) if isinstance(t, tuple) else t.numel() * t.element_size() for t in tensors)
