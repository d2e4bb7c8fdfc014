#!/usr/bin/env python
"""Benchmark of the FP8 fine-grained-scaled GEMM path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Workload (every N): the column-parallel prefill GEMM  M=8192, N=28672, K=8192, e4m3 operands with
1x128 / 128x128 fp32 scales, bf16 output.  B is sharded along N over the ranks, A is replicated, no
collective is on the data path; total work is fixed, so scaling is "strong".
One step = quantize A (bf16 -> e4m3 + scales) followed by the GEMM over this rank's N/g columns.
Inputs are seeded synthetic tensors with the workload's shapes and distributions (A ~ N(0,1),
B ~ N(0, 0.02)); no dataset is involved.

Printed: ONE JSON line (rank 0).  `value` = 2*M*N*K / (max-over-ranks device time per step), inputs
resident in HBM.  `e2e` = the same step through the public API with A in pinned host memory and D read
back to the host every step.  `roofline` is for the GEMM kernel alone (CUDA events around each launch
on the launching stream).  `cpu_baseline` times the CPU oracle on a bounded slab on rank 0 at N=1.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

M, N, K = 8192, 28672, 8192
WORKLOAD = "C4 column-parallel prefill GEMM M=8192 N=28672 K=8192 (B sharded along N, A replicated)"
METRIC = "FP8 GEMM TFLOP/s (% FP8 peak); small-M HBM GB/s; 1/2/4/8-GPU scaling"
CPU_SLAB_ROWS = 256
# DRAM bytes of one GEMM launch of the benchmark's own 1-GPU workload (M=8192 N=28672 K=8192), from an ncu capture
# of three launches inside the quantize + GEMM sequence with the caches left as the sequence leaves them:
# dram__bytes_read 1023.5 MB + dram__bytes_write 482.6 MB.  The reads are A once (67 MB) plus B (235 MB, larger than
# the L2) once per band of 16 tile rows, four times in all; the writes are D (470 MB).  No capture exists for the
# narrower shards of the multi-GPU runs, so their line carries null.
GEMM_DRAM_TRAFFIC_BYTES_1GPU = 1023.5e6 + 482.6e6


def workload_config(world: int) -> dict:
    """The `config` object of the JSON line; both arms print the same one."""
    return {"workload": WORKLOAD, "M": M, "N": N, "K": K, "n_per_gpu": N // world,
            "step": "per_token_cast_to_fp8(A) + gemm_fp8_fp8_bf16_nt", "parallelism": f"n-split x{world}",
            "l2": "per-step operands (A8 67 MB + B8 shard + D shard) exceed the 126 MB L2"}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples the SM clock and the throttle reasons of one GPU while the timed region runs.  Reads only
    (NVML queries every few milliseconds from a thread); falls back to nvidia-smi when NVML is not importable."""
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, device_index: int, period_s: float = 0.003) -> None:
        self.device_index = device_index
        self.period_s = period_s
        self.samples = []
        self.reason_bits = 0
        self.max_mhz = None
        self.thread = None
        self.stop_flag = threading.Event()
        self.smi = None

    def _physical_index(self) -> int:
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if self.device_index < len(ids) and ids[self.device_index].isdigit():
                return int(ids[self.device_index])
        return self.device_index

    def start(self) -> None:
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
        except Exception:
            self.nvml = None
            self._start_smi()

    def _poll(self) -> None:
        nv = self.nvml
        while not self.stop_flag.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)
                bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                self.samples.append((time.perf_counter(), float(mhz)))
                self.reason_bits |= int(bits)
            except Exception:
                pass
            time.sleep(self.period_s)

    def _start_smi(self) -> None:
        query = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
                 "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
                 "clocks_event_reasons.sw_power_cap")
        try:
            self.smi = subprocess.Popen(["nvidia-smi", f"--query-gpu={query}", "--format=csv,noheader,nounits", "-i",
                                         str(self._physical_index()), "-lms", "50"], stdout=subprocess.PIPE,
                                        stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.smi = None

    def stop(self, t_begin: float = None, t_end: float = None) -> dict:
        """Median SM clock of the samples taken between t_begin and t_end (perf_counter stamps of the timed region)."""
        if self.thread is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            inside = [m for (t, m) in self.samples if (t_begin is None or t >= t_begin) and (t_end is None or t <= t_end)]
            use = inside if inside else [m for (_, m) in self.samples]
            reasons = sorted(k for k, bit in self.REASONS.items() if self.reason_bits & bit)
            return {"sm_mhz": statistics.median(use) if use else None, "sm_max_mhz": self.max_mhz,
                    "samples_in_timed_region": len(inside), "samples": len(self.samples), "reasons": reasons,
                    "source": "nvml"}
        if self.smi is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock source available"]}
        time.sleep(0.2)
        self.smi.terminate()
        try:
            out, _ = self.smi.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.smi.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            r = [c.strip() for c in line.split(",")]
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, flag in zip(names, r[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons), "source": "nvidia-smi"}


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        return rank, world, local, dist
    assert n_gpus == 1, "launch with torch.distributed.run for --gpus > 1"
    torch.cuda.set_device(0)
    return 0, 1, 0, None


def make_device_inputs(m, n_local, k, rank, outliers=False):
    """Seeded synthetic operands created on the device (identical A on every rank, rank-specific B shard)."""
    import yan_b200
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn(m, k, generator=g, device="cuda", dtype=torch.float32)
    if outliers:
        cols = torch.randperm(k, generator=torch.Generator().manual_seed(0))[: k // 100].cuda()
        a[:, cols] *= 20.0
    a = a.to(torch.bfloat16)
    gb = torch.Generator(device="cuda").manual_seed(1000 + rank)
    b = (torch.randn(n_local, k, generator=gb, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
    rhs = yan_b200.per_block_cast_to_fp8(b)
    del b
    return a, rhs


def time_graph_replays(fn, replays: int, launches_per_graph: int) -> float:
    """Seconds per launch of `fn` captured `launches_per_graph` times in a CUDA graph (removes CPU launch gaps)."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(launches_per_graph):
            fn(i)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / 1e3 / (replays * launches_per_graph)


def bench_decode(m: int, peaks) -> dict:
    """Small-M weight-streaming GEMM (N=7168, K=2048): HBM-bound.  Rotates over enough distinct operand
    sets that consecutive launches never find their B in L2 (total footprint >= 2 x L2)."""
    import yan_b200
    n, k = 7168, 2048
    l2 = torch.cuda.get_device_properties(0).L2_cache_size
    per_set = n * k + m * k + 2 * m * n
    sets = max(4, -(-2 * l2 // per_set))
    a, _ = make_device_inputs(m, 128, k, 0, outliers=True)
    lhs = yan_b200.per_token_cast_to_fp8(a)
    rhs_list, outs = [], []
    for i in range(sets):
        _, rhs = make_device_inputs(m, n, k, 100 + i)
        rhs_list.append(rhs)
        outs.append(torch.empty(m, n, dtype=torch.bfloat16, device="cuda"))

    def fn(i=0):
        yan_b200.gemm_fp8_fp8_bf16_nt(lhs, rhs_list[i % sets], outs[i % sets])

    t_serial = time_graph_replays(fn, replays=20, launches_per_graph=sets)
    # Back-to-back decode GEMMs with programmatic dependent launch: the weights of launch i+1 start streaming while
    # launch i drains (weights are never produced by the preceding kernel in a decode loop).
    yan_b200.set_programmatic_dependent_launch(True)
    try:
        t = time_graph_replays(fn, replays=20, launches_per_graph=sets)
    finally:
        yan_b200.set_programmatic_dependent_launch(False)
    # bf16 in -> bf16 out: the quantizer and the GEMM of one fp8_linear call (the GEMM's weight loads overlap the quantizer)
    ws = torch.empty(yan_b200.fp8_linear_workspace_bytes(m, k), dtype=torch.uint8, device="cuda")

    def fn_linear(i=0):
        yan_b200.fp8_linear(a, rhs_list[i % sets], outs[i % sets], workspace=ws)

    t_linear = time_graph_replays(fn_linear, replays=20, launches_per_graph=sets)
    # the same chain with the quantizer launched programmatically too (its launch overlaps the previous GEMM's tail)
    yan_b200.set_programmatic_dependent_launch(True)
    try:
        t_linear_pdl = time_graph_replays(fn_linear, replays=20, launches_per_graph=sets)
    finally:
        yan_b200.set_programmatic_dependent_launch(False)
    algo_bytes = m * k + 4 * m * (k // 128) + n * k + 4 * (n // 128) * (k // 128) + 2 * m * n
    gbs = algo_bytes / t / 1e9
    return {"workload": f"C2 decode M={m} N={n} K={k}", "us": t * 1e6, "GB/s": gbs, "algorithmic_bytes": algo_bytes,
            "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], "frac_of_nominal_8TBs": gbs / 8000.0,
            "fp8_linear_us (quantize + GEMM, bf16 in)": t_linear * 1e6,
            "fp8_linear_us, quantizer launched programmatically too": t_linear_pdl * 1e6,
            "us_without_programmatic_launch": t_serial * 1e6, "GB/s_without_programmatic_launch": algo_bytes / t_serial / 1e9,
            "timing": f"CUDA graph of {sets} launches over {sets} distinct B/D sets (>= 2 x L2), 20 replays, "
                      "programmatic dependent launch between consecutive GEMMs"}


def bench_dense(name: str, m: int, n: int, k: int, peaks, iters: int = 10) -> dict:
    import yan_b200
    from yan_b200.utils import bench_events
    a, rhs = make_device_inputs(m, n, k, 0)
    lhs = yan_b200.per_token_cast_to_fp8(a)
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    t = bench_events(lambda: yan_b200.gemm_fp8_fp8_bf16_nt(lhs, rhs, out), num_tests=iters, flush_l2=True)
    tq = bench_events(lambda: yan_b200.per_token_cast_to_fp8(a, out=lhs), num_tests=iters, flush_l2=True)
    tf = 2.0 * m * n * k / t / 1e12
    qbytes = 3 * m * k + 4 * m * (k // 128)
    return {"workload": f"{name} M={m} N={n} K={k}", "gemm_us": t * 1e6, "TFLOP/s": tf,
            "frac_of_2x_measured_bf16_burst": tf / (2 * peaks["bf16_tflops"]), "frac_of_nominal_4.5PF": tf / 4500.0,
            "quant_us": tq * 1e6, "quant_GB/s": qbytes / tq / 1e9,
            "quant_frac_of_measured_hbm": qbytes / tq / 1e9 / peaks["hbm_gbs"]}


def bench_fused_epilogue(m: int, n: int, k: int, iters: int = 10, peaks=None) -> dict:
    """Layer i's GEMM followed by layer i+1's activation quantizer: two kernels through a bf16 tensor against the GEMM
    whose epilogue writes e4m3 + scales directly (the outputs are bit-identical; tests/test_gemm_e4m3_out_gpu.py)."""
    import yan_b200
    from yan_b200.utils import bench_events
    a, rhs = make_device_inputs(m, n, k, 0)
    lhs = yan_b200.per_token_cast_to_fp8(a)
    d = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    q = yan_b200.per_token_cast_to_fp8(d)
    fused_out = yan_b200.gemm_fp8_fp8_e4m3_nt(lhs, rhs)

    def two_kernels():
        yan_b200.gemm_fp8_fp8_bf16_nt(lhs, rhs, d)
        yan_b200.per_token_cast_to_fp8(d, out=q)

    t2 = bench_events(two_kernels, num_tests=iters, flush_l2=True)
    t1 = bench_events(lambda: yan_b200.gemm_fp8_fp8_e4m3_nt(lhs, rhs, out=fused_out), num_tests=iters, flush_l2=True)
    return {"workload": f"GEMM + next layer's quantizer M={m} N={n} K={k}", "gemm_then_quantizer_us": t2 * 1e6,
            "fused_epilogue_us": t1 * 1e6, "speedup": t2 / t1,
            "fused_TFLOP/s": 2.0 * m * n * k / t1 / 1e12,
            "fused_frac_of_2x_measured_bf16_burst": (2.0 * m * n * k / t1 / 1e12 / (2 * peaks["bf16_tflops"])) if peaks else None,
            "hbm_bytes_saved": 2 * m * n + 2 * m * n}


def bench_grouped(peaks, groups: int = 4, rows_per_group: int = 2048, n: int = 7168, k: int = 2048, iters: int = 10) -> dict:
    """Grouped GEMM, contiguous layout (MoE experts): `groups` weight matrices, each applied to its own run of rows."""
    import yan_b200
    from yan_b200.utils import bench_events
    m = groups * rows_per_group
    g = torch.Generator(device="cuda").manual_seed(11)
    a = torch.randn(m, k, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    lhs = yan_b200.per_token_cast_to_fp8(a)
    qs, ss = [], []
    for i in range(groups):
        w = (torch.randn(n, k, generator=g, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
        q, sc = yan_b200.per_block_cast_to_fp8(w)
        qs.append(q)
        ss.append(sc)
    rhs = (torch.stack(qs).contiguous(), torch.stack(ss).contiguous())
    m_indices = torch.arange(groups, device="cuda", dtype=torch.int32).repeat_interleave(rows_per_group).contiguous()
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    t = bench_events(lambda: yan_b200.m_grouped_gemm_fp8_fp8_bf16_nt_contiguous(lhs, rhs, out, m_indices),
                     num_tests=iters, flush_l2=True)
    tf = 2.0 * m * n * k / t / 1e12
    return {"workload": f"grouped GEMM (contiguous) {groups} groups x {rows_per_group} rows, N={n} K={k}", "gemm_us": t * 1e6,
            "TFLOP/s": tf, "frac_of_2x_measured_bf16_burst": tf / (2 * peaks["bf16_tflops"]),
            "frac_of_nominal_4.5PF": tf / 4500.0}


def bench_sustained(step, flops_per_step: float, burst_ms: float, device_index: int, seconds: float = 2.0) -> dict:
    """The same step back to back for about `seconds` (the power cap, not the burst clock, sets this figure), with the
    median SM clock of the NVML samples taken inside the window."""
    steps = max(20, int(seconds / (burst_ms / 1e3)))
    sampler = ClockSampler(device_index, period_s=0.01)
    torch.cuda.synchronize()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin = time.perf_counter()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop(t_begin, time.perf_counter())
    ms = e0.elapsed_time(e1) / steps
    return {"workload": f"C4 step (quantize + GEMM) back to back for {steps} steps (~{seconds:.0f} s)", "ms_per_step": ms,
            "TFLOP/s": flops_per_step / (ms / 1e3) / 1e12, "sm_mhz_median": clocks.get("sm_mhz"),
            "clock_samples": clocks.get("samples_in_timed_region"), "reasons": clocks.get("reasons")}


def bench_reference_blackwell_gemm(peaks, m: int = 8192, n: int = 8192, k: int = 8192) -> dict:
    """Same-GPU yardstick: the reference's own Blackwell program (comm/gemm.cu: CUTLASS fp16 GEMM, its own timing loop)
    run as a separate process on M=N=K=8192, beside this package's FP8 GEMM on the same M, N, K.  One GPU only."""
    import yan_b200
    from yan_b200.utils import bench_events
    a, rhs = make_device_inputs(m, n, k, 0)
    lhs = yan_b200.per_token_cast_to_fp8(a)
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    t = bench_events(lambda: yan_b200.gemm_fp8_fp8_bf16_nt(lhs, rhs, out), num_tests=10, flush_l2=True)
    ours = 2.0 * m * n * k / t / 1e12
    del a, rhs, lhs, out
    torch.cuda.empty_cache()
    res = {"workload": f"same-GPU yardstick M={m} N={n} K={k}", "fp8_gemm_TFLOP/s (this package)": ours,
           "fp8_gemm_us": t * 1e6}
    binary = os.path.join(ROOT, "oracle", "_ref", "ref_gemm_sm100")
    if not os.path.exists(binary):
        res["reference_fp16_gemm"] = "unavailable: oracle/_ref/ref_gemm_sm100 was not built (needs the reference tree and CUTLASS headers)"
        return res
    try:
        r = subprocess.run([binary, f"--m={m}", f"--n={n}", f"--k={k}", "--iterations=10"], capture_output=True, text=True,
                           timeout=180)
        gflops = [float(line.split(":")[1]) for line in r.stdout.splitlines() if line.strip().startswith("GFLOPS")]
        if r.returncode != 0 or not gflops:
            res["reference_fp16_gemm"] = f"unavailable: exit code {r.returncode}: {(r.stdout + r.stderr)[-200:]}"
            return res
        res["reference_fp16_gemm_TFLOP/s (comm/gemm.cu, CUTLASS 256x128x64, cluster 2x2)"] = gflops[0] / 1e3
        res["fp8_over_reference_fp16"] = ours / (gflops[0] / 1e3)
    except Exception as e:
        res["reference_fp16_gemm"] = f"unavailable: {type(e).__name__}: {e}"[:200]
    return res


def _time_k_split(step, dist, steps: int, m: int, n: int, k: int, flops: bool = True) -> dict:
    import yan_b200
    for _ in range(3):
        step()
    dist.barrier()
    torch.cuda.synchronize()
    # a wait between ranks that ran out during the warm-up (on any rank): the form is not timed -- every further launch
    # would sit out its bound as well
    expired = torch.tensor([float(yan_b200.read_device_status(reset=True) != 0)], device="cuda", dtype=torch.float64)
    dist.all_reduce(expired, op=dist.ReduceOp.MAX)
    if expired.item() != 0:
        return {"not_timed": "a bounded wait between the ranks ran out during the warm-up"}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / steps], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if not flops:
        return {"ms": t.item()}
    return {"ms_per_step": t.item(), "TFLOP/s": 2.0 * m * n * k / (t.item() / 1e3) / 1e12}


def bench_k_split(rank: int, world: int, dist, steps: int = 10, parity: dict = None) -> dict:
    """Row-parallel GEMM + allreduce (M=4096, N=8192, K=28672 split along K over the ranks): per step each rank
    quantizes its K shard of A, computes a full-size bf16 partial D in row chunks and sums the partials with an NCCL
    allreduce that overlaps the next chunk's GEMM.  Time = max over ranks, device events."""
    import yan_b200
    from yan_b200.comm import gemm_allreduce as ga
    m, n, k = 4096, 8192, 28672
    ks = k // world
    g = torch.Generator(device="cuda").manual_seed(7)
    a = torch.randn(m, k, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)[:, rank * ks:(rank + 1) * ks].contiguous()
    gb = torch.Generator(device="cuda").manual_seed(70 + rank)
    b = (torch.randn(n, ks, generator=gb, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
    rhs = yan_b200.per_block_cast_to_fp8(b)
    del b
    lhs = yan_b200.per_token_cast_to_fp8(a)
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    comm_stream = torch.cuda.Stream()
    results = {}

    def checked(prefix: str) -> bool:
        """False when the parity pass before the timed legs saw this form fail: it is then neither run nor timed."""
        if not parity:
            return True
        return all(v.get("pass", True) for key, v in parity.items() if key.startswith(prefix) and isinstance(v, dict))
    for label, chunks in (("NCCL, single allreduce", 1), ("NCCL, 4 row chunks overlapped", 4)):
        def step():
            yan_b200.per_token_cast_to_fp8(a, out=lhs)
            ga.gemm_k_split_allreduce(lhs, rhs, out, partial_dtype=torch.bfloat16, num_chunks=chunks, comm_stream=comm_stream)
        results[label] = _time_k_split(step, dist, steps, m, n, k)
    # The same step with the partials summed by this package's two-shot kernel over peer-mapped memory (the GEMM writes
    # straight into the shared buffer), and the two collectives alone on the same 64 MiB tensor.
    try:
        from yan_b200.comm import TwoShotAllreduce
        if not checked("k_split_two_shot") or not checked("two_shot_reduce_rows"):
            raise RuntimeError("the two-shot kernel failed the parity pass")
        comm = TwoShotAllreduce(m, n)
        variants = (("", 1, 24), (", 2 row chunks overlapped (24 SMs to the collective)", 2, 24),
                    (", 2 row chunks overlapped (64 SMs to the collective)", 2, 64),
                    (", 4 row chunks overlapped (64 SMs to the collective)", 4, 64))
        for suffix, chunks, comm_sms in variants:
            def step():
                yan_b200.per_token_cast_to_fp8(a, out=lhs)
                ga.gemm_k_split_two_shot(lhs, rhs, comm, num_chunks=chunks, comm_sms=comm_sms, comm_stream=comm_stream)
            results["two-shot peer allreduce" + suffix] = _time_k_split(step, dist, steps, m, n, k)
        try:
            if not checked("k_split_in_switch") or not checked("in_switch_reduce_rows"):
                raise RuntimeError("the in-switch kernel failed the parity pass")
            comm_sw = TwoShotAllreduce(m, n, in_switch=True)
            for suffix, chunks, comm_sms in variants:
                def step():
                    yan_b200.per_token_cast_to_fp8(a, out=lhs)
                    ga.gemm_k_split_two_shot(lhs, rhs, comm_sw, num_chunks=chunks, comm_sms=comm_sms, comm_stream=comm_stream)
                results["in-switch peer allreduce" + suffix] = _time_k_split(step, dist, steps, m, n, k)
            results["allreduce alone, in-switch"] = _time_k_split(lambda: comm_sw.reduce_rows(), dist, steps, m, n, k, flops=False)
            comm_sw.close()
        except Exception as e:
            results["in-switch peer allreduce"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
        try:
            from yan_b200.comm import TileFusedAllreduce
            if not checked("k_split_tile_fused"):
                raise RuntimeError("the tile-fused form failed the parity pass")
            fused = TileFusedAllreduce(m, n)

            def step():
                yan_b200.per_token_cast_to_fp8(a, out=lhs)
                fused.gemm_and_reduce(lhs, rhs)
            results["tile-fused: reduce-scatter in the GEMM epilogue + all-gather kernel"] = _time_k_split(step, dist, steps, m, n, k)
            # its two halves alone (the scatter writes peers' staging arrays that nobody reads meanwhile; the gather sums
            # whatever the last scatter left there)
            results["tile-fused, first half alone: GEMM with the scatter epilogue"] = _time_k_split(
                lambda: fused.scatter_gemm(lhs, rhs), dist, steps, m, n, k, flops=False)
            results["tile-fused, second half alone: gather kernel"] = _time_k_split(
                lambda: fused.gather(), dist, steps, m, n, k, flops=False)

            def plain_gemm():
                yan_b200.gemm_fp8_fp8_bf16_nt(lhs, rhs, out)
            results["this rank's K-shard GEMM alone, local output"] = _time_k_split(plain_gemm, dist, steps, m, n, k, flops=False)
            fused.close()
        except Exception as e:
            results["tile-fused"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
        results["allreduce alone, NCCL"] = _time_k_split(lambda: dist.all_reduce(out), dist, steps, m, n, k, flops=False)
        results["allreduce alone, two-shot"] = _time_k_split(lambda: comm.reduce_rows(), dist, steps, m, n, k, flops=False)
        results["device_status"] = yan_b200.read_device_status()
        comm.close()
    except Exception as e:  # peer mapping unavailable (e.g. ranks without peer access): the NCCL numbers stand alone
        results["two-shot peer allreduce"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    return {"workload": f"C5 row-parallel GEMM + allreduce M={m} N={n} K={k} (K/{world} per GPU, bf16 partials)",
            "allreduce_bytes": 2 * m * n, **results}


def multi_gpu_parity(rank: int, world: int, dist) -> dict:
    """Every sharded form once on a small checked case (M=512, N=1024, K=2048 per rank), before anything is timed:
    the same code paths the timed legs use, compared with the CPU oracle's unsplit / K-split results.  Each entry
    holds the worst figures over the ranks.  (The oracle is the checker here; nothing timed touches it.)"""
    import yan_b200
    from oracle import ref
    from yan_b200.comm import gemm_allreduce as ga
    m, n, k = 512, 1024, 2048 * world
    threads_before = torch.get_num_threads()
    torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))  # the launcher pins its ranks to one thread
    a, b = ref.make_inputs(m, n, k, seed=3)
    lhs, rhs = ref.per_token_cast_to_fp8(a), ref.per_block_cast_to_fp8(b)
    d_ref = ref.ref_gemm(lhs, rhs)
    d_split = ref.ref_gemm_k_split(lhs, rhs, world)
    torch.set_num_threads(threads_before)
    out = {}

    def record(name, got, want, tol, extra=None):
        got = got.float().cpu()
        fro = float(ref.rel_frobenius(got, want))
        mx = float((got - want.float()).abs().max())
        t = torch.tensor([fro, mx], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        entry = {"rel_frobenius": t[0].item(), "max_abs": t[1].item(), "tolerance": tol, "pass": bool(t[0].item() <= tol)}
        if extra:
            flags = torch.tensor([1.0 if v else 0.0 for v in extra.values()], device="cuda", dtype=torch.float64)
            dist.all_reduce(flags, op=dist.ReduceOp.MIN)
            for key, v in zip(extra.keys(), flags.tolist()):
                entry[key] = bool(v)
                entry["pass"] = entry["pass"] and bool(v)
        out[name] = entry

    # forms that ADD in bf16 (NCCL's bf16 ring, the switch's bf16 reduction) round after each of the world-1 additions
    # on top of the world rounded partials, so their distance from the oracle grows with the number of ranks
    tol_bf16_sum = 3e-3 * math.sqrt(world)
    lhs_dev = (lhs[0].contiguous().cuda(), lhs[1].t().contiguous().cuda().t())
    # N-split: every rank writes its own column slice of a zeroed full buffer; summing the buffers assembles D
    full = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
    rhs_n = tuple(t.contiguous().cuda() for t in ga.shard_n(rhs, rank, world))
    ga.gemm_n_split(lhs_dev, rhs_n, full, rank, world)
    dist.all_reduce(full)
    record("n_split", full, d_ref, 1e-3)
    # K-split over NCCL: bf16 partials (the specified arithmetic) and fp32 partials
    ks = k // world
    lhs_k = yan_b200.per_token_cast_to_fp8(a[:, rank * ks:(rank + 1) * ks].contiguous().cuda())
    rhs_k = tuple(t.contiguous().cuda() for t in ga.shard_k(rhs, rank, world))
    res = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ga.gemm_k_split_allreduce(lhs_k, rhs_k, res, partial_dtype=torch.bfloat16, num_chunks=2)
    torch.cuda.synchronize()
    record("k_split_nccl_bf16_partials", res, d_split, tol_bf16_sum)
    ga.gemm_k_split_allreduce(lhs_k, rhs_k, res, partial_dtype=torch.float32, num_chunks=2)
    torch.cuda.synchronize()
    record("k_split_nccl_fp32_partials", res, d_ref, 1e-3)
    # the peer-memory kernels: the fp32 sum of the ranks' bf16 partials in rank order, rounded once, is what the
    # plain load/store kernel must reproduce bit for bit
    partial = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    yan_b200.gemm_fp8_fp8_bf16_nt(lhs_k, rhs_k, partial)
    gathered = [torch.empty_like(partial) for _ in range(world)]
    dist.all_gather(gathered, partial)
    acc = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    for g in gathered:
        acc += g.float()
    rank_order_sum = acc.to(torch.bfloat16)
    try:
        from yan_b200.comm import TwoShotAllreduce
        for name, in_switch, tol in (("two_shot", False, 2e-3), ("in_switch", True, tol_bf16_sum)):
            try:
                comm = TwoShotAllreduce(m, n, in_switch=in_switch)
            except Exception as e:
                out["k_split_" + name] = {"unavailable": f"{type(e).__name__}: {e}"[:160]}
                continue
            for chunks in (1, 2):
                got = ga.gemm_k_split_two_shot(lhs_k, rhs_k, comm, num_chunks=chunks)
                torch.cuda.synchronize()
                extra = None if in_switch else {"bit_exact_vs_fp32_rank_order_sum": bool(torch.equal(got, rank_order_sum))}
                record(f"k_split_{name}_{chunks}_chunk" + ("s" if chunks > 1 else ""), got, d_split, tol, extra)
            # a row range alone: rows outside keep this rank's own partial
            comm.buffer.copy_(partial)
            comm.reduce_rows(128, 384, num_ctas=7)
            torch.cuda.synchronize()
            inside = comm.buffer[128:384]
            untouched = bool(torch.equal(comm.buffer[:128], partial[:128]) and torch.equal(comm.buffer[384:], partial[384:]))
            extra = {"rows_outside_untouched": untouched}
            if not in_switch:
                extra["bit_exact_vs_fp32_rank_order_sum"] = bool(torch.equal(inside, rank_order_sum[128:384]))
            record(f"{name}_reduce_rows_128_384", inside, d_split[128:384], tol, extra)
            comm.close()
    except Exception as e:
        out["peer_memory"] = {"unavailable": f"{type(e).__name__}: {e}"[:160]}
    # the tile-fused form: reduce-scatter inside the GEMM epilogue, all-gather kernel behind it; same arithmetic as two-shot
    try:
        from yan_b200.comm import TileFusedAllreduce
        fused = TileFusedAllreduce(m, n)
        for attempt in range(2):  # twice: the staging arrays and epochs are reused
            got = fused.gemm_and_reduce(lhs_k, rhs_k)
            torch.cuda.synchronize()
            record(f"k_split_tile_fused_call_{attempt + 1}", got, d_split, 2e-3,
                   {"bit_exact_vs_fp32_rank_order_sum": bool(torch.equal(got, rank_order_sum))})
        fused.close()
    except Exception as e:
        out["k_split_tile_fused"] = {"unavailable": f"{type(e).__name__}: {e}"[:160]}
    # the host front end with sharded input: the gathered operand must equal the quantizer's output on all of A
    pipe = yan_b200.HostFp8Linear(rhs_n, m, depth=1, shard_input=True)
    a_pinned = a.contiguous().pin_memory()
    d_pinned = torch.empty(m, n // world, dtype=torch.bfloat16).pin_memory()
    pipe.submit(a_pinned, d_pinned)
    pipe.wait()
    q_all, s_all = yan_b200.per_token_cast_to_fp8(a.cuda())
    same = bool(torch.equal(pipe.lhs[0][0].view(torch.uint8), q_all.view(torch.uint8)) and torch.equal(pipe.lhs[0][1], s_all))
    record("host_front_end_sharded_input", d_pinned, d_ref[:, rank * (n // world):(rank + 1) * (n // world)], 1e-3,
           {"gathered_operand_bit_exact_vs_local_quantizer": same})
    del pipe
    status = torch.tensor([float(yan_b200.read_device_status())], device="cuda", dtype=torch.float64)
    dist.all_reduce(status, op=dist.ReduceOp.MAX)
    out["device_status"] = int(status.item())
    out["all_pass"] = all(v.get("pass", True) for v in out.values() if isinstance(v, dict)) and out["device_status"] == 0
    out["case"] = f"M={m} N={n} K={k} ({world} ranks; oracle: CPU dequantize-and-matmul, K-split restated for the split forms)"
    return out


def cpu_reference_step(a_slab, rhs_cpu):
    """The CPU dequantize-and-matmul path on one slab: quantize A, dequantize both, fp32 matmul, bf16."""
    from oracle import ref
    lhs = ref.per_token_cast_to_fp8(a_slab)
    return ref.ref_gemm(lhs, rhs_cpu)


def make_cpu_inputs():
    from oracle import ref
    g = torch.Generator().manual_seed(0)
    a = torch.randn(CPU_SLAB_ROWS, K, generator=g).to(torch.bfloat16)
    b = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    rhs = ref.per_block_cast_to_fp8(b)
    return a, rhs


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torch.distributed.run exports OMP_NUM_THREADS=1 to its ranks: use the box's cores at every N all the same
    torch.set_num_threads(args.cpu_threads if args.cpu_threads > 0 else (os.cpu_count() or 1))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    a, rhs = make_cpu_inputs()
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_reference_step(a, rhs)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_reference_step(a, rhs)
    dt = (time.perf_counter() - t0) / args.steps
    flops = 2.0 * CPU_SLAB_ROWS * N * K
    value = flops / dt / 1e12
    cores = torch.get_num_threads()
    sample = (f"{CPU_SLAB_ROWS}-row slab of A against the full B (N={N}, K={K}) per step: quantize A, dequantize A and B "
              f"to fp32, torch.matmul fp32, round to bf16; flops counted for the slab only")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32 (dequantized e4m3)", "data": "synthetic",
            "config": workload_config(world),
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def run_ours(args) -> None:
    # Libraries may write to stdout (NCCL prints its version there): keep the real stdout for the one JSON line and send
    # everything else written to descriptor 1 to stderr.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    import yan_b200
    peaks = load_peaks()
    rank, world, local, dist = dist_setup(args.gpus)
    assert N % (world * 256) == 0
    n_local = N // world
    dev_name = torch.cuda.get_device_name()

    a, rhs = make_device_inputs(M, n_local, K, rank)
    lhs = (torch.empty(M, K, dtype=torch.float8_e4m3fn, device="cuda"),
           torch.empty(K // 128, M, dtype=torch.float32, device="cuda").t())
    out = torch.empty(M, n_local, dtype=torch.bfloat16, device="cuda")

    def step():
        yan_b200.per_token_cast_to_fp8(a, out=lhs)
        yan_b200.gemm_fp8_fp8_bf16_nt(lhs, rhs, out)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    if world > 1:
        # the ranks of this benchmark are lined up by barriers before every collective leg, so a wait between ranks that
        # takes seconds is a fault, not drift: 3 s instead of the library's 10 s keeps a faulty form from eating the run
        from yan_b200 import _lib as _yan_lib
        _yan_lib.lib().yan_b200_set_collective_timeout_ns(3_000_000_000)
    parity = multi_gpu_parity(rank, world, dist) if world > 1 else None

    for _ in range(args.warmup):
        step()
    barrier()

    # ---- timed region: exactly K steps; per-kernel events on the launching (current) stream ----
    probe = torch.zeros(16, dtype=torch.int64, device="cuda")
    yan_b200.set_clock_probe(probe)  # CTA 0 of every GEMM launch stamps clock64 / globaltimer at start and end
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.05)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    barrier()
    t_start = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    wall_begin = time.perf_counter()
    t_start.record()
    for i in range(args.steps):
        ev[i][0].record()
        yan_b200.per_token_cast_to_fp8(a, out=lhs)
        ev[i][1].record()
        yan_b200.gemm_fp8_fp8_bf16_nt(lhs, rhs, out)
        ev[i][2].record()
    t_end.record()
    barrier()
    clocks = sampler.stop(wall_begin, time.perf_counter())
    yan_b200.set_clock_probe(None)
    # the clock the last timed GEMM launch really ran at (a launch of a millisecond or two falls between NVML samples)
    clocks["gemm_kernel_sm_mhz"] = yan_b200.effective_sm_clock_mhz(probe)
    clocks["gemm_kernel_sm_mhz_source"] = "clock64 delta / globaltimer delta of CTA 0, last timed launch"
    elapsed_ms = t_start.elapsed_time(t_end)
    quant_ms = sum(e[0].elapsed_time(e[1]) for e in ev) / args.steps
    gemm_ms = sum(e[1].elapsed_time(e[2]) for e in ev) / args.steps
    assert yan_b200.read_device_status() == 0, "a device-side wait ran out during the benchmark"
    if dist is not None:
        t = torch.tensor([elapsed_ms, gemm_ms, quant_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, gemm_ms, quant_ms = t.tolist()
    ms_per_step = elapsed_ms / args.steps
    flops_total = 2.0 * M * N * K
    value = flops_total / (ms_per_step / 1e3) / 1e12

    # ---- end to end: A from pinned host memory, D back to pinned host memory, every step, through the package's
    # host front end (three streams, two rotating device slots: copies of one step overlap kernels of the next) ----
    a_host = a.cpu().pin_memory()
    out_hosts = [torch.empty(M, n_local, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    # several ranks: each pulls only its share of A's rows over its host link and the ranks all-gather the quantized rows
    pipe = yan_b200.HostFp8Linear(rhs, M, depth=2, shard_input=(world > 1))
    e2e_steps = max(4, min(args.steps, 10))
    for i in range(2):
        pipe.submit(a_host, out_hosts[i % 2])
    pipe.wait()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(e2e_steps):
        pipe.submit(a_host, out_hosts[i % 2])
    torch.cuda.current_stream().wait_stream(pipe.copy_out)
    e1.record()
    pipe.wait()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    # unpipelined latency of one step (copy in, kernels, copy out, strictly in sequence) for reference
    a_dev = torch.empty_like(a)
    torch.cuda.synchronize()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    serial = yan_b200.HostFp8Linear(rhs, M, depth=1, shard_input=(world > 1))
    serial.submit(a_host, out_hosts[0])
    serial.wait()
    barrier()
    s0.record()
    serial.submit(a_host, out_hosts[0])
    torch.cuda.current_stream().wait_stream(serial.copy_out)
    s1.record()
    serial.wait()
    e2e_serial_ms = s0.elapsed_time(s1)
    h2d_bytes = pipe.h2d_bytes_per_call()
    del serial
    if dist is not None:
        t = torch.tensor([e2e_ms, e2e_serial_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms, e2e_serial_ms = t.tolist()
    e2e_value = flops_total / (e2e_ms / 1e3) / 1e12
    out_host = out_hosts[0]

    # ---- roofline of the dominant kernel (the GEMM) ----
    gemm_flops = 2.0 * M * n_local * K
    achieved = gemm_flops / (gemm_ms / 1e3) / 1e12
    fp8_peak = 2.0 * peaks["bf16_tflops"]
    algo_bytes = M * K + 4 * M * (K // 128) + n_local * K + 4 * (n_local // 128) * (K // 128) + 2 * M * n_local
    traffic = GEMM_DRAM_TRAFFIC_BYTES_1GPU if world == 1 else None
    roofline = {"kernel": "fp8_gemm_kernel<BLOCK_N=256>", "bound": "tensor", "achieved": achieved, "peak": fp8_peak,
                "unit": "TFLOP/s", "frac": achieved / fp8_peak, "traffic": traffic, "algorithmic_bytes_per_launch": algo_bytes,
                "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of this workload's launch, caches as the "
                                  "step leaves them" if world == 1 else "no capture of this shard",
                "peak_source": f"2 x {peaks['source']} bf16 burst {peaks['bf16_tflops']} TFLOP/s "
                               "(e4m3 tensor rate is twice bf16; no FP8 figure is measured on this pool)",
                "frac_of_2x_sustained_bf16": achieved / (2.0 * peaks["bf16_tflops_sustained"]),
                "frac_of_nominal_4.5PF": achieved / 4500.0,
                "algorithmic_flops_per_launch": gemm_flops, "avg_launch_ms": gemm_ms,
                "quant_kernel": {"bound": "hbm", "achieved": (3.0 * M * K + 4 * M * (K // 128)) / (quant_ms / 1e3) / 1e9,
                                 "peak": peaks["hbm_gbs"], "unit": "GB/s", "avg_launch_ms": quant_ms}}
    roofline["quant_kernel"]["frac"] = roofline["quant_kernel"]["achieved"] / peaks["hbm_gbs"]

    line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "e4m3 (fp32 accumulate, bf16 out)", "data": "synthetic",
            "config": workload_config(world), "device": dev_name,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d_bytes * world, "d2h_bytes_per_step": out_host.numel() * 2 * world,
                    "h2d_bytes_per_step_per_gpu": h2d_bytes, "d2h_bytes_per_step_per_gpu": out_host.numel() * 2,
                    "single_step_latency_ms": e2e_serial_ms,
                    "note": "yan_b200.HostFp8Linear: weights resident on the device; every step copies A in from pinned "
                            "host memory and D out to pinned host memory; copies of one step overlap the kernels of the "
                            "next (2 device slots, 3 streams)" +
                            ("; every rank copies and quantizes M/g rows of A and the ranks all-gather the e4m3 codes and "
                             "scales over NVLink (bit-identical to quantizing all of A on every rank)" if world > 1 else "")},
            "gpu_launches": 2 * args.steps, "clocks": clocks, "roofline": roofline}
    if parity is not None:
        line["parity"] = parity

    sustained = None
    if world == 1 and not args.no_extras:
        sustained = bench_sustained(step, flops_total, ms_per_step, local)
        sustained["frac_of_2x_sustained_bf16"] = sustained["TFLOP/s"] / (2.0 * peaks["bf16_tflops_sustained"])
    del a_host, out_host, out_hosts, pipe, a_dev, out, lhs, rhs, a
    torch.cuda.empty_cache()

    if world > 1 and not args.no_extras:
        k_split = bench_k_split(rank, world, dist, parity=parity)
        if rank == 0:
            line["other_workloads"] = [k_split]
    if rank == 0 and world == 1 and not args.no_extras:
        extras = []

        def leg(fn, *fn_args, **fn_kwargs):
            # every side measurement is a short burst; half a second of idle in front of it keeps the power-cap state the
            # previous leg left (a GPU that has just run tens of milliseconds of dense GEMMs clocks lower for a while)
            # out of its figure
            torch.cuda.synchronize()
            time.sleep(0.5)
            extras.append(fn(*fn_args, **fn_kwargs))
        for m_small in (16, 64):
            leg(bench_decode, m_small, peaks)
        leg(bench_dense, "C3 mid-size projection", 4096, 7168, 18432, peaks)
        leg(bench_dense, "C1 CPU-runnable", 256, 1024, 1024, peaks)
        leg(bench_fused_epilogue, 4096, 7168, 18432, peaks=peaks)
        leg(bench_fused_epilogue, 8192, 7168, 2048, peaks=peaks)
        leg(bench_fused_epilogue, M, N, K, iters=5, peaks=peaks)
        leg(bench_grouped, peaks)
        leg(bench_reference_blackwell_gemm, peaks)
        if sustained is not None:
            extras.append(sustained)
        line["other_workloads"] = extras
        line["other_workloads_note"] = ("each side measurement is a burst of about ten launches started after 0.5 s of idle; "
                                        "the sustained figure of the main workload is the entry timed over ~2 s")
        from yan_b200.utils import perf_log
        for record in extras:  # one JSON line per side measurement when YAN_PERF_LOG names a file
            perf_log(record)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        a_cpu, rhs_cpu = make_cpu_inputs()
        cpu_reference_step(a_cpu, rhs_cpu)
        reps, t0 = 0, time.perf_counter()
        while reps < 3 or (time.perf_counter() - t0 < 10.0 and reps < 50):
            cpu_reference_step(a_cpu, rhs_cpu)
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        line["cpu_baseline"] = {"value": 2.0 * CPU_SLAB_ROWS * N * K / dt / 1e12, "unit": "TFLOP/s",
                                "cores": torch.get_num_threads(), "kind": "port",
                                "sample": f"{reps} passes over a {CPU_SLAB_ROWS}-row slab of A against the full B "
                                          f"(quantize, dequantize both operands, fp32 torch.matmul, bf16)"}
    if rank == 0:
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    os.close(json_fd)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_case(args) -> None:
    """One shape, `steps` launches after `warmup`: the small workload that profiler captures are taken on."""
    import yan_b200
    dims = [int(v) for v in args.case.split(",")]
    m, n, k = dims[:3]
    block_n = dims[3] if len(dims) > 3 else 0
    torch.cuda.set_device(0)
    a, rhs = make_device_inputs(m, n, k, 0, outliers=(m <= 64))
    lhs = yan_b200.per_token_cast_to_fp8(a)
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    for _ in range(args.warmup):
        yan_b200.per_token_cast_to_fp8(a, out=lhs)
        yan_b200.gemm_fp8_fp8_bf16_nt(lhs, rhs, out, block_n=block_n)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        yan_b200.per_token_cast_to_fp8(a, out=lhs)
        yan_b200.gemm_fp8_fp8_bf16_nt(lhs, rhs, out, block_n=block_n)
    e1.record()
    torch.cuda.synchronize()
    assert yan_b200.read_device_status() == 0
    ms = e0.elapsed_time(e1) / args.steps
    print(json.dumps({"case": [m, n, k], "block_n": block_n, "ms_per_step": ms,
                      "TFLOP/s": 2.0 * m * n * k / (ms / 1e3) / 1e12}), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the decode / C3 / C1 side measurements")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-threads", type=int, default=0, help="host threads of the CPU arm (0 = all cores)")
    ap.add_argument("--case", default=None, metavar="M,N,K[,BLOCK_N]",
                    help="profiling aid: run quantize + GEMM of one shape `--steps` times on one GPU and print its timing")
    args = ap.parse_args()
    if args.case is not None:
        return run_case(args)
    assert args.warmup >= 3 or args.impl == "reference", "at least 3 warm-up steps"
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
