"""FP8 fine-grained-scaled GEMM: the Python entry the reference never wrote.

yan/jit_kernels/gemm.py:1-31 consists of a launch template only.  This module keeps that template
(same variable names: lhs, lhs_scales, rhs, rhs_scales, out, m, stream, num_sms, smem_size; same
JIT keys N, K, BLOCK_M, BLOCK_N, NUM_STAGES) and adds the missing functions.  The reference's sixth key, the number
of CTAs one TMA load is delivered to, is fixed at 1: every CTA of this kernel loads its own tiles.
By default a call goes to the prebuilt C-ABI library; `YAN_FP8_GEMM_JIT=1` routes it through
`jit_tuner.compile_and_tune` with the template below, specialising N and K at compile time exactly
as the reference intends (`YAN_FP8_GEMM_TUNE=1` additionally lets the tuner time every tile width).  Both run the same kernel source (include/gemm/fp8_gemm.cuh).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch

from .. import _lib
from .quant import per_token_cast_to_fp8
from .utils import ceil_div, get_col_major_tensor, get_m_alignment_for_contiguous_layout, get_num_sms

# C++ code templates (JIT path)
includes = ('"gemm/fp8_gemm.cuh"', )
template = """
using namespace yan;

// Templated args from Python JIT call
constexpr auto N = {N}, K = {K};
constexpr auto BLOCK_M = {BLOCK_M};
constexpr auto BLOCK_N = {BLOCK_N};
constexpr auto kNumStages = {NUM_STAGES};
constexpr auto kNumCtasPerLoad = 1;

// Make a templated GEMM
using GemmType = Gemm<N, K, BLOCK_M, BLOCK_N, 128, 1, kNumStages, kNumCtasPerLoad, GemmType::Normal>;

// Launch kernel
auto tma_a_desc = GemmType::make_2d_tma_a_desc(lhs, m);
auto tma_b_desc = GemmType::make_2d_tma_b_desc(rhs);
auto tma_scales_a_desc = GemmType::make_2d_tma_scales_a_desc(lhs_scales, m);
auto tma_d_desc = GemmType::make_2d_tma_d_desc(out, m);
__return_code = GemmType::run(out, rhs_scales, nullptr,
              m,
              tma_a_desc, tma_b_desc, tma_scales_a_desc, tma_d_desc,
              stream, num_sms, smem_size);
"""

arg_defs = (('lhs', torch.float8_e4m3fn), ('lhs_scales', torch.float),
            ('rhs', torch.float8_e4m3fn), ('rhs_scales', torch.float),
            ('out', torch.bfloat16), ('m', int),
            ('stream', torch.cuda.Stream), ('num_sms', int), ('smem_size', int))

_DEFAULT_STAGES = {32: 8, 64: 8, 96: 8, 128: 6, 160: 6, 192: 5, 224: 5, 256: 4}


def get_smem_size(block_n: int, num_stages: int) -> int:
    """Dynamic shared memory of one CTA: stages x (A 128x128 + B BLOCK_Nx128 e4m3) + the output staging boxes
    (8 x 2 KB, where the ring leaves room) + mbarriers + 1024 bytes of alignment slack (GemmSmemLayout in
    include/gemm/fp8_gemm.cuh)."""
    num_tmem_bufs = 2 if block_n > 128 else 4
    ring = num_stages * (128 * 128 + block_n * 128)
    store = 8 * 2048 if ring + 8 * 2048 + 2048 <= 232448 else 0
    return ring + store + (2 * num_stages + 4 * num_tmem_bufs) * 8 + 8 + 1024


# time of one tile relative to a 256-wide one (measured; see choose_block_n in csrc/capi.cu)
_TILE_COST = {256: 1.000, 224: 1.08, 192: 0.84, 160: 0.82, 128: 0.67, 96: 0.72, 64: 0.57, 32: 0.50}


def get_best_configs(m: int, n: int, k: int, num_sms: int) -> Tuple[int, int, int]:
    """(BLOCK_N, NUM_STAGES, smem_size) by the same wave model as the C library's default."""
    best, best_cost = 256, None
    for bn, tile_cost in _TILE_COST.items():
        if bn > 32 and n < bn:
            continue
        waves = ceil_div(ceil_div(m, 128) * ceil_div(n, bn), num_sms)
        cost = waves * tile_cost
        if best_cost is None or cost < best_cost * 0.98:
            best, best_cost = bn, cost
    stages = _DEFAULT_STAGES[best]
    return best, stages, get_smem_size(best, stages)


def _stream_ptr() -> ctypes.c_void_p:
    return _lib.current_stream_ptr()


def _check_operands(lhs, lhs_scales, rhs, rhs_scales, out, out_dtype) -> Tuple[int, int, int]:
    m, k = lhs.shape
    n, k_ = rhs.shape
    assert k == k_ and m > 0 and n > 0 and k > 0, "shape mismatch"
    assert k % 128 == 0, "K must be a multiple of 128 (one scale per 128-wide k-block)"
    assert n % 16 == 0
    assert lhs.is_cuda and rhs.is_cuda and out.is_cuda and lhs_scales.is_cuda and rhs_scales.is_cuda
    assert lhs.dtype == torch.float8_e4m3fn and rhs.dtype == torch.float8_e4m3fn
    assert lhs_scales.dtype == torch.float32 and rhs_scales.dtype == torch.float32
    assert out.dtype == out_dtype and out.shape == (m, n)
    assert lhs.is_contiguous() and rhs.is_contiguous() and rhs_scales.is_contiguous()
    assert lhs_scales.shape == (m, k // 128)
    assert rhs_scales.shape == (ceil_div(n, 128), k // 128)
    vec = 16 // out.element_size()
    assert out.stride(1) == 1 and out.stride(0) >= n and out.stride(0) % vec == 0 and out.data_ptr() % 16 == 0
    assert lhs.data_ptr() % 16 == 0 and rhs.data_ptr() % 16 == 0
    return m, n, k


def gemm_fp8_fp8_bf16_nt(lhs: Tuple[torch.Tensor, torch.Tensor], rhs: Tuple[torch.Tensor, torch.Tensor],
                         out: torch.Tensor, block_n: int = 0) -> None:
    """out[M,N] (bf16) = dequant(lhs)[M,K] @ dequant(rhs)[N,K]^T with fp32 accumulation.

    lhs = (e4m3 [M,K], fp32 scales [M, K/128]) -- 1x128 groups; column-major scales are used as
    they are, row-major ones are transposed first (get_col_major_tensor).
    rhs = (e4m3 [N,K], fp32 scales [N/128, K/128]) -- 128x128 blocks.
    `out` is caller-allocated and may be a column slice of a wider row-major buffer.
    """
    lhs_q, lhs_scales = lhs
    rhs_q, rhs_scales = rhs
    m, n, k = _check_operands(lhs_q, lhs_scales, rhs_q, rhs_scales, out, torch.bfloat16)
    lhs_scales = get_col_major_tensor(lhs_scales)
    if m == 1 or lhs_scales.stride(1) != m:
        lhs_scales = lhs_scales.t().contiguous().t()
    num_sms = get_num_sms()
    if os.environ.get("YAN_FP8_GEMM_JIT", "0") not in ("0", ""):
        from .tuner import jit_tuner
        assert out.stride(0) == n, "the JIT specialisation writes a dense [M, N] output"
        # smem_size = 0: each candidate checks its own requirement against the device limit and reports
        # kSmemTooLarge through the return code, which the tuner treats as "skip this configuration".
        args = (lhs_q, lhs_scales, rhs_q, rhs_scales, out, m, torch.cuda.current_stream(), num_sms, 0)
        if block_n == 0 and int(os.environ.get("YAN_FP8_GEMM_TUNE", "0")):
            # time every tile width that can fill the machine; the winner is remembered per (N, K, M bucket)
            space = tuple({'BLOCK_N': bn, 'NUM_STAGES': _DEFAULT_STAGES[bn]} for bn in (256, 224, 192, 160, 128, 96, 64, 32) if bn <= n)
            keys = {'N': n, 'K': k, 'BLOCK_M': 128, 'M_BUCKET': ceil_div(m, 128)}
        else:
            bn = get_best_configs(m, n, k, num_sms)[0] if block_n == 0 else block_n
            space = ()
            keys = {'N': n, 'K': k, 'BLOCK_M': 128, 'BLOCK_N': bn, 'NUM_STAGES': _DEFAULT_STAGES[bn]}
        runtime = jit_tuner.compile_and_tune(name='gemm_fp8_fp8_bf16_nt', keys=keys, space=space, includes=includes,
                                             arg_defs=arg_defs, template=template, args=args)
        rc = runtime(*args)
        if rc != 0:
            raise _lib.YanB200Error('gemm_fp8_fp8_bf16_nt[jit]', rc, 'see ReturnCode in include/gemm/utils.cuh')
        _jit_runtimes_used[runtime.path] = runtime
        return
    # the cut only ever applies to long K and more tiles than CTAs (choose_tail_slices in include/gemm/fp8_gemm.cuh)
    if block_n == 0 and k >= 96 * 128 and ceil_div(m, 128) * ceil_div(n, 256) > num_sms and tail_cut_enabled():
        # the library may cut the tiles of a nearly empty last wave along K (scratch per device and stream)
        ws = _tail_workspace(out.device, num_sms)
        _lib.call("yan_b200_gemm_fp8_fp8_bf16_nt_tail", lhs_q.data_ptr(), lhs_scales.data_ptr(), rhs_q.data_ptr(),
                  rhs_scales.data_ptr(), out.data_ptr(), m, n, k, out.stride(0), _stream_ptr(), num_sms, block_n,
                  ws.data_ptr(), ws.numel())
        return
    _lib.call("yan_b200_gemm_fp8_fp8_bf16_nt", lhs_q.data_ptr(), lhs_scales.data_ptr(), rhs_q.data_ptr(),
              rhs_scales.data_ptr(), out.data_ptr(), m, n, k, out.stride(0), _stream_ptr(), num_sms, block_n)


_tail_workspaces = {}
_tail_cut = [True]


def tail_cut_enabled() -> bool:
    return _tail_cut[0]


def set_tail_cut(enabled: bool) -> None:
    """Lets gemm_fp8_fp8_bf16_nt(block_n=0) cut the tiles of a nearly empty last wave along K (default on).  Off, or
    with an explicit block_n, every tile is computed whole by one CTA and the result does not depend on the grid."""
    _tail_cut[0] = bool(enabled)


def _tail_workspace(device: torch.device, num_sms: int) -> torch.Tensor:
    """Scratch for the partial tiles, one per (device, stream, grid): launches on one stream are ordered, launches on
    different streams must not share a workspace."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream, num_sms)
    ws = _tail_workspaces.get(key)
    if ws is None:
        need = int(_lib.lib().yan_b200_gemm_tail_workspace_bytes(num_sms))
        ws = torch.empty(need, dtype=torch.uint8, device=device)
        _tail_workspaces[key] = ws
    return ws


def gemm_fp8_fp8_f32_nt(lhs, rhs, out: torch.Tensor, block_n: int = 0) -> None:
    """Same GEMM with an fp32 output (partial sums of the K-split path keep full precision)."""
    lhs_q, lhs_scales = lhs
    rhs_q, rhs_scales = rhs
    m, n, k = _check_operands(lhs_q, lhs_scales, rhs_q, rhs_scales, out, torch.float32)
    lhs_scales = get_col_major_tensor(lhs_scales)
    if m == 1 or lhs_scales.stride(1) != m:
        lhs_scales = lhs_scales.t().contiguous().t()
    _lib.call("yan_b200_gemm_fp8_fp8_f32_nt", lhs_q.data_ptr(), lhs_scales.data_ptr(), rhs_q.data_ptr(),
              rhs_scales.data_ptr(), out.data_ptr(), m, n, k, out.stride(0), _stream_ptr(), get_num_sms(), block_n)


def gemm_fp8_fp8_e4m3_nt(lhs, rhs, out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
                         ) -> Tuple[torch.Tensor, torch.Tensor]:
    """The GEMM with the next layer's activation quantizer fused into its epilogue.

    Returns (e4m3 [M,N], fp32 scales [M, N/128] stored column-major) -- the `lhs` operand of the following
    gemm_fp8_fp8_*_nt -- equal bit for bit to per_token_cast_to_fp8(bf16 output of gemm_fp8_fp8_bf16_nt(..., block_n=256)),
    without the bf16 tensor being written or read.  N must be a multiple of 128.  The reference's epilogue writes
    bf16 only (yan/include/gemm/fp8_gemm.cuh:56,87)."""
    lhs_q, lhs_scales = lhs
    rhs_q, rhs_scales = rhs
    m, n = lhs_q.shape[0], rhs_q.shape[0]
    assert n % 128 == 0, "the fused quantizer works on whole 1 x 128 groups"
    if out is None:
        out = (torch.empty((m, n), dtype=torch.float8_e4m3fn, device=lhs_q.device),
               torch.empty((n // 128, m), dtype=torch.float32, device=lhs_q.device).t())
    out_q, out_scales = out
    m, n, k = _check_operands(lhs_q, lhs_scales, rhs_q, rhs_scales, out_q, torch.float8_e4m3fn)
    assert out_scales.dtype == torch.float32 and out_scales.shape == (m, n // 128) and out_scales.is_cuda
    assert out_scales.stride(0) == 1 and (n == 128 or out_scales.stride(1) >= m), "scales are stored column-major"
    lhs_scales = get_col_major_tensor(lhs_scales)
    if m == 1 or lhs_scales.stride(1) != m:
        lhs_scales = lhs_scales.t().contiguous().t()
    out_scales_ld = out_scales.stride(1) if n > 128 else m
    _lib.call("yan_b200_gemm_fp8_fp8_e4m3_nt", lhs_q.data_ptr(), lhs_scales.data_ptr(), rhs_q.data_ptr(),
              rhs_scales.data_ptr(), out_q.data_ptr(), out_scales.data_ptr(), m, n, k, out_q.stride(0), out_scales_ld,
              _stream_ptr(), get_num_sms())
    return out_q, out_scales


def m_grouped_gemm_fp8_fp8_bf16_nt_contiguous(lhs, rhs, out: torch.Tensor, m_indices: torch.Tensor,
                                              block_n: int = 0) -> None:
    """Grouped GEMM, contiguous layout (yan/include/gemm/scheduler.cuh:9, GemmType::GroupedContiguous):
    rows of lhs [M_sum, K] are concatenated groups, each padded to a multiple of 128 rows
    (get_m_alignment_for_contiguous_layout); m_indices[M_sum] (int32) names each row's group, -1 marks
    padding rows whose output is left untouched.  rhs = (e4m3 [G, N, K], scales [G, N/128, K/128])."""
    lhs_q, lhs_scales = lhs
    rhs_q, rhs_scales = rhs
    m, k = lhs_q.shape
    g, n, k_ = rhs_q.shape
    assert k == k_ and k % 128 == 0 and n % 128 == 0 and m % get_m_alignment_for_contiguous_layout() == 0
    assert lhs_q.dtype == torch.float8_e4m3fn and rhs_q.dtype == torch.float8_e4m3fn
    assert lhs_q.is_contiguous() and rhs_q.is_contiguous() and rhs_scales.is_contiguous() and out.is_contiguous()
    assert lhs_scales.shape == (m, k // 128) and rhs_scales.shape == (g, n // 128, k // 128)
    assert out.shape == (m, n) and out.dtype == torch.bfloat16
    assert m_indices.shape == (m,) and m_indices.dtype == torch.int32 and m_indices.is_contiguous()
    lhs_scales = get_col_major_tensor(lhs_scales)
    if lhs_scales.stride(1) != m:
        lhs_scales = lhs_scales.t().contiguous().t()
    _lib.call("yan_b200_m_grouped_gemm_fp8_fp8_bf16_nt_contiguous", lhs_q.data_ptr(), lhs_scales.data_ptr(),
              rhs_q.data_ptr(), rhs_scales.data_ptr(), out.data_ptr(), m_indices.data_ptr(), m, n, k, g,
              _stream_ptr(), get_num_sms(), block_n)


def m_grouped_gemm_fp8_fp8_bf16_nt_masked(lhs, rhs, out: torch.Tensor, masked_m: torch.Tensor,
                                          expected_m: int = 0, block_n: int = 0) -> None:
    """Grouped GEMM, masked layout (scheduler.cuh:10, GemmType::GroupedMasked): lhs = (e4m3 [G, M_max, K],
    scales [G, M_max, K/128]); only the first masked_m[g] rows of group g are computed and stored.
    `expected_m` (typical rows per group) only steers the tile choice."""
    lhs_q, lhs_scales = lhs
    rhs_q, rhs_scales = rhs
    g, m_max, k = lhs_q.shape
    g_, n, k_ = rhs_q.shape
    assert g == g_ and k == k_ and k % 128 == 0 and n % 128 == 0
    assert lhs_q.is_contiguous() and rhs_q.is_contiguous() and rhs_scales.is_contiguous() and out.is_contiguous()
    assert lhs_scales.shape == (g, m_max, k // 128) and rhs_scales.shape == (g, n // 128, k // 128)
    assert out.shape == (g, m_max, n) and out.dtype == torch.bfloat16
    assert masked_m.shape == (g,) and masked_m.dtype == torch.int32 and masked_m.is_contiguous()
    # k-block-major over the flattened G*M_max rows
    sa = lhs_scales.reshape(g * m_max, k // 128)
    sa = get_col_major_tensor(sa)
    if sa.stride(1) != g * m_max:
        sa = sa.t().contiguous().t()
    _lib.call("yan_b200_m_grouped_gemm_fp8_fp8_bf16_nt_masked", lhs_q.data_ptr(), sa.data_ptr(), rhs_q.data_ptr(),
              rhs_scales.data_ptr(), out.data_ptr(), masked_m.data_ptr(), m_max, n, k, g, _stream_ptr(),
              get_num_sms(), block_n)


_workspaces = {}


def fp8_linear(a: torch.Tensor, rhs: Tuple[torch.Tensor, torch.Tensor], out: Optional[torch.Tensor] = None,
               workspace: Optional[torch.Tensor] = None, block_n: int = 0) -> torch.Tensor:
    """bf16 a [M,K] -> quantize (1x128) -> FP8 GEMM with rhs -> bf16 [M,N], one C-ABI call.
    `workspace` (uint8, >= fp8_linear_workspace_bytes(M, K)) holds the quantized activations between the
    two kernels; when omitted a per-(device, size) buffer is allocated once and reused."""
    rhs_q, rhs_scales = rhs
    m, k = a.shape
    n = rhs_q.shape[0]
    assert a.is_cuda and a.dtype == torch.bfloat16 and a.is_contiguous() and k % 128 == 0
    assert rhs_q.dtype == torch.float8_e4m3fn and rhs_q.shape == (n, k) and rhs_q.is_contiguous()
    assert rhs_scales.shape == (ceil_div(n, 128), k // 128) and rhs_scales.is_contiguous()
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    assert out.shape == (m, n) and out.dtype == torch.bfloat16 and out.stride(1) == 1
    need = fp8_linear_workspace_bytes(m, k)
    if workspace is None:
        key = (a.device.index, need)
        if key not in _workspaces:
            _workspaces[key] = torch.empty(need, dtype=torch.uint8, device=a.device)
        workspace = _workspaces[key]
    assert workspace.is_cuda and workspace.dtype == torch.uint8 and workspace.numel() >= need
    _lib.call("yan_b200_fp8_linear_bf16", a.data_ptr(), rhs_q.data_ptr(), rhs_scales.data_ptr(), out.data_ptr(),
              workspace.data_ptr(), workspace.numel(), m, n, k, out.stride(0), _stream_ptr(), get_num_sms(), block_n)
    return out


def fp8_linear_workspace_bytes(m: int, k: int) -> int:
    return int(_lib.lib().yan_b200_fp8_linear_workspace_bytes(m, k))


def set_programmatic_dependent_launch(enabled: bool) -> None:
    """Lets the M <= 64 weight-streaming kernel start fetching weights while the previous kernel of the stream is
    still running (programmatic dependent launch), and lets the quantizer inside fp8_linear be launched over the tail of
    the kernel before it.  Only valid when the weights are not produced by the kernel that precedes a GEMM."""
    _lib.lib().yan_b200_set_programmatic_dependent_launch(int(bool(enabled)))


def set_clock_probe(buffer: Optional[torch.Tensor]) -> None:
    """Points the kernels' clock probe at `buffer` (int64, >= 16 elements, on the current device) or switches it off
    (None).  After a general-kernel GEMM, buffer[0:4] = CTA 0's {clock64, globaltimer ns} at start and end; see
    `effective_sm_clock_mhz`.  (The reference stamps clock64 per SM the same way, flash_attn_tk.cuh:56-63.)"""
    if buffer is None:
        _lib.lib().yan_b200_set_clock_probe(None)
        return
    assert buffer.is_cuda and buffer.dtype == torch.int64 and buffer.numel() >= 16 and buffer.is_contiguous()
    _lib.lib().yan_b200_set_clock_probe(buffer.data_ptr())


def effective_sm_clock_mhz(buffer: torch.Tensor) -> float:
    """SM clock the last probed GEMM ran at: CTA 0's clock64 delta over its globaltimer delta."""
    v = buffer[:4].tolist()
    return 1000.0 * (v[2] - v[0]) / max(v[3] - v[1], 1)


_jit_runtimes_used = {}  # kernel libraries the JIT route has launched: each has a status word of its own


def read_device_status(reset: bool = True) -> int:
    """Synchronises and returns the device status word (0 = no bounded wait ever ran out): the prebuilt library's, or,
    if that is clean, the first non-zero word of a JIT-compiled GEMM library this process has launched."""
    status = ctypes.c_int(0)
    _lib.call("yan_b200_read_device_status", ctypes.byref(status), int(reset))
    if status.value != 0:
        return status.value
    for runtime in _jit_runtimes_used.values():
        word = runtime.read_device_status(reset)
        if word != 0:
            return word
    return 0
