"""yan_b200: the FP8 fine-grained-scaled GEMM path of zoheth/yan, rebuilt for B200 (sm_100a).

Public names follow the reference's package (yan/__init__.py:1-5): `jit`, `gemm` (the operator
module, which here also holds the callables the reference never wrote), `bench_kineto`, `calc_diff`,
`get_col_major_tensor`.  The kernels are CUDA only; importing an operator without the built library
raises (no CPU or PyTorch fallback exists).
"""
from . import jit
from .jit_kernels import gemm
from .jit_kernels import (ceil_div, fp8_linear, fp8_linear_workspace_bytes, gemm_fp8_fp8_bf16_nt, gemm_fp8_fp8_e4m3_nt,
                          gemm_fp8_fp8_f32_nt,
                          get_col_major_tensor, get_m_alignment_for_contiguous_layout, get_num_sms,
                          m_grouped_gemm_fp8_fp8_bf16_nt_contiguous, m_grouped_gemm_fp8_fp8_bf16_nt_masked,
                          per_block_cast_to_fp8, per_token_cast_to_fp8, read_device_status, set_num_sms,
                          set_programmatic_dependent_launch, set_clock_probe, effective_sm_clock_mhz, set_tail_cut)
from .jit_kernels import HostFp8Linear
from .utils import bench_events, bench_kineto, calc_diff, count_bytes, perf_log

__version__ = "0.1.0"
