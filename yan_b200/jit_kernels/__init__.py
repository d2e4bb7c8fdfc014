from .gemm import (gemm_fp8_fp8_bf16_nt, gemm_fp8_fp8_e4m3_nt, gemm_fp8_fp8_f32_nt, m_grouped_gemm_fp8_fp8_bf16_nt_contiguous,
                   m_grouped_gemm_fp8_fp8_bf16_nt_masked, fp8_linear, fp8_linear_workspace_bytes, read_device_status,
                   set_programmatic_dependent_launch, set_clock_probe, effective_sm_clock_mhz, set_tail_cut)
from .quant import per_token_cast_to_fp8, per_block_cast_to_fp8
from .utils import (ceil_div, get_col_major_tensor, get_m_alignment_for_contiguous_layout, get_num_sms, set_num_sms)
from .tuner import jit_tuner
from .host import HostFp8Linear
