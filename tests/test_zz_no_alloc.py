"""The allocation-free quantize+GEMM entry point against the workspace-taking one.

Callers that cannot allocate device memory (all of it already belongs to a cache pool, or they run
inside another runtime's budget) use yan_b200_fp8_linear_bf16_static, whose scratch lives in a fixed
array inside the library.  It must give what yan_b200_fp8_linear_bf16 gives, call after call, because
every call reuses the same array with the previous call's bytes still in it.

This file sorts last so that a run stopping at the first failure has already run every other test.
"""
import ctypes

import pytest
import torch

from oracle import ref

pytestmark = pytest.mark.gpu

REL_FRO_TOL = 1e-3


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _both(a, rhs_q, rhs_s):
    """Runs both entry points through the C ABI on the same inputs; returns (static, workspace) outputs."""
    from yan_b200 import _lib
    m, k = a.shape
    n = rhs_q.shape[0]
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    out_static = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    out_ws = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    ws_bytes = _lib.lib().yan_b200_fp8_linear_workspace_bytes(m, k)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    _lib.call("yan_b200_fp8_linear_bf16_static", a.data_ptr(), rhs_q.data_ptr(), rhs_s.data_ptr(),
              out_static.data_ptr(), m, n, k, n, _stream(), sms, 0)
    _lib.call("yan_b200_fp8_linear_bf16", a.data_ptr(), rhs_q.data_ptr(), rhs_s.data_ptr(), out_ws.data_ptr(),
              ws.data_ptr(), ws_bytes, m, n, k, n, _stream(), sms, 0)
    torch.cuda.synchronize()
    return out_static, out_ws


def test_static_scratch_matches_workspace_entry_twice_in_a_row(cuda_lib):
    # Two different problems back to back: the second finds the first one's bytes in the shared array.
    for seed, (m, n, k) in enumerate([(256, 1024, 1024), (64, 512, 2048)]):
        a, b = ref.make_inputs(m, n, k, seed=seed, outliers=(m == 64))
        rhs = ref.per_block_cast_to_fp8(b)
        out_static, out_ws = _both(a.cuda(), rhs[0].cuda(), rhs[1].cuda())
        assert not torch.isnan(out_static.float()).any()
        # the two entry points run the same two kernels on the same inputs: nothing may differ
        assert torch.equal(out_static, out_ws), f"call {seed}: static and workspace entry points differ"
        # and both agree with the CPU oracle
        d_ref = ref.ref_gemm(ref.per_token_cast_to_fp8(a), rhs)
        assert ref.rel_frobenius(out_static.cpu(), d_ref) <= REL_FRO_TOL


def test_static_scratch_rejects_oversized_problem(cuda_lib):
    from yan_b200 import _lib
    limit = _lib.STATIC_SCRATCH_MAX_ELEMENTS
    m, k = 4096, 4096  # 16 Mi elements
    assert m * k > limit
    p = torch.zeros(1 << 12, dtype=torch.uint8, device="cuda").data_ptr()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    rc = _lib.call_rc("yan_b200_fp8_linear_bf16_static", p, p, p, p, m, 128, k, 128, _stream(), sms, 0)
    assert rc == 7, "expected YAN_B200_WORKSPACE_TOO_SMALL"
