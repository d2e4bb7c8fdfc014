"""The bounded device-side waits: a probe kernel waits on an mbarrier that nothing arrives on, with the same
bounded wait the GEMM kernels use; the wait runs out after its bound, the kernel records the site in the device
status word and returns; the context stays usable.  Nothing faults, traps or hangs in this test."""
import ctypes
import time

import pytest
import torch

from oracle import ref

pytestmark = pytest.mark.gpu


def test_wait_bound_expiry_sets_status_and_context_survives(cuda_lib):
    import yan_b200
    from yan_b200 import _lib
    assert yan_b200.read_device_status() == 0
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    t0 = time.perf_counter()
    _lib.call("yan_b200_wait_probe", 2_000_000, stream)          # 2 ms bound
    torch.cuda.synchronize()                                      # the kernel returns by itself
    assert time.perf_counter() - t0 < 1.0
    status = yan_b200.read_device_status(reset=True)
    assert status == (6 << 8) | 15, f"expected YAN_B200_DEVICE_TIMEOUT at site 15, got {status:#x}"
    assert yan_b200.read_device_status() == 0                     # reset worked
    assert _lib.call_rc("yan_b200_wait_probe", 5_000_000_000, stream) == 1   # probes may not wait longer than 1 s

    # the context is intact: a GEMM right after is correct
    a, b = ref.make_inputs(256, 1024, 1024, seed=0)
    lhs, rhs = ref.per_token_cast_to_fp8(a), ref.per_block_cast_to_fp8(b)
    out = torch.zeros(256, 1024, dtype=torch.bfloat16, device="cuda")
    yan_b200.gemm_fp8_fp8_bf16_nt((lhs[0].cuda(), lhs[1].t().contiguous().cuda().t()), (rhs[0].cuda(), rhs[1].cuda()), out)
    torch.cuda.synchronize()
    assert yan_b200.read_device_status() == 0
    assert ref.rel_frobenius(out.cpu(), ref.ref_gemm(lhs, rhs)) <= 1e-3
