"""GEMM with the next layer's quantizer fused into the epilogue (e4m3 output + 1x128 scales).

Two checks: bit-exact against the two-kernel path it replaces (bf16 GEMM with the same tile, then
per_token_cast_to_fp8), and the dequantized result against the CPU oracle within the GEMM tolerance plus the
quantization step of e4m3 (3 mantissa bits: relative error <= 2^-4 per element).
"""
import pytest
import torch

from oracle import ref

pytestmark = pytest.mark.gpu


def _device_operands(m, n, k, seed, outliers=False):
    a, b = ref.make_inputs(m, n, k, seed=seed, outliers=outliers)
    lhs = ref.per_token_cast_to_fp8(a)
    rhs = ref.per_block_cast_to_fp8(b)
    lhs_d = (lhs[0].cuda(), lhs[1].t().contiguous().cuda().t())
    rhs_d = (rhs[0].cuda(), rhs[1].cuda())
    return lhs, rhs, lhs_d, rhs_d


@pytest.mark.parametrize("m,n,k", [(256, 1024, 1024), (1, 128, 128), (130, 384, 256), (77, 256, 512), (512, 2560, 2048)])
def test_bit_exact_against_gemm_then_quantizer(cuda_lib, m, n, k):
    import yan_b200
    _, _, lhs_d, rhs_d = _device_operands(m, n, k, seed=m + k, outliers=True)
    q, s = yan_b200.gemm_fp8_fp8_e4m3_nt(lhs_d, rhs_d)
    d = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    yan_b200.gemm_fp8_fp8_bf16_nt(lhs_d, rhs_d, d, block_n=256)
    q2, s2 = yan_b200.per_token_cast_to_fp8(d)
    torch.cuda.synchronize()
    assert yan_b200.read_device_status() == 0
    assert s.shape == (m, n // 128) and s.stride(0) == 1
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8))
    assert torch.equal(s, s2)
    # and the oracle's quantizer on the same bf16 tensor
    q3, s3 = ref.per_token_cast_to_fp8(d.cpu())
    assert torch.equal(q.cpu().view(torch.uint8), q3.view(torch.uint8))
    assert torch.equal(s.cpu(), s3)


def test_dequantized_output_against_oracle(cuda_lib):
    import yan_b200
    lhs, rhs, lhs_d, rhs_d = _device_operands(256, 1024, 1024, seed=0)
    q, s = yan_b200.gemm_fp8_fp8_e4m3_nt(lhs_d, rhs_d)
    torch.cuda.synchronize()
    d_ref = ref.ref_gemm(lhs, rhs).float()
    d = ref.dequant_a(q.cpu(), s.cpu().contiguous())
    # e4m3 rounding: half a step of a 3-bit mantissa relative to the element, 2^-4; subnormal codes of a group are
    # bounded by the group's scale (2^-9 * 448 * scale ... = scale * 2^-10 absolute half-step).
    err = (d - d_ref).abs()
    bound = d_ref.abs() * 2.0 ** -4 + s.cpu().repeat_interleave(128, dim=1) * 2.0 ** -9 + 2.0 ** -6
    assert bool((err <= bound).all()), float((err - bound).max())
    assert ref.rel_frobenius(d, d_ref) <= 4e-2  # rounding error of a 3-bit mantissa: at most 2^-4 / sqrt(3) = 3.6e-2 rms


def test_feeds_the_next_gemm(cuda_lib):
    """The fused output is consumed as the lhs of a second GEMM; equal to the unfused chain bit for bit."""
    import yan_b200
    _, _, lhs_d, rhs1 = _device_operands(192, 512, 256, seed=4)
    _, _, _, rhs2 = _device_operands(192, 384, 512, seed=5)
    h = yan_b200.gemm_fp8_fp8_e4m3_nt(lhs_d, rhs1)
    out = torch.empty((192, 384), dtype=torch.bfloat16, device="cuda")
    yan_b200.gemm_fp8_fp8_bf16_nt(h, rhs2, out)
    d = torch.empty((192, 512), dtype=torch.bfloat16, device="cuda")
    yan_b200.gemm_fp8_fp8_bf16_nt(lhs_d, rhs1, d, block_n=256)
    want = torch.empty_like(out)
    yan_b200.gemm_fp8_fp8_bf16_nt(yan_b200.per_token_cast_to_fp8(d), rhs2, want)
    torch.cuda.synchronize()
    assert torch.equal(out, want)


def test_caller_buffers_and_limits(cuda_lib):
    import ctypes
    import yan_b200
    from yan_b200 import _lib
    _, _, lhs_d, rhs_d = _device_operands(64, 256, 256, seed=8)
    wide = torch.zeros((64, 512), dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    scales = torch.full((2, 96), -1.0, dtype=torch.float32, device="cuda")  # leading dimension 96 > M
    q, s = yan_b200.gemm_fp8_fp8_e4m3_nt(lhs_d, rhs_d, out=(wide[:, 256:], scales[:, :64].t()))
    q2, s2 = yan_b200.gemm_fp8_fp8_e4m3_nt(lhs_d, rhs_d)
    torch.cuda.synchronize()
    assert torch.equal(wide[:, 256:].view(torch.uint8), q2.view(torch.uint8))
    assert torch.equal(scales[:, :64].t(), s2)
    assert bool((wide[:, :256].view(torch.uint8) == 0).all()) and bool((scales[:, 64:] == -1.0).all())
    p = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda").data_ptr()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    f = "yan_b200_gemm_fp8_fp8_e4m3_nt"
    assert _lib.call_rc(f, p, p, p, p, p, p, 64, 192, 256, 192, 64, stream, sms) == 1   # N not a multiple of 128
    assert _lib.call_rc(f, p, p, p, p, p, p, 64, 256, 256, 256, 32, stream, sms) == 1   # scale leading dimension < M
    assert _lib.call_rc(f, p, p, p, p, p, None, 64, 256, 256, 256, 64, stream, sms) == 1  # no scale buffer
