"""GPU parity of the quantizers: bit-exact against the CPU oracle, through the C ABI."""
import pytest
import torch

from oracle import ref

pytestmark = pytest.mark.gpu


def _cmp_token(x_cpu):
    import yan_b200
    q_ref, s_ref = ref.per_token_cast_to_fp8(x_cpu)
    q, s = yan_b200.per_token_cast_to_fp8(x_cpu.cuda())
    torch.cuda.synchronize()
    assert s.shape == s_ref.shape and s.stride(0) == 1, "scales must be M-contiguous per k-block"
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8)), "e4m3 codes differ from the oracle"
    assert torch.equal(s.cpu().view(torch.int32), s_ref.view(torch.int32)), "scales differ bitwise from the oracle"


@pytest.mark.parametrize("m,k", [(1, 128), (7, 256), (16, 2048), (64, 2048), (129, 384), (256, 1024), (1000, 1152),
                                 (1024, 512), (4096, 1024), (1031, 640)])
def test_per_token_cast_bit_exact(cuda_lib, m, k):
    g = torch.Generator().manual_seed(m * 131 + k)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    _cmp_token(x)


def test_per_token_cast_decode_outliers(cuda_lib):
    a, _ = ref.make_inputs(64, 128, 2048, seed=0, outliers=True)
    _cmp_token(a)


def test_per_token_cast_edge_values(cuda_lib):
    """all-zero groups (amax floor), tiny and huge magnitudes, exact ties, negative zero."""
    x = torch.zeros(8, 512, dtype=torch.float32)
    x[1, :128] = 1e-6
    x[2, 128:256] = torch.linspace(-1.5e38, 1.5e38, 128)  # finite: NaN/Inf inputs are outside the contract
    x[3] = torch.arange(512, dtype=torch.float32) - 256.0
    x[4, ::2] = -0.0
    x[5] = torch.tensor([17.0, 19.0, 448.0, 464.0] * 128)
    x[6, 5] = 1.0
    x[7] = 2.0 ** -130
    _cmp_token(x.to(torch.bfloat16))


def test_per_token_cast_strided_rows_and_preallocated_out(cuda_lib):
    import yan_b200
    g = torch.Generator().manual_seed(5)
    big = torch.randn(33, 1024, generator=g).to(torch.bfloat16)
    x = big[:, 256:768]  # row stride 1024, K = 512
    q_ref, s_ref = ref.per_token_cast_to_fp8(x.contiguous())
    xd = big.cuda()[:, 256:768]
    q = torch.empty(33, 512, dtype=torch.float8_e4m3fn, device="cuda")
    s = torch.empty(4, 33, dtype=torch.float32, device="cuda").t()
    yan_b200.per_token_cast_to_fp8(xd, out=(q, s))
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(s.cpu(), s_ref)


@pytest.mark.parametrize("n,k", [(128, 128), (256, 384), (1024, 1024), (7168, 2048)])
def test_per_block_cast_bit_exact(cuda_lib, n, k):
    import yan_b200
    g = torch.Generator().manual_seed(n + k)
    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)
    q_ref, s_ref = ref.per_block_cast_to_fp8(w)
    q, s = yan_b200.per_block_cast_to_fp8(w.cuda())
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(s.cpu().view(torch.int32), s_ref.view(torch.int32))


def test_quantizer_rejects_bad_arguments(cuda_lib):
    import ctypes
    from yan_b200 import _lib
    x = torch.zeros(4, 200, dtype=torch.bfloat16, device="cuda")
    q = torch.empty(4, 200, dtype=torch.uint8, device="cuda")
    s = torch.empty(8, dtype=torch.float32, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # K not a multiple of 128
    assert _lib.call_rc("yan_b200_per_token_cast_to_fp8", x.data_ptr(), q.data_ptr(), s.data_ptr(), 4, 200, 200, 4, stream) == 1
    # null pointer
    assert _lib.call_rc("yan_b200_per_token_cast_to_fp8", None, q.data_ptr(), s.data_ptr(), 4, 128, 128, 4, stream) == 1
    # scale leading dimension smaller than M
    assert _lib.call_rc("yan_b200_per_token_cast_to_fp8", x.data_ptr(), q.data_ptr(), s.data_ptr(), 4, 128, 200, 2, stream) == 1
