"""GPU parity of the FP8 GEMM against the CPU oracle (dequantize -> fp32 matmul -> bf16).

Tolerance (both sides rounded to bf16): relative Frobenius error <= 1e-3 and max-abs error <= one bf16
ulp at the binade of max|D_oracle|.
"""
import pytest
import torch

from oracle import ref

pytestmark = pytest.mark.gpu

REL_FRO_TOL = 1e-3


def _operands(m, n, k, seed=0, outliers=False):
    a, b = ref.make_inputs(m, n, k, seed=seed, outliers=outliers)
    lhs = ref.per_token_cast_to_fp8(a)
    rhs = ref.per_block_cast_to_fp8(b)
    return lhs, rhs


def _check(d, d_ref, what=""):
    fro = ref.rel_frobenius(d, d_ref)
    mx = ref.max_abs_err(d, d_ref)
    bound = ref.bf16_ulp_at(float(d_ref.float().abs().max()))
    assert fro <= REL_FRO_TOL, f"{what}: rel Frobenius {fro:.3e} > {REL_FRO_TOL}"
    assert mx <= bound, f"{what}: max abs err {mx} > 1 bf16 ulp at max|D| ({bound})"


def _run(lhs, rhs, block_n=0, out=None):
    import yan_b200
    m, n = lhs[0].shape[0], rhs[0].shape[0]
    lhs_d = (lhs[0].cuda(), lhs[1].t().contiguous().cuda().t())
    rhs_d = (rhs[0].cuda(), rhs[1].cuda())
    if out is None:
        out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    yan_b200.gemm_fp8_fp8_bf16_nt(lhs_d, rhs_d, out, block_n=block_n)
    torch.cuda.synchronize()
    assert yan_b200.read_device_status() == 0
    return out


@pytest.mark.parametrize("block_n", [0, 32, 64, 96, 128, 160, 192, 224, 256])
def test_config1_all_tiles(cuda_lib, block_n):
    """M=256 N=1024 K=1024 seed 0: the CPU-runnable configuration."""
    lhs, rhs = _operands(256, 1024, 1024)
    d = _run(lhs, rhs, block_n)
    _check(d.cpu(), ref.ref_gemm(lhs, rhs), f"C1 block_n={block_n}")


@pytest.mark.parametrize("m", [1, 7, 16, 64, 128, 129, 300])
@pytest.mark.parametrize("n,k", [(128, 128), (256, 256), (384, 1024)])
def test_small_shapes(cuda_lib, m, n, k):
    lhs, rhs = _operands(m, n, k, seed=m + n + k)
    d_ref = ref.ref_gemm(lhs, rhs)
    for block_n in (0, 256):
        d = _run(lhs, rhs, block_n)
        _check(d.cpu(), d_ref, f"m={m} n={n} k={k} block_n={block_n}")


@pytest.mark.parametrize("m", [16, 64])
def test_decode_shape(cuda_lib, m):
    """M in {16, 64}, N=7168, K=2048 with 1 % outlier channels x20."""
    lhs, rhs = _operands(m, 7168, 2048, outliers=True)
    d = _run(lhs, rhs)
    _check(d.cpu(), ref.ref_gemm(lhs, rhs), f"decode m={m}")


@pytest.mark.parametrize("m,n,k", [(1, 128, 256), (16, 256, 512), (17, 384, 1024), (33, 128, 2048), (64, 7168, 2048),
                                   (16, 7168, 2048), (64, 256, 256), (32, 512, 2560), (48, 256, 1536)])
def test_weight_streaming_kernel(cuda_lib, m, n, k):
    """block_n=1 forces the small-M kernel (swap-AB, split-K over a CTA pair); compare with the oracle and with
    the general kernel."""
    lhs, rhs = _operands(m, n, k, seed=m * 7 + k, outliers=True)
    d_ref = ref.ref_gemm(lhs, rhs)
    d_small = _run(lhs, rhs, block_n=1)
    _check(d_small.cpu(), d_ref, f"small-M m={m} n={n} k={k}")
    d_general = _run(lhs, rhs, block_n=64)
    assert ref.rel_frobenius(d_small.cpu(), d_general.cpu()) <= 1e-3


def test_weight_streaming_kernel_limits(cuda_lib):
    import ctypes
    from yan_b200 import _lib
    p = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda").data_ptr()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    f = "yan_b200_gemm_fp8_fp8_bf16_nt"
    assert _lib.call_rc(f, p, p, p, p, p, 128, 128, 256, 128, stream, sms, 1) == 1   # M > 64
    assert _lib.call_rc(f, p, p, p, p, p, 16, 192, 256, 192, stream, sms, 1) == 1    # N not a multiple of 128
    assert _lib.call_rc(f, p, p, p, p, p, 16, 128, 128, 128, stream, sms, 1) == 1    # K not a multiple of 256
    assert _lib.call_rc(f, p, p, p, p, p, 64, 128, 8192, 128, stream, sms, 1) == 1   # too many k-blocks for TMEM


@pytest.mark.parametrize("m,n,k", [(1, 128, 512), (16, 7168, 2048), (9, 256, 1024), (16, 384, 4096), (17, 7168, 2048),
                                   (32, 512, 2048), (5, 2048, 1536)])
def test_stacked_k_kernel(cuda_lib, m, n, k):
    """block_n=2 forces the stacked-K weight-streaming kernel (32 weight rows and all of K per CTA, the four
    k-quarters on the four lane quarters of one MMA); compare with the oracle and with the general kernel."""
    lhs, rhs = _operands(m, n, k, seed=m * 11 + k, outliers=True)
    d_ref = ref.ref_gemm(lhs, rhs)
    d_stacked = _run(lhs, rhs, block_n=2)
    _check(d_stacked.cpu(), d_ref, f"stacked-K m={m} n={n} k={k}")
    d_general = _run(lhs, rhs, block_n=64)
    assert ref.rel_frobenius(d_stacked.cpu(), d_general.cpu()) <= 1e-3


@pytest.mark.parametrize("m,n,k", [(16, 4096, 7168), (3, 256, 2560), (16, 7168, 4096), (9, 96, 16384), (1, 2048, 3072),
                                   (32, 4096, 7168), (17, 256, 2560), (25, 7168, 4096)])
def test_stacked_k_ring_kernel_long_k(cuda_lib, m, n, k):
    """More than four steps (K > 2048): the stacked-K kernel recycles four shared-memory and four tensor-memory slots.
    block_n=2 asks for it, block_n=0 must pick it by itself; both against the oracle."""
    lhs, rhs = _operands(m, max(n, 128), k, seed=m + k, outliers=True)
    d_ref = ref.ref_gemm(lhs, rhs)[:, :n]
    if n < 128:  # three CTAs of 32 weight rows inside one 128-row scale block
        rhs = (rhs[0][:n].contiguous(), rhs[1])
    for block_n in (2, 0):
        _check(_run(lhs, rhs, block_n=block_n).cpu(), d_ref, f"ring m={m} n={n} k={k} block_n={block_n}")


def test_stacked_k_kernel_partial_weight_block(cuda_lib):
    """N = 96: three CTAs of 32 weight rows inside one 128-row scale block, output a slice of a wider buffer."""
    lhs, rhs = _operands(12, 128, 1024, seed=5)
    rhs96 = (rhs[0][:96].contiguous(), rhs[1])
    full = torch.full((12, 256), 7.0, dtype=torch.bfloat16, device="cuda")
    _run(lhs, rhs96, block_n=2, out=full[:, 64:160])
    full = full.cpu()
    _check(full[:, 64:160], ref.ref_gemm(lhs, rhs)[:, :96], "stacked-K slice")
    assert bool((full[:, :64] == 7.0).all()) and bool((full[:, 160:] == 7.0).all())


def test_stacked_k_kernel_limits(cuda_lib):
    import ctypes
    from yan_b200 import _lib
    p = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda").data_ptr()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    f = "yan_b200_gemm_fp8_fp8_bf16_nt"
    assert _lib.call_rc(f, p, p, p, p, p, 33, 128, 512, 128, stream, sms, 2) == 1    # M > 32
    assert _lib.call_rc(f, p, p, p, p, p, 16, 144, 512, 144, stream, sms, 2) == 1    # N not a multiple of 32
    assert _lib.call_rc(f, p, p, p, p, p, 16, 128, 768, 128, stream, sms, 2) == 1    # K not a multiple of 512
    assert _lib.call_rc(f, p, p, p, p, p, 16, 128, 32768, 128, stream, sms, 2) == 1  # more than 32 steps


@pytest.mark.parametrize("block_n", [96, 160, 192, 224])
@pytest.mark.parametrize("m,n,k", [(300, 896, 512), (128, 1024, 1536), (257, 384, 256), (1024, 2560, 2048)])
def test_tile_widths_that_straddle_scale_blocks(cuda_lib, block_n, m, n, k):
    """BLOCK_N in {96, 160, 192, 224}: a promotion warpgroup's column range crosses a 128-column scale block at a
    multiple of 16 (two B scales per k-block), N is not a multiple of the tile width (the last tile reads rows beyond
    N as zeros and stores only the valid columns), and BLOCK_N/2 may end in a 16-column chunk."""
    lhs, rhs = _operands(m, n, k, seed=block_n + m, outliers=True)
    # make neighbouring scale blocks differ strongly so that a wrong block choice cannot pass the tolerance
    q, s = rhs
    s = s * (1.0 + torch.arange(s.shape[0], dtype=torch.float32).view(-1, 1) % 3)
    rhs = (q, s)
    d = _run(lhs, rhs, block_n)
    _check(d.cpu(), ref.ref_gemm(lhs, rhs), f"m={m} n={n} k={k} block_n={block_n}")


def test_long_k_many_tiles(cuda_lib):
    """More tiles than SMs and a long K loop: exercises ring wrap-around and persistent scheduling."""
    lhs, rhs = _operands(1024, 2560, 4096, seed=3)
    d_ref = ref.ref_gemm(lhs, rhs)
    for block_n in (128, 256):
        _check(_run(lhs, rhs, block_n).cpu(), d_ref, f"block_n={block_n}")


def test_output_slice_of_wider_buffer(cuda_lib):
    """The N-split form writes a column slice of a full [M, N_total] buffer and must not touch the rest."""
    lhs, rhs = _operands(192, 256, 512, seed=9)
    full = torch.full((192, 1024), 7.0, dtype=torch.bfloat16, device="cuda")
    _run(lhs, rhs, out=full[:, 512:768])
    full = full.cpu()
    _check(full[:, 512:768], ref.ref_gemm(lhs, rhs), "slice")
    assert bool((full[:, :512] == 7.0).all()) and bool((full[:, 768:] == 7.0).all())


def test_rows_beyond_m_are_not_written(cuda_lib):
    lhs, rhs = _operands(130, 256, 256, seed=11)
    buf = torch.full((256, 256), 3.0, dtype=torch.bfloat16, device="cuda")
    _run(lhs, rhs, out=buf[:130])
    assert bool((buf[130:].cpu() == 3.0).all())


def test_linearity_in_scales(cuda_lib):
    """Size-independent property: doubling every A scale doubles D exactly (power-of-two factor)."""
    lhs, rhs = _operands(256, 512, 1024, seed=21)
    d1 = _run(lhs, rhs).cpu().float()
    d2 = _run((lhs[0], lhs[1] * 2.0), rhs).cpu().float()
    assert torch.equal(d2, d1 * 2.0)


def test_fp32_output(cuda_lib):
    import yan_b200
    lhs, rhs = _operands(200, 384, 1024, seed=4)
    out = torch.empty(200, 384, dtype=torch.float32, device="cuda")
    yan_b200.gemm_fp8_fp8_f32_nt((lhs[0].cuda(), lhs[1].t().contiguous().cuda().t()), (rhs[0].cuda(), rhs[1].cuda()), out)
    d_ref = ref.ref_gemm_f32(lhs, rhs)
    assert ref.rel_frobenius(out.cpu(), d_ref) <= 1e-5


def test_fp8_linear_matches_two_step(cuda_lib):
    import yan_b200
    a, b = ref.make_inputs(256, 1024, 1024, seed=0)
    rhs = ref.per_block_cast_to_fp8(b)
    rhs_d = (rhs[0].cuda(), rhs[1].cuda())
    out = yan_b200.fp8_linear(a.cuda(), rhs_d)
    lhs = ref.per_token_cast_to_fp8(a)
    _check(out.cpu(), ref.ref_gemm(lhs, rhs), "fp8_linear")


@pytest.mark.parametrize("m", [16, 48])
def test_chained_fp8_linear_with_programmatic_launch(cuda_lib, m):
    """Six dependent decode layers (each layer's output is the next one's input, one shared workspace) with every
    kernel launched programmatically: the quantizer may be resident while the GEMM before it still runs, the GEMM
    streams weights while its quantizer runs.  The results must equal the serially launched chain bit for bit."""
    import yan_b200
    a, b = ref.make_inputs(m, 2048, 2048, seed=21)
    rhs = tuple(t.cuda() for t in ref.per_block_cast_to_fp8(b))
    ws = torch.empty(yan_b200.fp8_linear_workspace_bytes(m, 2048), dtype=torch.uint8, device="cuda")

    def chain():
        x, outs = a.cuda(), []
        for _ in range(6):
            x = yan_b200.fp8_linear(x, rhs, torch.empty(m, 2048, dtype=torch.bfloat16, device="cuda"), workspace=ws)
            outs.append(x)
        torch.cuda.synchronize()
        return outs

    serial = chain()
    yan_b200.set_programmatic_dependent_launch(True)
    try:
        overlapped = chain()
    finally:
        yan_b200.set_programmatic_dependent_launch(False)
    assert yan_b200.read_device_status() == 0
    assert all(torch.equal(s, o) for s, o in zip(serial, overlapped))
    lhs = ref.per_token_cast_to_fp8(a)
    _check(serial[0].cpu(), ref.ref_gemm(lhs, tuple(t.cpu() for t in rhs)), "first layer")


def test_gemm_rejects_bad_arguments(cuda_lib):
    import ctypes
    from yan_b200 import _lib
    t = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p = t.data_ptr()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    f = "yan_b200_gemm_fp8_fp8_bf16_nt"
    assert _lib.call_rc(f, p, p, p, p, p, 128, 128, 100, 128, stream, sms, 0) == 1      # K % 128
    assert _lib.call_rc(f, p, p, p, p, p, 128, 128, 128, 64, stream, sms, 0) == 1       # ldd < N
    assert _lib.call_rc(f, p, p, p, p, p, 128, 128, 128, 128, stream, sms + 1, 0) == 1  # too many SMs
    assert _lib.call_rc(f, p, p, p, p, p, 128, 128, 128, 128, stream, sms, 48) == 1     # unknown tile
    assert _lib.call_rc(f, p + 8, p, p, p, p, 128, 128, 128, 128, stream, sms, 0) == 1  # misaligned lhs
    assert _lib.call_rc(f, None, p, p, p, p, 128, 128, 128, 128, stream, sms, 0) == 1   # null
    assert _lib.call_rc(f, p, p, p, p, p, 0, 128, 128, 128, stream, sms, 0) == 1        # empty M


def test_host_front_end_pipelines_three_calls(cuda_lib):
    """HostFp8Linear: pinned host in, pinned host out, rotating device slots; each call checked against the oracle."""
    import yan_b200
    m, n, k = 192, 512, 1024
    _, b = ref.make_inputs(m, n, k, seed=40)
    rhs = ref.per_block_cast_to_fp8(b)
    pipe = yan_b200.HostFp8Linear((rhs[0].cuda(), rhs[1].cuda()), m, depth=2)
    ins, outs = [], []
    for i in range(3):
        a, _ = ref.make_inputs(m, 128, k, seed=41 + i)
        ins.append(a.pin_memory())
        outs.append(torch.empty(m, n, dtype=torch.bfloat16).pin_memory())
        pipe.submit(ins[-1], outs[-1])
    pipe.wait()
    for a, o in zip(ins, outs):
        _check(o, ref.ref_gemm(ref.per_token_cast_to_fp8(a), rhs), "host front end")


@pytest.mark.parametrize("num_sms", [148, 100])
def test_tail_cut_along_k_matches_oracle_and_whole_tile_kernel(cuda_lib, num_sms):
    """160 tiles of 128 x 256 on 148 (or 100) CTAs: the last wave would be nearly empty, so the automatic policy computes
    the full waves as whole tiles, cuts the remaining tiles along K across all CTAs (fp32 partial tiles in a workspace)
    and sums the partials in slice order.  Checked against the CPU oracle, against the whole-tile kernel (last-bit
    differences only), twice on the same workspace, and for run-to-run reproducibility."""
    import yan_b200
    from yan_b200.jit_kernels.utils import get_num_sms, set_num_sms
    m, n, k = 2048, 2560, 12288  # 96 k-blocks: the policy only cuts when K is long
    a, b = ref.make_inputs(m, n, k, seed=41)
    lhs, rhs = ref.per_token_cast_to_fp8(a), ref.per_block_cast_to_fp8(b)
    d_ref = ref.ref_gemm(lhs, rhs)
    lhs_d = (lhs[0].cuda(), lhs[1].t().contiguous().cuda().t())
    rhs_d = (rhs[0].cuda(), rhs[1].cuda())
    whole = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    yan_b200.gemm_fp8_fp8_bf16_nt(lhs_d, rhs_d, whole, block_n=256)
    sms_before = get_num_sms()
    try:
        set_num_sms(min(num_sms, sms_before))
        results = []
        for attempt in range(2):
            out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
            yan_b200.gemm_fp8_fp8_bf16_nt(lhs_d, rhs_d, out)
            torch.cuda.synchronize()
            assert yan_b200.read_device_status() == 0
            assert not torch.isnan(out.float()).any(), f"attempt {attempt}: a tile was never stored"
            assert ref.rel_frobenius(out.cpu(), d_ref) <= 1e-3
            assert ref.max_abs_err(out.cpu(), d_ref) <= ref.bf16_ulp_at(float(d_ref.float().abs().max()))
            assert ref.rel_frobenius(out.cpu(), whole.cpu()) <= 1e-4
            results.append(out)
        assert torch.equal(results[0], results[1])
    finally:
        set_num_sms(sms_before)
