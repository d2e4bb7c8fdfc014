"""Grouped FP8 GEMMs (contiguous and masked layouts) against the CPU oracle, group by group."""
import pytest
import torch

from oracle import ref

pytestmark = pytest.mark.gpu


def _col_major(s):
    return s.t().contiguous().t()


@pytest.mark.parametrize("block_n", [0, 128, 256])
def test_contiguous_layout(cuda_lib, block_n):
    import yan_b200
    g, n, k = 3, 512, 1024
    rows = [256, 128, 384]                      # each a multiple of the 128-row alignment
    m = sum(rows) + 128                         # one trailing padding tile (group -1)
    gen = torch.Generator().manual_seed(17)
    a = torch.randn(m, k, generator=gen).to(torch.bfloat16)
    b = (torch.randn(g, n, k, generator=gen) * 0.02).to(torch.bfloat16)
    lhs = ref.per_token_cast_to_fp8(a)
    rhs_list = [ref.per_block_cast_to_fp8(b[i]) for i in range(g)]
    rhs_q = torch.stack([r[0].view(torch.uint8) for r in rhs_list]).view(torch.float8_e4m3fn)
    rhs_s = torch.stack([r[1] for r in rhs_list])
    m_indices = torch.full((m,), -1, dtype=torch.int32)
    r0 = 0
    for i, r in enumerate(rows):
        m_indices[r0:r0 + r] = i
        r0 += r
    out = torch.full((m, n), 5.0, dtype=torch.bfloat16, device="cuda")
    yan_b200.m_grouped_gemm_fp8_fp8_bf16_nt_contiguous((lhs[0].cuda(), _col_major(lhs[1]).cuda().t().contiguous().t()),
                                                       (rhs_q.cuda(), rhs_s.cuda()), out, m_indices.cuda(), block_n=block_n)
    torch.cuda.synchronize()
    assert yan_b200.read_device_status() == 0
    out = out.cpu()
    r0 = 0
    for i, r in enumerate(rows):
        d_ref = ref.ref_gemm((lhs[0][r0:r0 + r], lhs[1][r0:r0 + r]), rhs_list[i])
        assert ref.rel_frobenius(out[r0:r0 + r], d_ref) <= 1e-3, f"group {i}"
        r0 += r
    assert bool((out[r0:] == 5.0).all()), "padding rows must stay untouched"


@pytest.mark.parametrize("block_n", [0, 256])
def test_masked_layout(cuda_lib, block_n):
    import yan_b200
    g, m_max, n, k = 4, 256, 384, 512
    masked = [256, 1, 130, 0]
    gen = torch.Generator().manual_seed(23)
    a = torch.randn(g, m_max, k, generator=gen).to(torch.bfloat16)
    b = (torch.randn(g, n, k, generator=gen) * 0.02).to(torch.bfloat16)
    lhs_list = [ref.per_token_cast_to_fp8(a[i]) for i in range(g)]
    rhs_list = [ref.per_block_cast_to_fp8(b[i]) for i in range(g)]
    lhs_q = torch.stack([l[0].view(torch.uint8) for l in lhs_list]).view(torch.float8_e4m3fn)
    lhs_s = torch.stack([l[1].contiguous() for l in lhs_list])          # [G, M_max, K/128]
    rhs_q = torch.stack([r[0].view(torch.uint8) for r in rhs_list]).view(torch.float8_e4m3fn)
    rhs_s = torch.stack([r[1] for r in rhs_list])
    out = torch.full((g, m_max, n), 9.0, dtype=torch.bfloat16, device="cuda")
    yan_b200.m_grouped_gemm_fp8_fp8_bf16_nt_masked((lhs_q.cuda(), lhs_s.cuda()), (rhs_q.cuda(), rhs_s.cuda()), out,
                                                   torch.tensor(masked, dtype=torch.int32).cuda(), block_n=block_n)
    torch.cuda.synchronize()
    assert yan_b200.read_device_status() == 0
    out = out.cpu()
    for i in range(g):
        mm = masked[i]
        if mm:
            d_ref = ref.ref_gemm((lhs_list[i][0][:mm], lhs_list[i][1][:mm]), rhs_list[i])
            assert ref.rel_frobenius(out[i, :mm], d_ref) <= 1e-3, f"group {i}"
        assert bool((out[i, mm:] == 9.0).all()), f"group {i}: rows beyond masked_m must stay untouched"


def test_masked_layout_clamps_row_counts(cuda_lib):
    """masked_m lives in device memory where no host check can see it: a count above M_max computes the whole group
    and nothing beyond it, a negative one computes nothing."""
    import yan_b200
    g, m_max, n, k = 4, 256, 256, 256
    masked = [256, 300, -5, 256]
    effective = [256, 256, 0, 256]
    gen = torch.Generator().manual_seed(29)
    a = torch.randn(g, m_max, k, generator=gen).to(torch.bfloat16)
    b = (torch.randn(g, n, k, generator=gen) * 0.02).to(torch.bfloat16)
    lhs_list = [ref.per_token_cast_to_fp8(a[i]) for i in range(g)]
    rhs_list = [ref.per_block_cast_to_fp8(b[i]) for i in range(g)]
    lhs_q = torch.stack([l[0].view(torch.uint8) for l in lhs_list]).view(torch.float8_e4m3fn)
    lhs_s = torch.stack([l[1].contiguous() for l in lhs_list])
    rhs_q = torch.stack([r[0].view(torch.uint8) for r in rhs_list]).view(torch.float8_e4m3fn)
    rhs_s = torch.stack([r[1] for r in rhs_list])
    # one guard group behind the output: it must come back untouched
    storage = torch.full((g + 1, m_max, n), 9.0, dtype=torch.bfloat16, device="cuda")
    out = storage[:g]
    yan_b200.m_grouped_gemm_fp8_fp8_bf16_nt_masked((lhs_q.cuda(), lhs_s.cuda()), (rhs_q.cuda(), rhs_s.cuda()), out,
                                                   torch.tensor(masked, dtype=torch.int32).cuda())
    torch.cuda.synchronize()
    assert yan_b200.read_device_status() == 0
    got = storage.cpu()
    assert bool((got[g] == 9.0).all()), "rows behind the last group were written"
    for i in range(g):
        mm = effective[i]
        if mm:
            d_ref = ref.ref_gemm((lhs_list[i][0][:mm], lhs_list[i][1][:mm]), rhs_list[i])
            assert ref.rel_frobenius(got[i, :mm], d_ref) <= 1e-3, f"group {i}"
        assert bool((got[i, mm:] == 9.0).all()), f"group {i}"
