"""Parity at the full benchmark sizes (C3, C4 and its 8-way N shard, C5's per-rank K shard).

The CPU oracle cannot multiply these shapes in seconds, so each case checks
  (1) sampled blocks: whole 128-row x 256-column tiles of D (the corners and seeded random ones, at least one per band
      of 16 m-blocks) against the oracle, computed from the same e4m3 codes and scales copied back from the device;
  (2) size-independent properties over the whole output: exact linearity in a power-of-two rescaling of the
      activation scales, and agreement of the full-K product with the fp32 sum of two half-K products.
Inputs are the seeded synthetic workloads (A ~ N(0,1), B ~ N(0,0.02)), generated and quantized on the device
with the kernels whose bit-exactness the quantizer tests establish.
"""
import pytest
import torch

from oracle import ref

pytestmark = pytest.mark.gpu

REL_FRO_TOL = 1e-3


def _device_operands(m, n, k, seed):
    import yan_b200
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn(m, k, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    b = (torch.randn(n, k, generator=g, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
    lhs = yan_b200.per_token_cast_to_fp8(a)
    rhs = yan_b200.per_block_cast_to_fp8(b)
    del a, b
    return lhs, rhs


def _check_sampled_blocks(lhs, rhs, d, m_tiles, n_tiles):
    for mt in m_tiles:
        rows = slice(mt * 128, mt * 128 + 128)
        qa = lhs[0][rows].cpu()
        sa = lhs[1][rows].cpu().contiguous()
        for nt in n_tiles:
            cols = slice(nt * 256, nt * 256 + 256)
            qb = rhs[0][cols].cpu()
            sb = rhs[1][nt * 2:nt * 2 + 2].cpu().contiguous()
            d_ref = ref.ref_gemm((qa, sa), (qb, sb))
            got = d[rows, cols].cpu()
            fro = ref.rel_frobenius(got, d_ref)
            assert fro <= REL_FRO_TOL, f"tile ({mt},{nt}): rel Frobenius {fro:.2e}"
            assert ref.max_abs_err(got, d_ref) <= ref.bf16_ulp_at(float(d_ref.float().abs().max())), f"tile ({mt},{nt})"


@pytest.mark.parametrize("name,m,n,k", [("C3", 4096, 7168, 18432), ("C4", 8192, 28672, 8192),
                                        ("C4/8 shard", 8192, 3584, 8192), ("C5/8 shard", 4096, 8192, 3584)])
def test_full_size_blocks_and_properties(cuda_lib, name, m, n, k):
    import yan_b200
    lhs, rhs = _device_operands(m, n, k, seed=len(name))
    d = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    yan_b200.gemm_fp8_fp8_bf16_nt(lhs, rhs, d)
    torch.cuda.synchronize()
    assert yan_b200.read_device_status() == 0
    assert bool(torch.isfinite(d.float()).all())
    # Sampled tiles: the four corners plus seeded random ones, one m-tile out of every band of 16 m-blocks the
    # scheduler sweeps (a fault confined to an interior band or an interior column panel would otherwise pass).
    m_blocks, n_blocks = m // 128, n // 256
    rng = torch.Generator().manual_seed(1000 + m + n + k)
    tiles = {(0, 0), (0, n_blocks - 1), (m_blocks - 1, 0), (m_blocks - 1, n_blocks - 1)}
    for band in range(0, m_blocks, 16):
        rows_in_band = min(16, m_blocks - band)
        mt = band + int(torch.randint(rows_in_band, (1,), generator=rng))
        tiles.add((mt, int(torch.randint(n_blocks, (1,), generator=rng))))
    while len(tiles) < 12:
        tiles.add((int(torch.randint(m_blocks, (1,), generator=rng)), int(torch.randint(n_blocks, (1,), generator=rng))))
    for mt, nt in sorted(tiles):
        _check_sampled_blocks(lhs, rhs, d, m_tiles=(mt,), n_tiles=(nt,))

    # linearity: doubling every activation scale doubles D exactly
    d2 = torch.empty_like(d)
    yan_b200.gemm_fp8_fp8_bf16_nt((lhs[0], lhs[1] * 2.0), rhs, d2)
    assert torch.equal(d2.float(), d.float() * 2.0)
    del d2

    # split consistency: D(full K) == D(first half of K) + D(second half), partials in fp32
    kh = (k // 256) * 128
    parts = []
    for k0, k1 in ((0, kh), (kh, k)):
        sl, ss = slice(k0, k1), slice(k0 // 128, k1 // 128)
        part = torch.empty(m, n, dtype=torch.float32, device="cuda")
        yan_b200.gemm_fp8_fp8_f32_nt((lhs[0][:, sl].contiguous(), lhs[1][:, ss].t().contiguous().t()),
                                     (rhs[0][:, sl].contiguous(), rhs[1][:, ss].contiguous()), part)
        parts.append(part)
    total = (parts[0] + parts[1]).to(torch.bfloat16)
    del parts
    diff = (total.float() - d.float())
    fro = float(diff.norm() / d.float().norm())
    assert fro <= REL_FRO_TOL, f"{name}: full-K vs split-K rel Frobenius {fro:.2e}"


def test_tile_widths_agree_bit_for_bit_at_full_size(cuda_lib):
    """Every tile width adds the same scaled k-block products in the same order, so the C4 shard of an 8-GPU job must
    come out identical from the 256-wide tiles and from the 224-wide ones (two B scales per warpgroup, 16-column tail
    chunk, last tile partly beyond N for 192)."""
    import yan_b200
    m, n, k = 8192, 3584, 8192
    lhs, rhs = _device_operands(m, n, k, seed=11)
    want = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    yan_b200.gemm_fp8_fp8_bf16_nt(lhs, rhs, want, block_n=256)
    for block_n in (224, 192, 160, 128):
        got = torch.empty_like(want)
        yan_b200.gemm_fp8_fp8_bf16_nt(lhs, rhs, got, block_n=block_n)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"block_n={block_n}"
    assert yan_b200.read_device_status() == 0
