"""Sharded GEMMs on real GPUs over NCCL (needs at least two visible devices; skipped on a one-GPU box)."""
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import yan_b200
        from oracle import ref
        from yan_b200.comm import gemm_allreduce as ga
        m, n, k = 512, 1024, 2048
        a, b = ref.make_inputs(m, n, k, seed=3)
        lhs, rhs = ref.per_token_cast_to_fp8(a), ref.per_block_cast_to_fp8(b)
        d_ref = ref.ref_gemm(lhs, rhs)
        cm = lambda op: (op[0].contiguous().cuda(), op[1].t().contiguous().cuda().t())
        rm = lambda op: (op[0].contiguous().cuda(), op[1].contiguous().cuda())
        ok = True
        # N-split into the full buffer, then gather the slices for the check only
        full = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
        ga.gemm_n_split(cm(lhs), rm(ga.shard_n(rhs, rank, world)), full, rank, world)
        dist.all_reduce(full)
        ok &= ref.rel_frobenius(full.cpu(), d_ref) <= 1e-3
        # K-split: local quantization of the A shard, bf16 partials and fp32 partials, chunked
        ks = k // world
        lhs_local = yan_b200.per_token_cast_to_fp8(a[:, rank * ks:(rank + 1) * ks].contiguous().cuda())
        rhs_k = rm(ga.shard_k(rhs, rank, world))
        out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        ga.gemm_k_split_allreduce(lhs_local, rhs_k, out, partial_dtype=torch.bfloat16, num_chunks=2)
        torch.cuda.synchronize()
        ok &= ref.rel_frobenius(out.cpu(), ref.ref_gemm_k_split(lhs, rhs, world)) <= 2e-3
        ga.gemm_k_split_allreduce(lhs_local, rhs_k, out, partial_dtype=torch.float32, num_chunks=4)
        torch.cuda.synchronize()
        ok &= ref.rel_frobenius(out.cpu(), d_ref) <= 1e-3
        ok &= yan_b200.read_device_status() == 0
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_n_split_and_k_split_over_nccl(cuda_lib):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    env = dict(NCCL_NVLS_ENABLE="0")
    os.environ.update(env)
    procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        assert not p.is_alive(), "rank did not finish"
    assert [p.exitcode for p in procs] == [0, 0]
    assert dict(results) == {0: True, 1: True}


def _two_shot_worker(rank, world, port, results):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import yan_b200
        from oracle import ref
        from yan_b200.comm import TwoShotAllreduce, gemm_allreduce as ga
        m, n, k = 512, 1024, 2048
        checks = {}

        def same(got, want, exact):
            # The peer kernel adds in fp32 in rank order and rounds once (reproducible bit for bit); the switch's adder
            # is only required to be within one bf16 step of that.
            if exact:
                return bool(torch.equal(got, want))
            err = (got.float() - want.float()).abs()
            return bool((err <= want.float().abs() * 2.0 ** -7 + 1e-30).all())

        for device_barriers, in_switch in ((True, False), (False, False), (True, True)):
            tag = f"barriers={device_barriers},in_switch={in_switch}"
            comm = TwoShotAllreduce(m, n, device_barriers=device_barriers, in_switch=in_switch)
            # 1. the collective alone: every rank can reproduce every rank's input from its seed
            parts = []
            for r in range(world):
                g = torch.Generator(device="cuda").manual_seed(100 + r)
                parts.append(torch.randn(m, n, generator=g, device="cuda").to(torch.bfloat16))
            want = torch.zeros(m, n, device="cuda")
            for part in parts:
                want += part.float()
            want = want.to(torch.bfloat16)
            comm.buffer.copy_(parts[rank])
            comm.reduce_rows()
            torch.cuda.synchronize()
            checks[f"{tag}: whole tensor"] = same(comm.buffer, want, not in_switch)
            # 2. a row range only: the rows outside keep this rank's own values
            comm.buffer.copy_(parts[rank])
            comm.reduce_rows(128, 384, num_ctas=7)
            torch.cuda.synchronize()
            checks[f"{tag}: row range"] = same(comm.buffer[128:384], want[128:384], not in_switch)
            checks[f"{tag}: rows outside untouched"] = bool(
                torch.equal(comm.buffer[:128], parts[rank][:128]) and torch.equal(comm.buffer[384:], parts[rank][384:]))
            # 3. the K-split GEMM on top of it, whole and in two overlapped row chunks
            a, b = ref.make_inputs(m, n, k, seed=3)
            lhs, rhs = ref.per_token_cast_to_fp8(a), ref.per_block_cast_to_fp8(b)
            ks = k // world
            lhs_local = yan_b200.per_token_cast_to_fp8(a[:, rank * ks:(rank + 1) * ks].contiguous().cuda())
            rhs_k = tuple(t.contiguous().cuda() for t in ga.shard_k(rhs, rank, world))
            d_split = ref.ref_gemm_k_split(lhs, rhs, world)
            nccl = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
            ga.gemm_k_split_allreduce(lhs_local, rhs_k, nccl, partial_dtype=torch.bfloat16)
            for chunks in (1, 2):
                out = ga.gemm_k_split_two_shot(lhs_local, rhs_k, comm, num_chunks=chunks)
                torch.cuda.synchronize()
                # the switch's adder does not round to nearest (measured: ~3e-3 against the round-to-nearest sum)
                tol = 6e-3 if in_switch else 2e-3
                checks[f"{tag}: K-split {chunks} chunk(s) vs oracle"] = ref.rel_frobenius(out.cpu(), d_split) <= tol
                if world == 2 and not in_switch:  # the sum of two bf16 numbers rounded once: the same whoever adds them
                    checks[f"{tag}: K-split {chunks} chunk(s) vs NCCL"] = bool(torch.equal(out, nccl))
            checks[f"{tag}: status"] = yan_b200.read_device_status() == 0
            comm.close()
        # the tile-fused form (reduce-scatter in the GEMM epilogue, all-gather kernel): same sum as the two-shot kernel
        from yan_b200.comm import TileFusedAllreduce
        partial = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        yan_b200.gemm_fp8_fp8_bf16_nt(lhs_local, rhs_k, partial, block_n=256)
        gathered = [torch.empty_like(partial) for _ in range(world)]
        dist.all_gather(gathered, partial)
        acc = torch.zeros(m, n, dtype=torch.float32, device="cuda")
        for g in gathered:
            acc += g.float()
        fused = TileFusedAllreduce(m, n)
        for call in range(3):
            got = fused.gemm_and_reduce(lhs_local, rhs_k)
            torch.cuda.synchronize()
            checks[f"tile-fused call {call}: equals the fp32 rank-order sum"] = bool(torch.equal(got, acc.to(torch.bfloat16)))
            checks[f"tile-fused call {call}: vs oracle"] = ref.rel_frobenius(got.cpu(), d_split) <= 2e-3
        checks["tile-fused: status"] = yan_b200.read_device_status() == 0
        fused.close()
        results[rank] = {name: bool(v) for name, v in checks.items()}
    finally:
        dist.destroy_process_group()


def test_two_shot_peer_allreduce_and_k_split(cuda_lib):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    os.environ.update(NCCL_NVLS_ENABLE="0")
    procs = [ctx.Process(target=_two_shot_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        assert not p.is_alive(), "rank did not finish"
    assert [p.exitcode for p in procs] == [0, 0]
    failed = {r: [name for name, v in dict(results[r]).items() if not v] for r in range(world)}
    assert failed == {0: [], 1: []}, failed
    assert len(dict(results[0])) >= 20
