"""Host-side logic of the sharded GEMMs on CPU ranks (gloo, world size 2): shard slicing, reassembly and the
allreduce of partials.  The arithmetic is substituted by the CPU oracle through `gemm_fn`; the CUDA kernels are
covered by the GPU tests."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_gemm(lhs, rhs, out):
    from oracle import ref
    qa, sa = lhs
    d = ref.ref_gemm_f32((qa.contiguous(), sa.contiguous()), (rhs[0].contiguous(), rhs[1].contiguous()))
    out.copy_(d.to(out.dtype))


def _worker(rank: int, world: int, port: int, mode: str, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import ref
        from yan_b200.comm import gemm_allreduce as ga
        torch.set_num_threads(2)
        m, n, k = 160, 512, 1024
        a, b = ref.make_inputs(m, n, k, seed=3)
        lhs, rhs = ref.per_token_cast_to_fp8(a), ref.per_block_cast_to_fp8(b)
        d_ref = ref.ref_gemm(lhs, rhs)
        if mode == "n_split":
            full = torch.zeros(m, n, dtype=torch.bfloat16)
            ga.gemm_n_split(lhs, ga.shard_n(rhs, rank, world), full, rank, world, gemm_fn=_oracle_gemm)
            ns = n // world
            assert bool((full[:, :rank * ns] == 0).all()) and bool((full[:, (rank + 1) * ns:] == 0).all())
            dist.all_reduce(full_f := full.float())                     # test-only reassembly of the column slices
            ok = ref.rel_frobenius(full_f.to(torch.bfloat16), d_ref) <= 1e-3
            own = torch.empty(m, ns, dtype=torch.bfloat16)
            ga.gemm_n_split(lhs, ga.shard_n(rhs, rank, world), own, rank, world, gemm_fn=_oracle_gemm)
            ok = ok and torch.equal(own, full[:, rank * ns:(rank + 1) * ns])
        elif mode == "k_split_f32":
            # quantize the local K shard of A: equals the shard of the quantized A
            ks = k // world
            lhs_local = ref.per_token_cast_to_fp8(a[:, rank * ks:(rank + 1) * ks].contiguous())
            sh = ga.shard_k(lhs, rank, world)
            assert torch.equal(lhs_local[0].view(torch.uint8), sh[0].view(torch.uint8)) and torch.equal(lhs_local[1], sh[1])
            out = torch.empty(m, n, dtype=torch.bfloat16)
            ga.gemm_k_split_allreduce(lhs_local, ga.shard_k(rhs, rank, world), out, partial_dtype=torch.float32,
                                      num_chunks=2, gemm_fn=_oracle_gemm)
            ok = ref.rel_frobenius(out, d_ref) <= 1e-3
        elif mode == "k_split_bf16":
            out = torch.empty(m, n, dtype=torch.bfloat16)
            ga.gemm_k_split_allreduce(ga.shard_k(lhs, rank, world), ga.shard_k(rhs, rank, world), out,
                                      partial_dtype=torch.bfloat16, gemm_fn=_oracle_gemm)
            d_split = ref.ref_gemm_k_split(lhs, rhs, world)
            ok = ref.rel_frobenius(out, d_split) <= 2e-3 and ref.rel_frobenius(out, d_ref) <= 6e-3
        elif mode == "k_split_two_shot_host":
            # the orchestration of the peer-memory path with a stand-in communicator: fp32 sum in rank order, one rounding
            class HostComm:
                def __init__(self):
                    self.m, self.n = m, n
                    self.buffer = torch.zeros(m, n, dtype=torch.bfloat16)
                    self.calls = []

                def reduce_rows(self, r0=0, r1=None, num_ctas=None, exclusive_sms=False):
                    self.calls.append((r0, r1))
                    parts = [torch.empty(r1 - r0, n) for _ in range(world)]
                    dist.all_gather(parts, self.buffer[r0:r1].float())
                    acc = torch.zeros(r1 - r0, n)
                    for part in parts:
                        acc += part
                    self.buffer[r0:r1] = acc.to(torch.bfloat16)

            comm = HostComm()
            res = ga.gemm_k_split_two_shot(ga.shard_k(lhs, rank, world), ga.shard_k(rhs, rank, world), comm,
                                           gemm_fn=_oracle_gemm)
            ok = res is comm.buffer and comm.calls == [(0, m)]
            ok = ok and ref.rel_frobenius(res, ref.ref_gemm_k_split(lhs, rhs, world)) <= 2e-3
        elif mode in ("peer_export_failure", "peer_open_failure"):
            # One rank cannot export (or cannot map a peer's) buffer: every rank must raise, with that rank's message,
            # and none may be left waiting in a collective.  The C calls are replaced by stand-ins; no GPU involved.
            from yan_b200 import _lib
            from yan_b200.comm import peer_memory

            def fake_call(name, *args):
                if name == "yan_b200_ipc_export" and mode == "peer_export_failure" and rank == 1:
                    raise _lib.YanB200Error(name, 5, "collective library reported an error")
                if name == "yan_b200_ipc_open" and mode == "peer_open_failure" and rank == 0:
                    raise _lib.YanB200Error(name, 5, "collective library reported an error")

            peer_memory._lib.call = fake_call
            try:
                peer_memory.PeerSharedTensor((64,), torch.uint8, device="cpu")
                ok = False
            except RuntimeError as e:
                culprit = "rank 1" if mode == "peer_export_failure" else "rank 0 mapping rank 1"
                ok = culprit in str(e) and not peer_memory._opened
        elif mode == "rank_failure":
            # A rank that raises before the collective: the survivor's allreduce must end with an error, not hang.
            if rank == 1:
                raise RuntimeError("injected host-side failure before the allreduce")
            out = torch.empty(m, n, dtype=torch.bfloat16)
            try:
                ga.gemm_k_split_allreduce(ga.shard_k(lhs, rank, world), ga.shard_k(rhs, rank, world), out,
                                          partial_dtype=torch.float32, gemm_fn=_oracle_gemm)
                ok = False
            except Exception:
                ok = True
        else:
            ok = False
        results[rank] = bool(ok)
    finally:
        if mode != "rank_failure":
            dist.destroy_process_group()


def _run(mode: str, expect_all: bool = True):
    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        if p.is_alive():
            p.terminate()
            pytest.fail(f"{mode}: rank did not finish")
    return dict(results), [p.exitcode for p in procs]


@pytest.mark.parametrize("mode", ["n_split", "k_split_f32", "k_split_bf16", "k_split_two_shot_host"])
def test_sharded_gemm_world2_gloo(mode):
    results, codes = _run(mode)
    assert codes == [0, 0], codes
    assert results == {0: True, 1: True}, results


@pytest.mark.parametrize("mode", ["peer_export_failure", "peer_open_failure"])
def test_peer_memory_setup_fails_on_every_rank_together(mode):
    results, codes = _run(mode)
    assert codes == [0, 0], codes
    assert results == {0: True, 1: True}, results


def test_rank_failure_surfaces_as_error_not_hang():
    results, codes = _run("rank_failure")
    assert codes[1] != 0                    # the failing rank exits with its exception
    assert results.get(0) is True           # the survivor saw an error from the collective


def test_shard_helpers_reject_ragged_cuts():
    from yan_b200.comm import gemm_allreduce as ga
    q = torch.zeros(384, 256, dtype=torch.uint8)
    s = torch.zeros(3, 2)
    with pytest.raises(AssertionError):
        ga.shard_n((q, s), 0, 2)            # 384 / 2 = 192 rows: not whole 128-row blocks
    with pytest.raises(AssertionError):
        ga.shard_k((q, s), 0, 4)            # 256 / 4 = 64 columns: not whole k-blocks
    qs, ss = ga.shard_k((q, s), 1, 2)
    assert qs.shape == (384, 128) and ss.shape == (3, 1)


def test_two_shot_slices_partition_the_range():
    """Every 16-byte vector of the range is reduced by exactly one rank, for ranges that do not divide evenly too."""
    from yan_b200.comm import slice_bounds
    for world in range(2, 9):
        for count in (1, 7, 8, 9, 1000, 4096 * 8192 // 8):
            covered = []
            for rank in range(world):
                first, last = slice_bounds(count, world, rank)
                assert 0 <= first <= last <= count
                covered.append((first, last))
            assert covered[0][0] == 0 and covered[-1][1] == count
            assert all(covered[i][1] == covered[i + 1][0] for i in range(world - 1))


class _ModelRank:
    """Device half of one rank's ordering state as the allreduce kernels keep it (PeerSignals in
    include/comm/peer_allreduce.cuh), reduced to what the bookkeeping needs: a cumulative CTA counter and the epoch it
    has published as done.  `timed_out` models a launch whose entry wait ran out on every CTA."""

    def __init__(self):
        self.cta_counter = 0
        self.done_epoch = 0

    def launch(self, epoch, counter_target, ctas, timed_out=False, counts_on_timeout=True):
        published = False
        for _ in range(ctas):
            if timed_out and not counts_on_timeout:
                continue  # the old behaviour: a CTA that gave up at entry returned without counting itself
            self.cta_counter = (self.cta_counter + 1) & 0xFFFFFFFF
            if self.cta_counter == counter_target:
                self.done_epoch = epoch
                published = True
        return published


def test_collective_clock_survives_a_timed_out_launch():
    from yan_b200.comm.peer_memory import CollectiveClock
    clock, device = CollectiveClock(), _ModelRank()
    assert device.launch(*clock.next_launch(148), 148)
    # a launch whose entry wait ran out still counts its CTAs and publishes its epoch ...
    assert device.launch(*clock.next_launch(24), 24, timed_out=True)
    # ... so the launches after it reach their targets again
    for ctas in (148, 7, 64):
        epoch, target = clock.next_launch(ctas)
        assert device.launch(epoch, target, ctas) and device.done_epoch == epoch
    assert device.cta_counter == clock.cta_count

    # the behaviour this replaces: the counter falls behind for good and no later launch publishes
    clock, device = CollectiveClock(), _ModelRank()
    device.launch(*clock.next_launch(24), 24, timed_out=True, counts_on_timeout=False)
    assert not device.launch(*clock.next_launch(24), 24)

    # reset() starts both halves over (the device half is zeroed by TwoShotAllreduce.reset)
    clock.reset()
    device = _ModelRank()
    epoch, target = clock.next_launch(5)
    assert (epoch, target) == (1, 5) and device.launch(epoch, target, 5)


def test_collective_clock_wraps_without_using_epoch_zero():
    from yan_b200.comm.peer_memory import CollectiveClock
    clock = CollectiveClock()
    clock.epoch = 0xFFFFFFFF
    clock.cta_count = 0xFFFFFFF0
    epoch, target = clock.next_launch(32)
    assert epoch == 1 and target == 0x10
