"""The multi-GPU host logic on CPU: two gloo ranks each take their shard of one seeded problem, run it (here
through the CPU oracle, standing in for the per-GPU operator), and the gathered pieces equal the unsharded
result; per-rank times reduce to their max."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flash_pop_b200.parallel import max_over_ranks, partition
from oracle import retention_oracle as orc


def test_partition_covers_every_pair_once():
    for B, H, world in ((8, 16, 2), (8, 16, 8), (3, 4, 2), (1, 16, 8), (2, 3, 8), (5, 2, 4), (0, 4, 2)):
        seen = torch.zeros(B, H, dtype=torch.int32)
        for r in range(world):
            s = partition(B, H, r, world)
            seen[s.batch, s.heads] += 1
        assert (seen == 1).all(), (B, H, world, seen)
    with pytest.raises(ValueError):
        partition(4, 4, 2, 2)


def _worker(rank, world, port, case, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, T, H, dk, dv = case
        g = torch.Generator().manual_seed(0)            # every rank builds the same global tensors
        q, k = (torch.randn(B, T, H, dk, generator=g, dtype=torch.float64) for _ in range(2))
        v = torch.randn(B, T, H, dv, generator=g, dtype=torch.float64)
        s0 = torch.randn(B, H, dk, dv, generator=g, dtype=torch.float64)
        decays = orc.head_decays(H, (5, 12))
        sh = partition(B, H, rank, world)
        o_full = torch.zeros(B, T, H, dv, dtype=torch.float64)
        s_full = torch.zeros(B, H, dk, dv, dtype=torch.float64)
        if sh.batch.stop > sh.batch.start and sh.heads.stop > sh.heads.start:
            o, s = orc.retention_chunkwise(sh.take_seq(q), sh.take_seq(k), sh.take_seq(v), sh.take_state(s0),
                                           sh.take_decays(decays), 64)
            o_full[sh.batch, :, sh.heads] = o
            s_full[sh.batch, sh.heads] = s
        dist.all_reduce(o_full), dist.all_reduce(s_full)   # disjoint pieces: the sum is the concatenation
        slowest = max_over_ranks(10.0 + rank)
        if rank == 0:
            o_ref, s_ref = orc.retention_chunkwise(q, k, v, s0, decays, 64)
            out.put((torch.allclose(o_full, o_ref, atol=1e-12), torch.allclose(s_full, s_ref, atol=1e-12), slowest))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("case", [(4, 70, 3, 8, 8), (1, 40, 4, 8, 16)])
def test_two_ranks_reproduce_the_unsharded_result(case):
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = 29500 + (os.getpid() + case[0]) % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, case, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    o_ok, s_ok, slowest = out.get()
    assert o_ok and s_ok and slowest == 11.0


def _failing_worker(rank, world, port, out):
    """Rank 1 fails on the host before the gradient all-reduce; rank 0 must get an error out of its collective
    within the process-group timeout instead of waiting for ever."""
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    dist.barrier()                                     # both ranks are up
    if rank == 1:
        os._exit(0)                                    # dies between steps, nothing of its own in flight
    t0 = time.time()
    try:
        dist.all_reduce(torch.ones(4))
        out.put(("no error", time.time() - t0))
    except Exception as e:                             # gloo reports the lost peer or the timeout
        out.put((type(e).__name__, time.time() - t0))
    os._exit(0)                                        # the group is broken: leave without the collective teardown


def test_a_lost_rank_ends_the_survivors_collective_with_an_error():
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    kind, waited = out.get()
    assert kind != "no error" and waited < 30, (kind, waited)
