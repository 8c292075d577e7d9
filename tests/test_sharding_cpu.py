"""Multi-GPU host logic on CPU: unit partitioning, halo planning, and the halo exchange itself run
as two gloo ranks (the same code path NCCL takes on GPUs)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from natten_b200 import sharding
from natten_b200.functional import window_end, window_start


def test_unit_ranges_cover_everything_once():
    for n, world in [(64, 1), (64, 8), (24, 8), (10, 4), (7, 3)]:
        seen = []
        for r in range(world):
            lo, hi = sharding.unit_range(n, world, r)
            seen += list(range(lo, hi))
        assert seen == list(range(n))


def test_shard_batch_heads_blocks():
    # config 2: B=4, H=16
    assert sharding.shard_batch_heads(4, 16, 1, 0) == (slice(0, 4), slice(0, 16))
    assert sharding.shard_batch_heads(4, 16, 4, 3) == (slice(3, 4), slice(0, 16))
    assert sharding.shard_batch_heads(4, 16, 8, 5) == (slice(2, 3), slice(8, 16))
    # config 5: B=1, H=24 over 8 ranks -> 3 heads each
    assert sharding.shard_batch_heads(1, 24, 8, 7) == (slice(0, 1), slice(21, 24))
    with pytest.raises(ValueError):
        sharding.shard_batch_heads(1, 24, 5, 0)


@pytest.mark.parametrize("extent,world,k,s,causal", [
    (32, 8, 16, 1, True),      # config 5's T axis: 15 frames before the slab, none after
    (32, 4, 16, 1, True), (32, 2, 16, 1, True),
    (40, 4, 7, 1, False), (37, 3, 8, 4, False), (64, 8, 9, 3, True),
])
@pytest.mark.parametrize("balanced", [False, True])
def test_halo_plan_covers_every_window(extent, world, k, s, causal, balanced):
    plan = sharding.make_halo_plan(extent, world, k, s, causal, balanced=balanced)
    assert plan.slabs[0][0] == 0 and plan.slabs[-1][1] == extent
    assert all(plan.slabs[r][1] == plan.slabs[r + 1][0] for r in range(world - 1))
    for r, (t0, t1) in enumerate(plan.slabs):
        lo, hi = plan.needs[r]
        for i in range(t0, t1):
            st = window_start(i, k, s, extent, causal)
            en = window_end(i, st, k, extent, causal)
            assert lo <= st and en <= hi
        # tight: the first / last needed frame is really used
        assert lo == window_start(t0, k, s, extent, causal)
        # every needed frame outside the slab arrives from exactly its owner
        got = set(range(t0, t1))
        for src, (a, b) in plan.recv_list(r):
            assert plan.slabs[src][0] <= a < b <= plan.slabs[src][1]
            assert not (got & set(range(a, b)))
            got |= set(range(a, b))
        assert got == set(range(lo, hi))
    if (extent, world, k, s, causal, balanced) == (32, 8, 16, 1, True, False):
        # a causal window of 16 reaches 15 frames back, not kernel_size / 2
        assert plan.needs[4] == (16 - 15, 20)
        assert plan.halo_frames(4) == 15 and plan.halo_frames(0) == 0


def test_balanced_slabs_equalise_the_work_of_a_causal_axis():
    """Config 5's T axis over two ranks: frames 0..15 have windows of 1..16 key frames, the rest
    16 each (392 in all); equal-length slabs give 136 / 256, balanced ones 200 / 192."""
    def work(t0, t1):
        return sum(window_end(t, window_start(t, 16, 1, 32, True), 16, 32, True)
                   - window_start(t, 16, 1, 32, True) for t in range(t0, t1))
    even = sharding.make_halo_plan(32, 2, 16, 1, True).slabs
    bal = sharding.make_halo_plan(32, 2, 16, 1, True, balanced=True, align=2).slabs
    assert [work(*x) for x in even] == [136, 256]
    assert bal == [(0, 20), (20, 32)] and [work(*x) for x in bal] == [200, 192]
    # boundaries respect the alignment, every rank keeps at least one aligned block
    for world in (2, 4, 8):
        slabs = sharding.make_halo_plan(32, world, 16, 1, True, balanced=True, align=2).slabs
        assert all(a % 2 == 0 and b > a for a, b in slabs)
        assert max(work(*x) for x in slabs) <= max(work(*x) for x in
                                                   sharding.make_halo_plan(32, world, 16, 1, True).slabs)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _exchange_worker(rank, world, port, extent, k, s, causal, batch, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        K = torch.randn(batch, extent, 3, 5, 2, 4)
        V = torch.randn(batch, extent, 3, 5, 2, 4)
        plan = sharding.make_halo_plan(extent, world, k, s, causal)
        t0, t1 = plan.slabs[rank]
        ks, vs, lo = sharding.exchange_halo(K[:, t0:t1].contiguous(), V[:, t0:t1].contiguous(),
                                            plan, rank)
        lo2, hi2 = plan.needs[rank]
        ok = lo == lo2 and torch.equal(ks, K[:, lo2:hi2]) and torch.equal(vs, V[:, lo2:hi2])
        # the non-blocking form used by the overlapped path: received blocks only, own frames
        # are not copied
        parts, reqs, keep = sharding.exchange_halo_parts(K[:, t0:t1].contiguous(),
                                                         V[:, t0:t1].contiguous(), plan, rank)
        for r in reqs:
            r.wait()
        covered = set()
        for kp, vp, first in parts:
            n = kp.shape[1]
            ok = ok and torch.equal(kp, K[:, first:first + n]) and torch.equal(vp, V[:, first:first + n])
            covered |= set(range(first, first + n))
        ok = ok and covered == set(range(lo2, hi2)) - set(range(t0, t1))
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("extent,k,s,causal,batch", [(16, 6, 1, True, 1), (18, 5, 2, False, 2)])
def test_halo_exchange_two_gloo_ranks(extent, k, s, causal, batch):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_exchange_worker,
                         args=(r, world, port, extent, k, s, causal, batch, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]
