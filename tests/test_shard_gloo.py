"""Multi-rank host logic on CPU: two gloo ranks shard the sequences and reduce their statistics."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from subspec_b200.shard import reduce_stats, shard_sequences


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sh = shard_sequences(512, world, rank, 64)
        ids = [i for w in range(sh.n_waves) for i in sh.wave_ids(w)]
        stats = reduce_stats({"ms_total": 10.0 + rank, "ms_kernel": 1.0 - 0.1 * rank},
                             {"accepted": float(len(ids)), "first": float(ids[0])})
        gathered = [None] * world
        dist.all_gather_object(gathered, ids)
        out.put((rank, sh.total, stats, gathered))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_two_ranks_partition_and_reduce(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, total, stats, gathered in results:
        assert total == 512
        every = sorted(i for ids in gathered for i in ids)
        assert every == list(range(512))                      # a partition: nothing lost, nothing twice
        assert stats["ms_total"] == 10.0 + (world - 1)          # max over ranks
        assert stats["ms_kernel"] == 1.0                        # max over ranks
        assert stats["accepted"] == 512.0                       # sum over ranks
        assert stats["first"] == sum(r * (512 // world) for r in range(world))


def test_sharding_edges():
    sh = shard_sequences(512, 8, 3, 64)
    assert (sh.first, sh.count, sh.n_waves, sh.total) == (192, 64, 1, 512)
    sh = shard_sequences(100, 3, 2, 64)   # 33 per rank -> wave shrinks to 33
    assert (sh.count, sh.wave, sh.total) == (33, 33, 99)
    sh = shard_sequences(512, 1, 0, 64)
    assert sh.n_waves == 8 and sh.wave_ids(7)[-1] == 511
    with pytest.raises(ValueError):
        shard_sequences(4, 8, 0, 64)
    with pytest.raises(IndexError):
        sh.wave_ids(8)
    assert reduce_stats({"a": 1.0}, {"b": 2.0}) == {"a": 1.0, "b": 2.0}   # not distributed: identity


def test_ranks_are_spread_over_the_box():
    from subspec_b200.shard import device_for_rank

    assert [device_for_rank(r, 8, 8) for r in range(8)] == list(range(8))
    assert [device_for_rank(r, 4, 8) for r in range(4)] == [0, 2, 4, 6]
    assert [device_for_rank(r, 2, 8) for r in range(2)] == [0, 4]
    assert device_for_rank(0, 1, 8) == 0
    assert [device_for_rank(r, 2, 2) for r in range(2)] == [0, 1]
    assert [device_for_rank(r, 3, 8) for r in range(3)] == [0, 2, 4]
    with pytest.raises(ValueError):
        device_for_rank(2, 2, 8)
