"""The N>1 path of the benchmark on CPU: two gloo ranks shard the streams, time a fake step and
agree on the whole-job number (sum of work over the slowest rank)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from breeze_tts_cpp_b200.sharding import shard_streams, whole_job_rate


def test_shards_are_disjoint_and_cover():
    for total in (64, 63, 7, 1, 0):
        for world in (1, 2, 4, 8):
            owned = []
            for rank in range(world):
                first, count = shard_streams(total, world, rank)
                owned += list(range(first, first + count))
            assert owned == list(range(total))
    assert shard_streams(64, 8, 3) == (24, 8)
    with pytest.raises(ValueError):
        shard_streams(64, 2, 2)


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    first, count = shard_streams(64, world, rank)
    units = float(count * 1000)            # work proportional to the streams this rank owns
    seconds = 1.0 + 0.5 * rank             # rank 1 is slower: it sets the whole-job time
    dist.barrier()
    rate, total, slowest = whole_job_rate(units, seconds, dist)
    if rank == 0:
        results.put((rate, total, slowest, first, count))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_report_sum_of_work_over_slowest_rank():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    rate, total, slowest, first, count = results.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert (first, count) == (0, 32)
    assert total == 64000.0 and slowest == 1.5 and abs(rate - 64000.0 / 1.5) < 1e-9


def test_single_process_passthrough():
    assert whole_job_rate(10.0, 2.0) == (5.0, 10.0, 2.0)
