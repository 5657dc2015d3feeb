"""Multi-rank host logic on CPU: two gloo ranks shard a batch, run independently, gather for checking."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from disentangled_flash_b200 import sharding


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _fake_forward(x: torch.Tensor) -> torch.Tensor:
    # stands in for the per-sequence encoder: any function applied row by row
    return torch.tanh(x * 1.5) + x.flip(-1)


def _worker(rank: int, world: int, port: int, n_items: int, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.arange(n_items * 6, dtype=torch.float32).reshape(n_items, 6) / 7.0
        mine = sharding.shard_indices(n_items, rank, world)
        per_rank = -(-n_items // world)
        local = torch.zeros(per_rank, 6)
        local[: len(mine)] = _fake_forward(full[mine])
        gathered = sharding.gather_for_check(local)
        merged = sharding.reassemble(gathered, n_items)
        slowest = sharding.max_over_ranks(float(rank + 1))
        if rank == 0:
            results.put((torch.equal(merged, _fake_forward(full)), slowest))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
@pytest.mark.parametrize("n_items", (8, 7))
def test_two_ranks_shard_and_gather(n_items):
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, n_items, results)) for r in range(2)]
    for p in procs:
        p.start()
    ok, slowest = results.get(timeout=90)
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    assert ok and slowest == 2.0


def test_shard_helpers_single_process():
    assert sharding.shard_indices(7, 1, 3) == [1, 4]
    buckets = sharding.shard_buckets({512: 170, 128: 171, 256: 171}, 0, 8)
    assert list(buckets) == [128, 256, 512] and len(buckets[128]) == 22 and len(buckets[512]) == 22
    total = sum(len(sharding.shard_indices(171, r, 8)) for r in range(8))
    assert total == 171
    x = torch.randn(4, 3)
    assert sharding.gather_for_check(x)[0] is x
    assert sharding.max_over_ranks(3.5) == 3.5
    with pytest.raises(ValueError):
        sharding.shard_indices(4, 2, 2)
