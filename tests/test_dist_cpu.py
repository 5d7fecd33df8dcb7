"""World-size-2 gloo run of the sharding / gather plumbing on CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from stof_b200 import dist as sd


def test_shard_ranges_partition():
    for n in (1, 7, 16, 64, 192):
        for world in (1, 2, 3, 4, 8):
            spans = [sd.shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    assert sd.attention_shard(16, 12, 3, 8) == ((6, 8), (0, 12))
    assert sd.attention_shard(6, 16, 1, 4) == ((0, 6), (4, 8))
    with pytest.raises(ValueError):
        sd.shard_range(4, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, total):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    r, w, _ = sd.init_from_env("gloo")
    assert (r, w) == (rank, world)
    full = torch.arange(total * 3, dtype=torch.float32).view(total, 3)
    lo, hi = sd.shard_range(total, rank, world)
    got = sd.gather_shards(full[lo:hi].clone(), total, dim=0)
    assert torch.equal(got, full)
    assert sd.max_over_ranks(10.0 + rank) == 10.0 + world - 1
    assert sd.sum_over_ranks(float(hi - lo)) == float(total)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_gloo_world2_gather_and_reduce():
    mp.spawn(_worker, args=(2, _free_port(), 5), nprocs=2, join=True)
