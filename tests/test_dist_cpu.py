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


def _sharded_attention_worker(rank, world, port):
    """The flow of the benchmark's sharded attention record with the CPU oracle in the kernel's place: every rank takes its
    (batch, head) slice of the same seeded tensors, computes it, the slices are gathered along the split dimension and every
    rank checks the whole tensor against the unsharded computation."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    sd.init_from_env("gloo")
    from oracle import attention as oa
    from stof_b200 import workloads as wl
    S = 128
    mask = wl.expand_block_mask(wl.block_sliding(S // 64, 1)).float()
    for batch, heads in ((4, 3), (3, 4), (5, 3)):                 # batch split, head split, uneven batch split
        g = torch.Generator().manual_seed(batch * 10 + heads)
        q, k, v = (torch.randn(batch, heads, S, 64, generator=g).half() for _ in range(3))
        (b0, b1), (h0, h1) = sd.attention_shard(batch, heads, rank, world)
        mine = oa.masked_attention_fp32(q[b0:b1, h0:h1], k[b0:b1, h0:h1], v[b0:b1, h0:h1], mask)
        dim = 1 if (h1 - h0) < heads else 0
        whole = sd.gather_shards(mine.contiguous(), batch if dim == 0 else heads, dim=dim)
        want = oa.masked_attention_fp32(q, k, v, mask)
        assert whole.shape == want.shape and torch.allclose(whole, want, atol=1e-6)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_gloo_world2_sharded_attention_gather():
    mp.spawn(_sharded_attention_worker, args=(2, _free_port()), nprocs=2, join=True)
