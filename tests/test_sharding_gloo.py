"""Multi-process path on CPU (gloo, world size 2): every rank takes its contiguous shard of
the batch exactly as bench.py and the sharded front-end do, no data-path collective is
needed, and gathering the per-rank results reproduces the single-process answer.  The
compute stand-in is the CPU oracle (a checker is allowed in tests); what is under test is
the partitioning and the max-over-ranks timing reduction."""
import os

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import brownian_paths
from oracle import oracle
from pysiglib_b200.sharded import all_gather_signatures, shard_bounds


def _worker(rank, world, port, batch, tmpdir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        path = brownian_paths(3, batch, 12, 3)
        begin, end = shard_bounds(batch, world)[rank]
        chunk, rem = divmod(batch, world)          # bench.py's formula
        assert end - begin == chunk + (1 if rank < rem else 0)
        local = torch.tensor(oracle.sig(path[begin:end], 3))
        # optional gather of the results onto every rank (ragged shards: pad to the largest)
        biggest = chunk + (1 if rem else 0)
        padded = torch.zeros((biggest, local.shape[1]), dtype=local.dtype)
        padded[: local.shape[0]] = local
        pieces = [torch.zeros_like(padded) for _ in range(world)]
        dist.all_gather(pieces, padded)
        full = torch.cat([p[: e - b] for p, (b, e) in zip(pieces, shard_bounds(batch, world))])
        # the library's own gather (one all_gather_into_tensor, ragged shards padded and trimmed)
        assert torch.equal(all_gather_signatures(local, batch), full)
        # timing reduction used by bench.py: the slowest rank defines the step time
        t = torch.tensor([1.0 + rank], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            np.save(os.path.join(tmpdir, "full.npy"), full.numpy())
            np.save(os.path.join(tmpdir, "t.npy"), t.numpy())
    finally:
        dist.destroy_process_group()


def test_two_rank_batch_sharding(tmp_path):
    batch, world = 7, 2
    port = 29600 + os.getpid() % 300
    mp.spawn(_worker, args=(world, port, batch, str(tmp_path)), nprocs=world, join=True)
    full = np.load(tmp_path / "full.npy")
    np.testing.assert_array_equal(full, oracle.sig(brownian_paths(3, batch, 12, 3), 3))
    assert np.load(tmp_path / "t.npy")[0] == 2.0
