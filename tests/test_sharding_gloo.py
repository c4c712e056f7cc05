"""Batch sharding across ranks (one process per GPU in production) exercised with two gloo
ranks on CPU: contiguous slices, ragged splits, gather of per-rank logits, metric reductions."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from layer_quant_b200.sharding import shard_batch


def test_shard_batch_partitions_exactly():
    for gb in (0, 1, 7, 8, 255, 256):
        for world in (1, 2, 3, 8):
            shards = [shard_batch(gb, r, world) for r in range(world)]
            assert shards[0].start == 0 and shards[-1].stop == gb
            assert all(a.stop == b.start for a, b in zip(shards, shards[1:]))
            sizes = [s.local_batch for s in shards]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_batch(8, 2, 2)


def _worker(rank, world, port, global_batch, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    import torch.distributed as dist
    from layer_quant_b200 import sharding
    r, lr, w = sharding.init_from_env(backend="gloo")
    assert (r, w) == (rank, world) and sharding.world_size() == world
    sh = sharding.shard_batch(global_batch, rank, world)
    full = torch.arange(global_batch * 6, dtype=torch.float32).reshape(global_batch, 6)
    local = sh.slice(full).clone() * 1.0
    sharding.barrier()
    gathered = sharding.gather_batch(local, sh, dst=0)
    mx = sharding.all_reduce_max(float(rank + 1), torch.device("cpu"))
    sm = sharding.all_reduce_sum(float(sh.local_batch), torch.device("cpu"))
    ok = mx == world and sm == global_batch
    if rank == 0:
        ok = ok and gathered is not None and torch.equal(gathered, full)
    else:
        ok = ok and gathered is None
    out[rank] = bool(ok)
    dist.destroy_process_group()


@pytest.mark.parametrize("global_batch", [8, 5])
def test_two_rank_gather_and_reductions(global_batch):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, global_batch, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert dict(out) == {0: True, 1: True}
