"""Data-parallel sharding of independent decode sequences: one process per GPU, a contiguous
slice of the batch per rank, no collective on the hot path.  ``torch.distributed`` (NCCL on
GPUs, gloo in CPU tests) is used only to gather logits and to reduce metrics.

The reference is single-process, single-GPU; this module is what the multi-GPU launcher of the
benchmark and of an evaluation loop use around the two kernels."""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class BatchShard:
    rank: int
    world_size: int
    global_batch: int
    start: int
    stop: int

    @property
    def local_batch(self) -> int:
        return self.stop - self.start

    def slice(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor:
        return t.narrow(dim, self.start, self.local_batch)


def shard_batch(global_batch: int, rank: int, world_size: int) -> BatchShard:
    """Contiguous split; the first ``global_batch % world_size`` ranks take one extra sequence."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"rank={rank} outside world_size={world_size}")
    if global_batch < 0:
        raise ValueError(f"global_batch={global_batch}")
    base, extra = divmod(global_batch, world_size)
    start = rank * base + min(rank, extra)
    return BatchShard(rank, world_size, global_batch, start, start + base + (1 if rank < extra else 0))


def init_from_env(backend: str | None = None) -> tuple[int, int, int]:
    """(rank, local_rank, world_size) from the torchrun environment; initialises the default
    process group when WORLD_SIZE > 1 and binds the CUDA device of LOCAL_RANK."""
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if torch.cuda.is_available():
        torch.cuda.set_device(local_rank)
    if world > 1 and not dist.is_initialized():
        backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        kwargs = {}
        if backend == "nccl":
            kwargs["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kwargs)
    return rank, local_rank, world


def world_size() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def barrier() -> None:
    if world_size() > 1:
        dist.barrier()


def all_reduce_max(value: float, device: torch.device) -> float:
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def all_reduce_sum(value: float, device: torch.device) -> float:
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def gather_batch(local: torch.Tensor, shard: BatchShard, dst: int = 0) -> torch.Tensor | None:
    """Concatenate per-rank slices ``[local_batch, ...]`` (e.g. logits) along dim 0 on rank ``dst``.
    Ragged splits are padded to the largest slice for the collective and trimmed afterwards."""
    if shard.world_size == 1:
        return local
    sizes = [shard_batch(shard.global_batch, r, shard.world_size).local_batch for r in range(shard.world_size)]
    width = max(sizes)
    padded = local
    if local.shape[0] < width:
        pad = local.new_zeros((width - local.shape[0],) + tuple(local.shape[1:]))
        padded = torch.cat([local, pad], dim=0)
    outs = [torch.empty_like(padded) for _ in range(shard.world_size)]
    dist.all_gather(outs, padded.contiguous())
    if shard.rank != dst:
        return None
    return torch.cat([o[:n] for o, n in zip(outs, sizes)], dim=0)
