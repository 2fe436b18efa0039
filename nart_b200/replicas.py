"""Batch-sharded replicas: the only multi-GPU form this path has.  Every op is per image, so GPU
`rank` of `world` runs the same case on its own slice of the batch and nothing crosses between
GPUs on the data path (the reference has no distributed code at all: one workspace per device id,
art/modules/cuda_quant/src/cuda_quant_module.c:98-141 of ModelTC/NART).  torch.distributed is used
only to start together and to agree on the slowest rank's time."""
from __future__ import annotations

import os


def env_rank_world():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def shard(total_images: int, rank: int, world: int):
    """Images [lo, hi) of a global batch that rank `rank` owns; sizes differ by at most one."""
    if not 0 <= rank < world:
        raise ValueError("rank %d outside 0..%d" % (rank, world - 1))
    base, extra = divmod(total_images, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def init(backend: str, device=None):
    import torch.distributed as dist
    rank, world, _ = env_rank_world()
    if world > 1 and not dist.is_initialized():
        kw = {}
        if device is not None:
            kw["device_id"] = device
        dist.init_process_group(backend, **kw)
    return rank, world


def barrier():
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


def max_over_ranks(value: float, device="cpu") -> float:
    """The slowest rank's figure: a job of replicas is as fast as its slowest member."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, device="cpu") -> float:
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def all_ranks_hold(payload: bytes, device="cpu") -> bool:
    """True when every rank passed the same bytes (at most 64; a digest): the check that batch-sharded
    replicas given the same images produce the same result.  A single process trivially agrees."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return True
    if len(payload) > 64:
        raise ValueError("pass a digest, not the data")
    buf = bytes(payload).ljust(64, b"\0")
    mine = torch.tensor(list(buf), dtype=torch.uint8, device=device)
    gathered = [torch.empty_like(mine) for _ in range(dist.get_world_size())]
    dist.all_gather(gathered, mine)
    return all(bool(torch.equal(g, gathered[0])) for g in gathered)


def images_per_sec(images_this_rank: int, steps: int, elapsed_ms_this_rank: float, device="cpu") -> float:
    """Whole-job throughput: all ranks' images over the slowest rank's time."""
    total = sum_over_ranks(images_this_rank * steps, device)
    return total / (max_over_ranks(elapsed_ms_this_rank, device) / 1e3)
