"""Replica-parallel plumbing: the only multi-GPU mode of the quantized-linear path.

A single GEMM does not shard naturally and the reference has no multi-GPU code, so work is split by whole
images / batch rows: item i runs on rank i mod world (one process per GPU), every rank holds a full copy of the
weights, and nothing crosses NVLink on the data path.  torch.distributed is used only to line ranks up for timing
and to take the maximum of the per-rank elapsed times; it works with the `nccl` backend on GPUs and `gloo` on CPU.
"""

import os

import torch
import torch.distributed as dist


def env_rank_world():
    """(rank, local_rank, world_size) from the torchrun environment; (0, 0, 1) when launched as a plain process."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


def items_for_rank(n_items, rank, world):
    """Indices of the independent items (images, batch rows) that `rank` owns: item i -> rank i mod world."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank/world: %d/%d" % (rank, world))
    return list(range(rank, n_items, world))


def init(backend, device=None):
    """Initialises the default process group from the environment if world_size > 1; returns True if it did."""
    _, _, world = env_rank_world()
    if world <= 1:
        return False
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if dist.is_initialized():
        return True
    kwargs = {}
    if backend == "nccl" and device is not None:
        kwargs["device_id"] = device
    dist.init_process_group(backend, **kwargs)
    return True


def barrier(device=None):
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
    if device is not None and torch.device(device).type == "cuda":
        torch.cuda.synchronize(device)


def max_over_ranks(values, device=None):
    """Element-wise maximum over ranks of a list of floats (each rank's device-measured times)."""
    t = torch.tensor(list(values), dtype=torch.float64, device=device if device is not None else "cpu")
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t.cpu()]


def sum_over_ranks(value, device=None):
    t = torch.tensor([float(value)], dtype=torch.float64, device=device if device is not None else "cpu")
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.cpu()[0])


def shutdown():
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()
