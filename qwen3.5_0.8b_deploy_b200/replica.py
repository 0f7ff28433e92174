"""Replica data parallelism over sequences: one process per GPU, the model replicated, sequences
partitioned, no collective on the data path.  The only exchange is a reduction of benchmark counters
(NCCL on GPUs, gloo in CPU tests)."""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def env_rank() -> tuple[int, int, int]:
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def partition(total_sequences: int, world: int, rank: int) -> range:
    """Sequence s belongs to rank s % world (each rank owns its KV pages, DeltaNet state and conv cache)."""
    return range(rank, total_sequences, world)


def init(backend: str, local_rank: int = 0) -> None:
    if dist.is_initialized():
        return
    if backend == "nccl":
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    else:
        dist.init_process_group(backend)


def barrier() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


def reduce_counters(max_values: list[float], sum_values: list[float], device: str = "cpu") -> tuple[list[float], list[float]]:
    """MAX over ranks of the timings, SUM over ranks of the unit counts."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return list(max_values), list(sum_values)
    a = torch.tensor(max_values, dtype=torch.float64, device=device)
    b = torch.tensor(sum_values, dtype=torch.float64, device=device)
    dist.all_reduce(a, op=dist.ReduceOp.MAX)
    dist.all_reduce(b, op=dist.ReduceOp.SUM)
    return a.tolist(), b.tolist()


def job_throughput(tokens_all_ranks: float, ms_max_over_ranks: float) -> float:
    return tokens_all_ranks / (ms_max_over_ranks / 1e3)
