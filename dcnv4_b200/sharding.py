"""Host-side batch sharding for multi-GPU runs (one process per GPU).

The operator path shards by batch with no exchange: every output element, and every
gradient element, depends only on its own sample's `value` and packed offset/mask row
(DCNv4_op/src/cuda/dcnv4_im2col_cuda.cuh:163,199-201; the backward scatter stays inside
`grad_im + bi*H*W*C`, DCNv4_op/src/cuda/dcnv4_col2im_cuda.cuh:287).  So a rank runs the
single-GPU operator on its slice and nothing crosses NVLink on this path; the only collective
in a training job is the data-parallel gradient all-reduce of the surrounding Linear layers
(classification/main.py:228-235), which is outside the operator.
"""
from __future__ import annotations

from typing import Tuple


def shard_bounds(n: int, rank: int, world: int) -> Tuple[int, int]:
    """[lo, hi) of the samples rank `rank` owns: contiguous, balanced to within one sample,
    covering 0..n exactly once over all ranks (ranks past `n` get an empty range)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world: {rank}/{world}")
    if n < 0:
        raise ValueError("negative batch")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard(tensor, rank: int, world: int):
    """The rank's slice of a batch-major tensor (a view; no copy)."""
    lo, hi = shard_bounds(tensor.shape[0], rank, world)
    return tensor[lo:hi]


def job_throughput(units_per_rank, elapsed_s_per_rank) -> float:
    """Whole-job throughput: all ranks' units over the slowest rank's time."""
    slowest = max(elapsed_s_per_rank)
    return sum(units_per_rank) / slowest if slowest > 0 else float("inf")
