"""Gradient-compression communication hooks for DistributedDataParallel.

The reference's classification trainer wraps the model in DDP and registers a hook that sends
every gradient bucket over the wire in 16 bits (classification/main.py:228-235,
classification/ddp_hooks.py:44-109): the bucket is cast to fp16 (or bf16), divided by the world
size BEFORE the all-reduce so that the sum cannot overflow the narrow type, all-reduced
asynchronously, and the result is copied back into the bucket's own fp32 storage.  This module
provides the same three hooks for training jobs built on this package.  The operator itself has
no part in this exchange: DCNv4 / FlashDeformAttn produce no parameter gradients, the buckets
hold the gradients of the Linear / Conv / LayerNorm layers around them.
"""
from typing import Callable, Optional

import torch
import torch.distributed as dist

# DDP inspects a hook's annotations at registration: `bucket` must be annotated with the GradBucket
# class itself and the return type with Future[Tensor] (so no postponed evaluation of annotations here).
Hook = Callable[[Optional[dist.ProcessGroup], dist.GradBucket], torch.futures.Future[torch.Tensor]]


def _group(process_group: Optional[dist.ProcessGroup]) -> dist.ProcessGroup:
    return process_group if process_group is not None else dist.group.WORLD


def allreduce_hook(process_group: Optional[dist.ProcessGroup],
                   bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """Mean of the bucket over the group in the bucket's own dtype (what DDP does without a hook)."""
    group = _group(process_group)
    buf = bucket.buffer()
    buf.div_(group.size())
    work = dist.all_reduce(buf, group=group, async_op=True)
    return work.get_future().then(lambda fut: fut.value()[0])


def make_compress_hook(wire_dtype: torch.dtype) -> Hook:
    """Hook that all-reduces each bucket in `wire_dtype` (half the bytes of fp32 gradients)."""

    def hook(process_group: Optional[dist.ProcessGroup],
             bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
        group = _group(process_group)
        full = bucket.buffer()
        wire = full.to(wire_dtype).div_(group.size())      # divide first: the sum stays in range
        work = dist.all_reduce(wire, group=group, async_op=True)

        def widen(fut):
            full.copy_(fut.value()[0])                      # back into the bucket's storage, in place
            return full

        return work.get_future().then(widen)

    hook.__name__ = f"{str(wire_dtype).split('.')[-1]}_compress_hook"
    return hook


fp16_compress_hook = make_compress_hook(torch.float16)
bf16_compress_hook = make_compress_hook(torch.bfloat16)

HOOKS = {"none": None, "fp32": allreduce_hook, "fp16": fp16_compress_hook, "bf16": bf16_compress_hook}


def register(ddp_model: torch.nn.parallel.DistributedDataParallel, kind: str = "fp16") -> bool:
    """Register the hook named `kind` ("fp16" as the reference's trainer does, "bf16", "fp32", or
    "none") on a DDP model; returns whether a hook was registered."""
    hook = HOOKS[kind]
    if hook is None:
        return False
    ddp_model.register_comm_hook(state=None, hook=hook)
    return True
