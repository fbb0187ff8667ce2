"""Data-parallel plumbing for the Mellin layers: one process per GPU, utterances
sharded over ranks, weight and bias gradients summed with ONE all-reduce.

The operators themselves never communicate: forward and grad-input are
independent per utterance, and the only cross-rank dependency of a training
step is the sum of grad_w / grad_b.  ``torch.distributed`` (NCCL on GPUs, gloo
in the CPU tests) carries that sum; there is no custom collective.
"""
from typing import Iterable, List, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_range(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous [begin, end) slice of `total` utterances owned by `rank`;
    sizes differ by at most one and the slices tile [0, total)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad world/rank %d/%d" % (world, rank))
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def balanced_shards(lengths: Sequence[int], world: int) -> List[List[int]]:
    """Assign ragged utterances to ranks so that the summed lengths are as even
    as a greedy longest-first pass gets them (ties broken by rank order, so every
    rank computes the same assignment without talking to the others)."""
    order = sorted(range(len(lengths)), key=lambda i: (-lengths[i], i))
    loads = [0] * world
    shards: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda k: (loads[k], k))
        shards[r].append(i)
        loads[r] += lengths[i]
    return shards


class GradBucket:
    """Flat buffer holding the gradients of a set of parameters so that one
    all-reduce sums them all."""

    def __init__(self, shapes: Iterable[Sequence[int]], device, dtype=torch.float32):
        self.shapes = [tuple(s) for s in shapes]
        self.sizes = [int(torch.Size(s).numel()) for s in self.shapes]
        self.flat = torch.zeros(sum(self.sizes), device=device, dtype=dtype)

    def views(self) -> List[torch.Tensor]:
        out, o = [], 0
        for shape, n in zip(self.shapes, self.sizes):
            out.append(self.flat[o:o + n].view(shape))
            o += n
        return out

    def pack(self, grads: Sequence[torch.Tensor]) -> None:
        for v, g in zip(self.views(), grads):
            v.copy_(g)

    def all_reduce(self, group=None, async_op: bool = False):
        """Sum over ranks, in place."""
        if not dist.is_initialized() or dist.get_world_size(group) == 1:
            return None
        return dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group, async_op=async_op)
