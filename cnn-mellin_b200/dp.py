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


def snake_shards(lengths: Sequence[int], world: int) -> List[List[int]]:
    """Equal-count, length-balanced assignment: utterances sorted longest first
    are dealt to the ranks in boustrophedon order (0..world-1, world-1..0, ...),
    so every rank gets len(lengths) / world of them, the sums of lengths differ
    by little, and the longest utterances (which set each rank's padded length)
    land on different ranks.  Deterministic: every rank computes the same deal."""
    if world < 1 or len(lengths) % world != 0:
        raise ValueError("%d utterances do not split evenly over %d ranks" % (len(lengths), world))
    order = sorted(range(len(lengths)), key=lambda i: (-lengths[i], i))
    shards: List[List[int]] = [[] for _ in range(world)]
    for k, i in enumerate(order):
        lap, pos = divmod(k, world)
        shards[pos if lap % 2 == 0 else world - 1 - pos].append(i)
    return shards


class BucketedReducer:
    """Averages the gradients of a model over the ranks while backward still runs.

    The parameters are grouped, in the order backward produces their gradients
    (last layer first), into flat buckets of about ``bucket_bytes``; every
    parameter's ``.grad`` is a view into its bucket, so the gradient kernels
    write straight into the buffer that is reduced -- nothing is packed.  A
    hook fires when a parameter's gradient is complete; when the last one of a
    bucket has fired, the bucket's all-reduce is launched asynchronously (the
    communication library runs it on its own stream, ordered after the kernels
    queued so far) and backward carries on.  ``finish_step`` makes the compute
    stream wait for the reductions before the optimizer reads the gradients.
    """

    def __init__(self, params: Iterable[torch.nn.Parameter], bucket_bytes: int = 32 << 20, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        params = [p for p in params if p.requires_grad]
        self.buckets: List[torch.Tensor] = []
        self._bucket_of = {}
        self._pending: List[int] = []
        self._sizes: List[int] = []
        self._works = []
        self._hooks = []
        group_params: List[torch.nn.Parameter] = []
        nbytes = 0

        def close():
            nonlocal group_params, nbytes
            if not group_params:
                return
            flat = torch.zeros(sum(p.numel() for p in group_params), device=group_params[0].device,
                               dtype=group_params[0].dtype)
            o = 0
            for p in group_params:
                p.grad = flat[o:o + p.numel()].view_as(p)
                self._bucket_of[p] = len(self.buckets)
                o += p.numel()
            self.buckets.append(flat)
            self._sizes.append(len(group_params))
            group_params, nbytes = [], 0

        for p in reversed(params):
            if group_params and (p.dtype != group_params[0].dtype or nbytes + p.numel() * p.element_size() > bucket_bytes):
                close()
            group_params.append(p)
            nbytes += p.numel() * p.element_size()
        close()
        for p in params:
            self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad))
        self.reduced_bytes = sum(b.numel() * b.element_size() for b in self.buckets)

    def begin_step(self) -> None:
        """Zero the buckets (the gradients accumulate into them) and re-arm the hooks."""
        for flat in self.buckets:
            flat.zero_()
        self._pending = list(self._sizes)
        self._works = []

    def _on_grad(self, p: torch.nn.Parameter) -> None:
        k = self._bucket_of[p]
        self._pending[k] -= 1
        if self._pending[k] == 0 and self.world > 1:
            self._works.append(dist.all_reduce(self.buckets[k], op=dist.ReduceOp.SUM, group=self.group, async_op=True))

    def finish_step(self) -> None:
        """Order the compute stream after every reduction and turn the sums into means."""
        if any(n != 0 for n in self._pending):
            raise RuntimeError("a parameter received no gradient this step: its bucket was never reduced")
        for work in self._works:
            work.wait()
        if self.world > 1:
            for flat in self.buckets:
                flat.div_(self.world)
        self._works = []

    def remove(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks = []
