"""Data-parallel plumbing: which samples a rank takes and how the gradient buffers are summed.

The training step shards naturally: samples are independent and the only coupling is the sum of the
per-parameter gradients.  Rank r of N takes the contiguous block [r*B/N, (r+1)*B/N) of every step's
batch; after learnGradient each rank holds the gradient sum of its block in the flat fp32 gradient
segment; one all-reduce (sum) of that segment, plus one of the two loss words, makes every rank hold
the whole batch's gradient, and every rank then runs the same adjustParameters, so the parameters
stay identical without a broadcast.  torch.distributed carries the collective (NCCL on GPUs, gloo
for the CPU tests of this logic).
"""
import torch
import torch.distributed as dist


def shard_range(global_count, rank, world):
    """[begin, end) of the samples rank `rank` of `world` processes takes."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    return global_count * rank // world, global_count * (rank + 1) // world


def allreduce_gradients(grads, loss_words=None, group=None, deterministic=False):
    """In-place sum of the flat gradient segment over the ranks; the loss words combine as
    (max of word 0 as float, sum of word 1 as float).  Tensors live wherever the backend needs them.

    The order in which a collective library adds the ranks' terms depends on its algorithm (ring, tree,
    in-switch), so the summed bits can differ from run to run and from N to N.  With
    deterministic=True every rank gathers all ranks' segments and adds them itself in ascending rank
    order: the result is the same on every rank and for every library, at N times the traffic (the
    segment is a few hundred KB at most)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    if deterministic:
        world = dist.get_world_size(group)
        parts = [torch.empty_like(grads) for _ in range(world)]
        dist.all_gather(parts, grads, group=group)
        grads.copy_(parts[0])
        for r in range(1, world):
            grads.add_(parts[r])
    else:
        dist.all_reduce(grads, op=dist.ReduceOp.SUM, group=group)
    if loss_words is not None:
        mx = loss_words[0:1].clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=group)
        sm = loss_words[1:2].clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM, group=group)
        loss_words[0:1] = mx
        loss_words[1:2] = sm
