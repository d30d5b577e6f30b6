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


# ----------------------------------------------------------------------------------------------
# Membership: learning on the host that a rank has gone, before the next collective is entered.
# ----------------------------------------------------------------------------------------------
class RankLeft(RuntimeError):
    """A peer announced that it is leaving (between steps, nothing of its in flight)."""

    def __init__(self, rank):
        super().__init__("rank %d has left the run" % rank)
        self.rank = rank


class RankTimeout(RuntimeError):
    """A peer did not reach the step within the time limit (crashed, hung or partitioned)."""

    def __init__(self, rank, step, seconds):
        super().__init__("rank %d did not reach step %d within %.1f s" % (rank, step, seconds))
        self.rank = rank


class Membership:
    """Step-boundary roll call over a key-value store (the process group's TCP store by default).

    A collective that one rank never joins blocks the others until the library's own timeout, with
    their kernels queued behind it.  So the ranks meet on the host first: before a step's gradient
    exchange every rank publishes the step number it has reached and waits, with a short limit, until
    every peer has published the same step.  A rank that stops does so only between steps, with none
    of its kernels or collectives in flight, and says so with leave(); a rank that dies silently is
    caught by the limit.  Either way the survivors get an exception before they launch anything that
    would wait for the missing rank, and can stop cleanly or rebuild a smaller group."""

    def __init__(self, rank, world, store=None, prefix="slang_b200/membership"):
        if store is None:
            store = dist.distributed_c10d._get_default_store()
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix

    def _key(self, kind, rank):
        return "%s/%s/%d" % (self.prefix, kind, rank)

    def leave(self):
        self.store.set(self._key("left", self.rank), "1")

    def arrive(self, step, timeout_s=5.0, poll_s=0.01):
        """Publishes `step` for this rank and returns once every peer has published a step >= `step`.
        Raises RankLeft or RankTimeout otherwise."""
        import time
        self.store.set(self._key("step", self.rank), str(int(step)))
        deadline = time.monotonic() + timeout_s
        pending = [r for r in range(self.world) if r != self.rank]
        while pending:
            still = []
            for r in pending:
                if self.store.check([self._key("left", r)]):
                    raise RankLeft(r)
                k = self._key("step", r)
                if self.store.check([k]) and int(self.store.get(k)) >= step:
                    continue
                still.append(r)
            pending = still
            if pending:
                if time.monotonic() > deadline:
                    raise RankTimeout(pending[0], step, timeout_s)
                time.sleep(poll_s)
