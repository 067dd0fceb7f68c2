"""Segment-sharded advantage + prioritised-replay weights over several GPUs.

Segments (rows) are independent, so a buffer of `segments x horizon` shards by
contiguous row blocks with no data-path communication; the only exchange is
one fp64 scalar per rank, the total priority weight that pufferl.py:361
divides by: either all-reduced by torch.distributed between the two priority
launches, or (with a `PeerExchange`) stored by the priority kernels straight
into every peer's memory.  The reference itself never shards this op (its DDP
ranks own private buffers, pufferl.py:913-939); this class is the layout the
multi-GPU benchmark measures: one process per GPU, `torch.distributed` for
the scalar.

`kernels` is the object that provides the three device steps.  The default is
the CUDA implementation; tests of the host-side logic on CPU ranks pass a
stand-in with the same three methods.
"""
import torch
import torch.distributed as dist

from .workloads import shard_rows


class CudaKernels:
    """The product path: the sm_100a kernels behind torch.ops.pufferlib."""

    def __init__(self):
        from . import advantage
        self._adv = advantage

    def advantage_prio(self, values, rewards, dones, importance, advantages, seg_abs_sum, hyper):
        self._adv.compute_puff_advantage_prio(values, rewards, dones, importance, advantages,
                                              seg_abs_sum, *hyper)

    def weights(self, seg_abs_sum, alpha):
        return self._adv.priority_weights(seg_abs_sum, alpha)

    def probs(self, weights, total):
        return self._adv.priority_probs(weights, total)


class ShardedAdvantage:
    """One rank's shard of the advantage path.

    step() computes advantages for the local rows, the local priority weights,
    all-reduces their total over `group`, and returns the local slice of the
    globally normalised sampling probabilities."""

    def __init__(self, global_segments, horizon, hyper, prio_alpha, group=None, kernels=None,
                 rank=None, world=None, exchange=None):
        self.group = group
        # exchange: a pufferlib_b200.exchange.PeerExchange -> the weight total crosses GPUs inside
        # the priority kernels; None -> torch.distributed all-reduce between them
        self.exchange = exchange
        if rank is None:
            rank = dist.get_rank(group) if dist.is_initialized() else 0
        if world is None:
            world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank, self.world = rank, world
        self.lo, self.hi = shard_rows(global_segments, rank, world)
        self.global_segments = global_segments
        self.horizon = horizon
        self.hyper = tuple(hyper)
        self.prio_alpha = prio_alpha
        self.kernels = kernels if kernels is not None else CudaKernels()

    @property
    def local_segments(self):
        return self.hi - self.lo

    def priorities(self, seg_abs_sum):
        """Local weights, their all-reduced total, globally normalised probabilities."""
        if self.exchange is not None:
            weights = self.exchange.weights_push(seg_abs_sum, self.prio_alpha)
            return self.exchange.probs_gathered(weights)
        k = self.kernels
        weights, total = k.weights(seg_abs_sum, self.prio_alpha)
        if self.world > 1:
            dist.all_reduce(total, op=dist.ReduceOp.SUM, group=self.group)
        return k.probs(weights, total), total

    def step_overlapped(self, values, rewards, dones, importance, advantages, seg_abs_sum, side_stream):
        """CUDA only.  The advantage kernel goes to the current stream; the
        priority launches and the all-reduce of their scalar go to
        `side_stream`, ordered after the kernel by an event, so that they
        overlap whatever the caller enqueues next on the current stream (for
        instance the next advantage pass on other buffers).

        Returns (probs, total, done): `done` is an event on the side stream.
        The caller must make a stream wait on it before that stream reads
        `probs`/`total` or overwrites `seg_abs_sum`."""
        main = torch.cuda.current_stream()
        self.kernels.advantage_prio(values, rewards, dones, importance, advantages, seg_abs_sum, self.hyper)
        ready = torch.cuda.Event()
        ready.record(main)
        with torch.cuda.stream(side_stream):
            side_stream.wait_event(ready)
            probs, total = self.priorities(seg_abs_sum)
            done = torch.cuda.Event()
            done.record(side_stream)
        return probs, total, done

    def step(self, values, rewards, dones, importance, advantages, seg_abs_sum):
        """All tensors are this rank's rows [local_segments, horizon] (and
        [local_segments] for seg_abs_sum).  Returns (probs, total) where total
        is the global weight sum as a 1-element fp64 tensor."""
        self.kernels.advantage_prio(values, rewards, dones, importance, advantages, seg_abs_sum, self.hyper)
        return self.priorities(seg_abs_sum)
