"""One rank's end of the cross-GPU exchange of the priority-weight total.

Wraps the `puff_exchange` object of include/puff_advantage.h: a small mailbox in
this rank's device memory into which every rank's priority kernel stores its
local weight total directly (plain stores over NVLink to peer-mapped memory),
so that the sampling probabilities of a segment-sharded buffer are normalised
by the global total without a collective call between the two kernels.  The
reference has no counterpart (its DDP ranks never share this op's buffers,
pufferl.py:913-939).

`PeerExchange.for_process_group()` is the one-process-per-GPU set-up: the
mailbox handles (CUDA IPC) travel through `torch.distributed.all_gather_object`
once.  `PeerExchange.in_process()` links several exchanges of ONE process by
pointer (several GPUs driven by one process; also what the single-GPU tests use).
"""
import ctypes

import torch

from . import cabi


class PeerExchange:
    def __init__(self, rank, world, want_handle=True):
        lib = cabi.load()
        self._lib = lib
        self.rank, self.world = rank, world
        self._ctx = ctypes.c_void_p()
        self._handle = ctypes.create_string_buffer(cabi.EXCHANGE_HANDLE_BYTES) if want_handle else None
        cabi.check(lib.puff_exchange_sm100_create(rank, world, self._handle, ctypes.byref(self._ctx)),
                   "puff_exchange_sm100_create")

    # -- set-up ---------------------------------------------------------------
    @classmethod
    def for_process_group(cls, group=None):
        """One exchange per rank of `group` (one process per GPU, all on one
        machine); the current CUDA device is this rank's.  Collective: every
        rank of the group must call it."""
        import torch.distributed as dist
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        x = cls(rank, world)
        if world > 1:
            handles = [None] * world
            dist.all_gather_object(handles, x._handle.raw, group=group)
            blob = b"".join(handles)
            cabi.check(x._lib.puff_exchange_sm100_connect(x._ctx, blob), "puff_exchange_sm100_connect")
        return x

    @classmethod
    def in_process(cls, world, devices=None):
        """`world` linked exchanges inside this process, rank r on devices[r]
        (default: all on the current device)."""
        cur = torch.cuda.current_device()
        devices = [cur] * world if devices is None else list(devices)
        out = []
        for r in range(world):
            with torch.cuda.device(devices[r]):
                out.append(cls(r, world, want_handle=False))
        boxes = (ctypes.c_void_p * world)(*[x._lib.puff_exchange_sm100_mailbox(x._ctx) for x in out])
        for x in out:
            cabi.check(x._lib.puff_exchange_sm100_connect_pointers(x._ctx, boxes), "puff_exchange_sm100_connect_pointers")
        return out

    def set_wait_ns(self, ns):
        cabi.check(self._lib.puff_exchange_sm100_set_wait_ns(self._ctx, int(ns)))

    @property
    def handle(self):
        """The puff_exchange* as an integer (what the torch ops take)."""
        return int(self._ctx.value)

    def close(self):
        if self._ctx:
            self._lib.puff_exchange_sm100_destroy(self._ctx)
            self._ctx = ctypes.c_void_p()

    # -- the two steps ----------------------------------------------------------
    def weights_push(self, seg_abs_sum, alpha):
        """Local weights (pufferl.py:360); their total goes to every rank."""
        from . import advantage
        return advantage._ops().puff_priority_weights_push(seg_abs_sum, alpha, self.handle)

    def probs_gathered(self, weights):
        """(probs, total): pufferl.py:361 with the total over all ranks."""
        from . import advantage
        return advantage._ops().puff_priority_probs_gathered(weights, self.handle)
