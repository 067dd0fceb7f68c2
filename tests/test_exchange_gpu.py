"""GPU: the cross-GPU exchange of the priority-weight total (puff_exchange).

On one GPU the ranks are emulated inside the process: their pushes are issued
first and their gathers afterwards on one stream, so no kernel ever waits for a
kernel that has not run yet.  The bounded wait is tested by leaving one rank's
push out: the gather gives up after a few milliseconds, records
PUFF_ERR_DEVICE_WAIT and returns; nothing faults or hangs.  With two or more
GPUs the same rounds run as two processes over CUDA IPC.
"""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ALPHA = 0.8


def _sums(n, seed):
    g = torch.Generator().manual_seed(seed)
    s = torch.rand(n, generator=g) * 50.0
    s[::97] = float("inf")      # non-finite sums get weight 0 (pufferl.py:360)
    return s.cuda()


def test_world_of_one_equals_the_plain_path():
    import pufferlib_b200
    from pufferlib_b200.exchange import PeerExchange
    x = PeerExchange(0, 1, want_handle=False)
    try:
        for n in (1, 1000, 131072):
            sums = _sums(n, n)
            w0, total0 = pufferlib_b200.priority_weights(sums, ALPHA)
            p0 = pufferlib_b200.priority_probs(w0, total0)
            w1 = x.weights_push(sums, ALPHA)
            p1, total1 = x.probs_gathered(w1)
            assert torch.equal(w0, w1) and torch.equal(total0, total1) and torch.equal(p0, p1)
    finally:
        x.close()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_emulated_ranks_agree_on_the_global_total(world):
    import pufferlib_b200
    from pufferlib_b200 import cabi
    from pufferlib_b200.exchange import PeerExchange
    ranks = PeerExchange.in_process(world)
    try:
        for round_ in range(10):     # more rounds than mailbox slots: the ring is reused
            shards = [_sums(0 if (r == 1 and round_ == 3) else 3000 + 17 * r, 100 * round_ + r) for r in range(world)]
            local = [pufferlib_b200.priority_weights(s, ALPHA) for s in shards]
            weights = [x.weights_push(s, ALPHA) for x, s in zip(ranks, shards)]
            got = [x.probs_gathered(w) for x, w in zip(ranks, weights)]
            # the global total: the local fp64 totals added in rank order, identical bits on every rank
            want_total = torch.zeros(1, dtype=torch.float64, device="cuda")
            for _, t in local:
                want_total = want_total + t
            for r in range(world):
                probs, total = got[r]
                assert torch.equal(total, want_total), (round_, r)
                assert torch.equal(weights[r], local[r][0])
                assert torch.equal(probs, pufferlib_b200.priority_probs(local[r][0], want_total))
        assert cabi.device_status() == 0
    finally:
        for x in ranks:
            x.close()


def test_a_missing_peer_ends_the_wait_with_a_status_not_a_hang():
    import pufferlib_b200
    from pufferlib_b200 import cabi
    from pufferlib_b200.exchange import PeerExchange
    a, b = PeerExchange.in_process(2)
    try:
        a.set_wait_ns(5_000_000)      # 5 ms
        sums_a, sums_b = _sums(5000, 1), _sums(4000, 2)
        wa = a.weights_push(sums_a, ALPHA)
        probs, total = a.probs_gathered(wa)          # rank 1 never pushed its total
        torch.cuda.synchronize()
        assert cabi.device_status() == cabi.ERR_DEVICE_WAIT
        assert cabi.device_status() == 0             # cleared by the read; the context is intact
        # the late rank arrives: the round completes on a second try
        wb = b.weights_push(sums_b, ALPHA)
        probs_a, total_a = a.probs_gathered(wa)
        probs_b, total_b = b.probs_gathered(wb)
        _, ta = pufferlib_b200.priority_weights(sums_a, ALPHA)
        _, tb = pufferlib_b200.priority_weights(sums_b, ALPHA)
        assert torch.equal(total_a, ta + tb) and torch.equal(total_b, total_a)
        assert torch.equal(probs_a, pufferlib_b200.priority_probs(wa, total_a))
        assert cabi.device_status() == 0
    finally:
        a.close()
        b.close()


def test_argument_checks():
    from pufferlib_b200 import cabi
    lib = cabi.load()
    import ctypes
    ctx = ctypes.c_void_p()
    assert lib.puff_exchange_sm100_create(2, 2, None, ctypes.byref(ctx)) == cabi.ERR_SHAPE
    assert lib.puff_exchange_sm100_create(0, 0, None, ctypes.byref(ctx)) == cabi.ERR_SHAPE
    assert lib.puff_exchange_sm100_create(0, 2, None, ctypes.byref(ctx)) == cabi.OK
    buf = torch.zeros(16, device="cuda")
    scratch = torch.zeros(64, dtype=torch.float64, device="cuda")
    # not connected yet: nothing is launched
    rc = lib.puff_priorities_sm100_weights_push(buf.data_ptr(), buf.data_ptr(), 0.5, 16, scratch.data_ptr(), 512,
                                                ctx, None)
    assert rc == cabi.ERR_WORKSPACE
    assert lib.puff_exchange_sm100_destroy(ctx) == cabi.OK


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_over_cuda_ipc(tmp_path):
    """One process per GPU, mailboxes shared through CUDA IPC handles; the
    host-side handle exchange runs over gloo, so no collective library touches
    the GPUs.  The last round leaves rank 1's push out (rank 1 stays alive and
    idle): rank 0's wait gives up after 20 ms and reports it."""
    env = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0")
    out = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
         "--master-addr", "127.0.0.1", "--master-port", "29653",
         os.path.join(ROOT, "tests", "exchange_worker.py")],
        env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert "rank 0 ok" in out.stdout and "rank 1 ok" in out.stdout
