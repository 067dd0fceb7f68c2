"""CPU, world size 2 over gloo: the host-side logic of the segment-sharded
path (row partition, all-reduce of the weight total, global normalisation).
The three device steps are replaced by an oracle-backed stand-in; the CUDA
kernels themselves are covered by the GPU tests."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pufferlib_b200.sharded import ShardedAdvantage
from pufferlib_b200.workloads import Workload, make_inputs, shard_rows

ALPHA = 0.8


class OracleKernels:
    """Stand-in with the interface of sharded.CudaKernels, for CPU ranks."""

    def advantage_prio(self, values, rewards, dones, importance, advantages, seg_abs_sum, hyper):
        from oracle import puff_oracle
        puff_oracle.advantage(values.numpy(), rewards.numpy(), dones.numpy(), importance.numpy(),
                              advantages.numpy(), *hyper)
        seg_abs_sum.copy_(torch.from_numpy(puff_oracle.abs_sum(advantages.numpy())).float())

    def weights(self, seg_abs_sum, alpha):
        w = torch.nan_to_num(seg_abs_sum ** alpha, 0, 0, 0)
        return w, w.double().sum().reshape(1)

    def probs(self, weights, total):
        return (weights + 1e-6) / (total.float() + 1e-6)


class GatherExchange:
    """Stand-in with the interface of exchange.PeerExchange for CPU ranks: every
    rank's total reaches every rank (an all-gather over gloo stands where the
    kernels store into peer mailboxes) and is added in rank order."""

    def weights_push(self, seg_abs_sum, alpha):
        w = torch.nan_to_num(seg_abs_sum ** alpha, 0, 0, 0)
        mine = w.double().sum().reshape(1)
        self._totals = [torch.zeros(1, dtype=torch.float64) for _ in range(dist.get_world_size())]
        dist.all_gather(self._totals, mine)
        return w

    def probs_gathered(self, weights):
        total = torch.zeros(1, dtype=torch.float64)
        for t in self._totals:          # rank order on every rank
            total = total + t
        return (weights + 1e-6) / (total.float() + 1e-6), total


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, wl, out_dir, use_exchange=False):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = make_inputs(wl)
        sh = ShardedAdvantage(wl.segments, wl.horizon, wl.hyper(), ALPHA, kernels=OracleKernels(),
                              exchange=GatherExchange() if use_exchange else None)
        assert (sh.lo, sh.hi) == shard_rows(wl.segments, rank, world)
        local = [t[sh.lo:sh.hi].contiguous() for t in full]
        adv = torch.zeros_like(local[0])
        abs_sum = torch.empty(sh.local_segments)
        probs, total = sh.step(*local, adv, abs_sum)
        np.save(os.path.join(out_dir, f"probs{rank}.npy"), probs.numpy())
        np.save(os.path.join(out_dir, f"adv{rank}.npy"), adv.numpy())
        np.save(os.path.join(out_dir, f"total{rank}.npy"), total.numpy())
    finally:
        dist.destroy_process_group()


import pytest  # noqa: E402


@pytest.mark.parametrize("use_exchange", [False, True])
def test_two_rank_sharded_step_matches_single_process(tmp_path, use_exchange):
    """Both ways the total can cross ranks: an all-reduce between the two
    priority steps, or an exchange object whose two steps move it themselves."""
    from oracle import puff_oracle
    wl = Workload("shard", 1001, 48, seed=17, done_p=0.05)
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), wl, str(tmp_path), use_exchange), nprocs=world, join=True)

    full = [t.numpy() for t in make_inputs(wl)]
    adv = np.zeros_like(full[0])
    puff_oracle.advantage(*full, adv, *wl.hyper())
    w, p, tot = puff_oracle.priorities(puff_oracle.abs_sum(adv), ALPHA)

    got_adv = np.concatenate([np.load(tmp_path / f"adv{r}.npy") for r in range(world)])
    got_p = np.concatenate([np.load(tmp_path / f"probs{r}.npy") for r in range(world)])
    totals = [float(np.load(tmp_path / f"total{r}.npy")[0]) for r in range(world)]
    assert np.array_equal(got_adv.view(np.uint32), adv.view(np.uint32))
    assert totals[0] == totals[1]                       # every rank holds the global sum
    assert abs(totals[0] - tot) <= 1e-5 * tot
    np.testing.assert_allclose(got_p, p, rtol=2e-5)
    assert abs(got_p.astype(np.float64).sum() - 1.0) < 1e-3   # normalised over ALL ranks' segments


def test_single_rank_needs_no_process_group():
    wl = Workload("one", 64, 16, seed=2)
    sh = ShardedAdvantage(wl.segments, wl.horizon, wl.hyper(), ALPHA, kernels=OracleKernels(), rank=0, world=1)
    local = list(make_inputs(wl))
    adv = torch.zeros_like(local[0])
    abs_sum = torch.empty(wl.segments)
    probs, total = sh.step(*local, adv, abs_sum)
    assert probs.shape == (64,) and abs(float(probs.sum()) - 1.0) < 1e-4
