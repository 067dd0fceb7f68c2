"""Worker of tests/test_exchange_gpu.py::test_two_processes_over_cuda_ipc:
one process per GPU, launched by torch.distributed.run."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import pufferlib_b200
    from pufferlib_b200 import cabi
    from pufferlib_b200.exchange import PeerExchange
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("gloo")
    x = PeerExchange.for_process_group()
    alpha = 0.8
    for round_ in range(12):
        g = torch.Generator().manual_seed(1000 * round_)
        all_sums = torch.rand(world, 4096 + 64 * round_, generator=g) * 30.0   # every rank draws every shard
        mine = all_sums[rank].cuda()
        weights = x.weights_push(mine, alpha)
        probs, total = x.probs_gathered(weights)
        want = torch.zeros(1, dtype=torch.float64, device="cuda")
        for r in range(world):
            want = want + pufferlib_b200.priority_weights(all_sums[r].cuda(), alpha)[1]
        assert torch.equal(total, want), (rank, round_, float(total), float(want))
        assert torch.equal(probs, pufferlib_b200.priority_probs(weights, want))
    assert cabi.device_status() == 0
    # a peer that stops taking part (it stays alive, idle, with nothing in flight): the other
    # rank's wait runs out and is reported, and its context stays usable
    dist.barrier()
    if rank == 0:
        x.set_wait_ns(20_000_000)
        w = x.weights_push(torch.ones(1000, device="cuda"), alpha)
        x.probs_gathered(w)
        torch.cuda.synchronize()
        assert cabi.device_status() == cabi.ERR_DEVICE_WAIT
        assert cabi.device_status() == 0
        assert float(pufferlib_b200.priority_weights(torch.ones(8, device="cuda"), alpha)[1]) == 8.0
    dist.barrier()          # rank 1 leaves only after rank 0 has finished every launch that names its mailbox
    torch.cuda.synchronize()
    x.close()
    print(f"rank {rank} ok", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
