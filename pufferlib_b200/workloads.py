"""Seeded synthetic inputs for the advantage path.

The reference ships no dataset, benchmark suite or golden vectors for
`compute_puff_advantage`; these generators stand in for the trainer's
experience buffers (pufferl.py:101-107: `[segments, horizon]` fp32 `values`,
`rewards`, `terminals`, `ratio`) with the shapes, value distributions and
hyper-parameters of the five benchmark configurations.

Draw order is fixed -- values, rewards, dones, importance -- from one CPU
`torch.Generator`, so that any machine with the same torch build regenerates
identical bits.
"""
from dataclasses import dataclass, replace

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    segments: int
    horizon: int
    gamma: float = 0.99
    lam: float = 0.95
    rho_clip: float = 1.0
    c_clip: float = 1.0
    done_p: float = 0.01
    importance_sigma: float = 0.1
    value_sigma: float = 1.0
    reward_sigma: float = 0.1
    sparse_reward_p: float = 0.0   # >0: rewards = Bernoulli(p) * N(1, 0.5)
    seed: int = 0
    epilogue: bool = False         # fused per-segment |advantage| sums wanted
    variant: str = "auto"          # kernel variant the configuration exercises

    @property
    def elements(self):
        return self.segments * self.horizon

    def hyper(self):
        return (self.gamma, self.lam, self.rho_clip, self.c_clip)

    def with_segments(self, segments, seed=None):
        return replace(self, segments=segments, seed=self.seed if seed is None else seed)


WORKLOADS = {
    # CPU reference run
    "cfg0": Workload("cfg0", 1024, 64),
    # typical PPO buffer (config/ocean/nmmo3.ini:27-29: 524288 / 64)
    "cfg1": Workload("cfg1", 8192, 64),
    # large sharded buffer
    "cfg2": Workload("cfg2", 131072, 256, gamma=0.995, lam=0.9, done_p=0.005, importance_sigma=0.3),
    # long-horizon narrow: the scan variant's case
    "cfg3": Workload("cfg3", 256, 4096, gamma=0.999, lam=0.95, done_p=0.001,
                     sparse_reward_p=0.02, variant="scan"),
    # clipping / non-tile-aligned stress, epilogue on, serial and bit-exact
    "cfg4": Workload("cfg4", 10007, 127, rho_clip=1.0, c_clip=0.9, done_p=0.2,
                     importance_sigma=1.0, value_sigma=10.0, epilogue=True, variant="serial"),
}


def make_inputs(wl, pin=False):
    """(values, rewards, dones, importance) as CPU fp32 tensors [S, H]."""
    g = torch.Generator(device="cpu").manual_seed(wl.seed)
    shape = (wl.segments, wl.horizon)
    values = torch.randn(shape, generator=g) * wl.value_sigma
    if wl.sparse_reward_p > 0.0:
        mask = (torch.rand(shape, generator=g) < wl.sparse_reward_p).float()
        rewards = mask * (torch.randn(shape, generator=g) * 0.5 + 1.0)
    else:
        rewards = torch.randn(shape, generator=g) * wl.reward_sigma
    dones = (torch.rand(shape, generator=g) < wl.done_p).float()
    importance = torch.exp(torch.randn(shape, generator=g) * wl.importance_sigma)
    out = (values, rewards, dones, importance)
    if pin:
        out = tuple(t.pin_memory() for t in out)
    return out


def shard_rows(segments, rank, world):
    """Contiguous row block [lo, hi) of rank `rank` out of `world`."""
    return (rank * segments) // world, ((rank + 1) * segments) // world
