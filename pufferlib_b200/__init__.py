"""B200-native (sm_100a) implementation of PufferLib's advantage hot path.

Importing the package does not load native code; `pufferlib_b200.advantage`
loads `pufferlib_b200._C` (the torch operator registration) and
`libpuff_advantage_sm100.so` (kernels + C ABI) on first use and raises if they
have not been built (`python -m pufferlib_b200.build`).
"""
__version__ = "0.1"

from .advantage import (  # noqa: F401
    compute_puff_advantage,
    compute_puff_advantage_fill,
    compute_puff_advantage_host,
    compute_puff_advantage_prio,
    minibatch_gather,
    prioritized_sample_probs,
    priority_probs,
    priority_weights,
    rollout_write,
    set_variant,
)
