"""Host-side mirror of the reference's advantage interface.

`compute_puff_advantage` keeps the name, argument order and return value of
pufferlib/pufferl.py:660-680; it calls the operator registered by
`pufferlib_b200._C` under the reference's own name,
`torch.ops.pufferlib.compute_puff_advantage` (schema of
pufferlib/extensions/pufferlib.cpp:88).  The reference wrapper's
"no CUDA toolchain -> move everything to the CPU" branch (pufferl.py:666-678)
has no counterpart: this implementation is the CUDA op, and it raises when the
extension is missing or the tensors are not on an sm_100 GPU.

The other functions expose what the reference computes right after the op
(pufferl.py:359-361) on top of the fused per-segment |advantage| sums.
"""
import torch

from . import cabi


def _ops():
    from . import _C  # noqa: F401  (loading it registers torch.ops.pufferlib.*)
    return torch.ops.pufferlib


def set_variant(name):
    """Kernel variant of the advantage ops ("auto", "serial", "scan",
    "generic"); returns the previous one.  The initial setting is "auto", or
    the environment variable PUFFER_ADV_VARIANT as it stood at the first op
    call; the op calls themselves read no environment."""
    prev = _ops().puff_set_variant(cabi.VARIANTS[name])
    return next(k for k, v in cabi.VARIANTS.items() if v == prev)


def compute_puff_advantage(values, rewards, terminals, ratio, advantages,
                           gamma, gae_lambda, vtrace_rho_clip, vtrace_c_clip):
    """In-place V-trace-clipped GAE; returns `advantages` (pufferl.py:660-680).

    Writes advantages[:, :H-1]; column H-1 keeps whatever the caller put there
    (the trainer passes zeros, pufferl.py:353)."""
    _ops().compute_puff_advantage(values, rewards, terminals, ratio, advantages,
                                  gamma, gae_lambda, vtrace_rho_clip, vtrace_c_clip)
    return advantages


def compute_puff_advantage_prio(values, rewards, terminals, ratio, advantages, seg_abs_sum,
                                gamma, gae_lambda, vtrace_rho_clip, vtrace_c_clip):
    """Same launch with the fused epilogue: additionally fills `seg_abs_sum`
    ([segments] fp32) with sum_t |advantages[s, t]|, t < H-1 -- the
    `advantages.abs().sum(axis=1)` of pufferl.py:359 without re-reading
    `advantages`.  Returns (advantages, seg_abs_sum)."""
    _ops().compute_puff_advantage_prio(values, rewards, terminals, ratio, advantages, seg_abs_sum,
                                       gamma, gae_lambda, vtrace_rho_clip, vtrace_c_clip)
    return advantages, seg_abs_sum


def compute_puff_advantage_fill(values, rewards, terminals, ratio, gamma, gae_lambda,
                                vtrace_rho_clip, vtrace_c_clip, advantages=None, seg_abs_sum=None):
    """The op with ownership of its whole output: writes advantages[:, H-1] = 0
    itself, so no zero-filled buffer is needed in front of it (replaces the
    `torch.zeros` + op pair of pufferl.py:352-356 and saves one 4 B/element
    write pass per call).  `advantages` may be any uninitialised [S, H] fp32
    tensor; one is allocated when omitted.  Returns it."""
    if advantages is None:
        advantages = torch.empty_like(values)
    _ops().compute_puff_advantage_fill(values, rewards, terminals, ratio, advantages, seg_abs_sum,
                                       gamma, gae_lambda, vtrace_rho_clip, vtrace_c_clip)
    return advantages


def priority_weights(seg_abs_sum, prio_alpha):
    """(weights, total): weights = nan_to_num(seg_abs_sum ** alpha, 0, 0, 0)
    (pufferl.py:360) and their fp64 sum as a 1-element CUDA tensor."""
    return _ops().puff_priority_weights(seg_abs_sum, prio_alpha)


def priority_probs(weights, total):
    """(weights + 1e-6) / (total + 1e-6)  (pufferl.py:361)."""
    return _ops().puff_priority_probs(weights, total)


def minibatch_gather(advantages, values, prio_probs, idx, anneal_beta, prio_segments=None):
    """What the trainer computes for the sampled segments `idx` (int64, CUDA)
    right after `torch.multinomial` (pufferl.py:363, 373-375, 408-409), in two
    launches.  Returns (mb_values, mb_returns, mb_advantages, adv, mb_prio):
    values[idx], advantages[idx] + values[idx], advantages[idx], the
    priority-weighted normalised advantages
    mb_prio * (a - a.mean()) / (a.std() + 1e-8), and
    mb_prio = (segments * prio_probs[idx, None]) ** -anneal_beta.
    `prio_segments` is that `segments` factor when it is not the row count of
    `advantages`: the global segment count of a sharded buffer whose
    probabilities were normalised over all shards."""
    return _ops().puff_minibatch_gather(advantages, values, prio_probs, idx, anneal_beta,
                                        -1 if prio_segments is None else int(prio_segments))


def rollout_write(rewards, terminals, values, step_rewards, step_dones, step_values,
                  row_begin, column, reward_clip=1.0):
    """One environment step into column `column` of the experience buffers for
    rows [row_begin, row_begin + len(step_rewards)): the clamp of pufferl.py:275
    and the three column assignments of :294-296 in one launch."""
    _ops().puff_rollout_write(rewards, terminals, values, step_rewards, step_dones, step_values.flatten(),
                              row_begin, column, reward_clip)


def prioritized_sample_probs(values, rewards, terminals, ratio, advantages,
                             gamma, gae_lambda, vtrace_rho_clip, vtrace_c_clip, prio_alpha,
                             process_group=None):
    """pufferl.py:352-361 in three launches: advantages, priority weights,
    sampling probabilities.  With `process_group`, segments are taken to be
    sharded over its ranks and the weight total is all-reduced, so every rank
    normalises by the global sum.  Returns (advantages, prio_probs)."""
    seg_abs_sum = torch.empty(values.shape[0], device=values.device, dtype=torch.float32)
    compute_puff_advantage_prio(values, rewards, terminals, ratio, advantages, seg_abs_sum,
                                gamma, gae_lambda, vtrace_rho_clip, vtrace_c_clip)
    weights, total = priority_weights(seg_abs_sum, prio_alpha)
    if process_group is not None:
        torch.distributed.all_reduce(total, group=process_group)
    return advantages, priority_probs(weights, total)


def compute_puff_advantage_host(values, rewards, terminals, ratio, advantages,
                                gamma, gae_lambda, vtrace_rho_clip, vtrace_c_clip,
                                seg_abs_sum=None, variant="auto", device=0):
    """The op for HOST tensors (pinned memory recommended) through the C ABI's
    pipelined entry point: row blocks are uploaded, processed and downloaded on
    rotating streams.  Synchronous; returns `advantages`."""
    lib = cabi.load()
    tensors = [values, rewards, terminals, ratio, advantages]
    S, H = values.shape
    for t in tensors:
        if t.device.type != "cpu" or t.dtype != torch.float32 or not t.is_contiguous() or t.shape != (S, H):
            raise RuntimeError("host entry point needs contiguous float32 CPU tensors of one shape")
    abs_ptr = None
    if seg_abs_sum is not None:
        if seg_abs_sum.device.type != "cpu" or seg_abs_sum.dtype != torch.float32 or seg_abs_sum.shape != (S,):
            raise RuntimeError("seg_abs_sum must be a float32 CPU tensor [segments]")
        abs_ptr = seg_abs_sum.data_ptr()
    rc = lib.puff_advantage_sm100_host(
        values.data_ptr(), rewards.data_ptr(), terminals.data_ptr(), ratio.data_ptr(),
        advantages.data_ptr(), abs_ptr, gamma, gae_lambda, vtrace_rho_clip, vtrace_c_clip,
        S, H, cabi.VARIANTS[variant], device)
    cabi.check(rc, "puff_advantage_sm100_host")
    return advantages


def launch_raw(values, rewards, terminals, ratio, advantages, gamma, gae_lambda,
               vtrace_rho_clip, vtrace_c_clip, seg_abs_sum=None, variant="auto", stream=None, flags=0):
    """Direct C-ABI launch on CUDA tensors (no dispatcher): used by tests and
    the benchmark to pick a kernel variant explicitly.  Only pointers and sizes
    cross the boundary; shapes are the caller's responsibility."""
    lib = cabi.load()
    S, H = values.shape
    if stream is None:
        stream = torch.cuda.current_stream(values.device).cuda_stream
    rc = lib.puff_advantage_sm100_launch_ex(
        values.data_ptr(), rewards.data_ptr(), terminals.data_ptr(), ratio.data_ptr(),
        advantages.data_ptr(), None if seg_abs_sum is None else seg_abs_sum.data_ptr(),
        gamma, gae_lambda, vtrace_rho_clip, vtrace_c_clip, S, H, cabi.VARIANTS[variant], flags, stream)
    cabi.check(rc, "puff_advantage_sm100_launch_ex")
    return advantages
