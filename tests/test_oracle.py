"""CPU: the oracle against the golden fixtures and the reference build."""
import os

import numpy as np
import pytest
import torch

from helpers import SENTINEL, bits_equal, first_mismatch, oracle_advantage, sha256_arrays
from pufferlib_b200.workloads import WORKLOADS, Workload, make_inputs, shard_rows

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_oracle_matches_golden_small(golden_small):
    """Fixtures were produced by the reference's own CPU op (make_golden.py)."""
    for name, case in golden_small.items():
        got = oracle_advantage([case[k] for k in ("values", "rewards", "dones", "importance")], case["hyper"])
        assert bits_equal(got, case["advantages"]), f"{name}: {first_mismatch(got, case['advantages'])}"


def test_last_column_untouched(golden_small):
    for name, case in golden_small.items():
        assert np.all(case["advantages"][:, -1] == np.float32(SENTINEL)), name


@pytest.mark.parametrize("name", ["cfg0", "cfg1", "cfg3", "cfg4"])
def test_oracle_matches_config_digest(name, config_digests):
    wl = WORKLOADS[name]
    inputs = make_inputs(wl)
    ref = config_digests["configs"][name]
    if sha256_arrays(*[t.numpy() for t in inputs]) != ref["inputs_sha256"]:
        pytest.skip("this torch build draws different random inputs than the fixture generator")
    got = oracle_advantage([t.numpy() for t in inputs], wl.hyper(), ref_sentinel(config_digests))
    assert sha256_arrays(got) == ref["advantages_sha256"]
    flat = got.reshape(-1)
    assert flat[np.array(ref["sample_index"])].view(np.uint32).tolist() == ref["sample_bits"]


def ref_sentinel(digests):
    return digests["sentinel"]


def test_oracle_matches_reference_build():
    """Live bit-equality with the reference source compiled into oracle/_ref/
    (present where the reference tree was mounted at build time)."""
    from oracle import puff_oracle
    ref = puff_oracle.load_reference()
    if ref is None:
        pytest.skip("oracle/_ref/ not built on this machine")
    for wl in [WORKLOADS["cfg0"], WORKLOADS["cfg4"], Workload("x", 300, 91, seed=3, c_clip=0.0),
               WORKLOADS["cfg3"]]:
        inputs = make_inputs(wl)
        adv = torch.full_like(inputs[0], SENTINEL)
        ref(*inputs, adv, *wl.hyper())
        got = oracle_advantage([t.numpy() for t in inputs], wl.hyper())
        assert bits_equal(got, adv.numpy()), first_mismatch(got, adv.numpy())


def test_plain_gae_cross_check():
    """With importance == 1 and clips >= 1 the op is ordinary GAE whose last
    step bootstraps nothing (compare pufferlib/cleanrl_ppo_atari.py:243-256,
    which differs only in bootstrapping from next_value at the last step)."""
    wl = Workload("gae", 6, 20, seed=21, done_p=0.15)
    v, r, d, _ = [t.double().numpy() for t in make_inputs(wl)]
    w = np.ones_like(v, dtype=np.float32)
    got = oracle_advantage([v, r, d, w], wl.hyper(), sentinel=0.0)
    exp = np.zeros_like(v)
    last = np.zeros(v.shape[0])
    for t in range(v.shape[1] - 2, -1, -1):
        nn = 1.0 - d[:, t + 1]
        delta = r[:, t + 1] + wl.gamma * v[:, t + 1] * nn - v[:, t]
        last = delta + wl.gamma * wl.lam * nn * last
        exp[:, t] = last
    np.testing.assert_allclose(got, exp, rtol=2e-5, atol=2e-6)


def test_abs_sum_and_priorities():
    from oracle import puff_oracle
    wl = WORKLOADS["cfg0"]
    inputs = [t.numpy() for t in make_inputs(wl)]
    adv = oracle_advantage(inputs, wl.hyper(), sentinel=0.0)
    s = puff_oracle.abs_sum(adv)
    np.testing.assert_allclose(s, np.abs(adv.astype(np.float64)).sum(1), rtol=1e-12)
    w, p, tot = puff_oracle.priorities(s, 0.8)
    t = torch.from_numpy(s)
    tw = torch.nan_to_num(t ** 0.8, 0, 0, 0)
    np.testing.assert_allclose(w, tw.numpy(), rtol=1e-12)
    np.testing.assert_allclose(p, ((tw + 1e-6) / (tw.sum() + 1e-6)).numpy(), rtol=1e-12)
    assert abs(tot - float(tw.sum())) < 1e-6


def test_shard_rows_cover():
    for S in (0, 1, 7, 10007, 131072):
        for W in (1, 2, 3, 4, 8):
            spans = [shard_rows(S, r, W) for r in range(W)]
            assert spans[0][0] == 0 and spans[-1][1] == S
            assert all(spans[i][1] == spans[i + 1][0] for i in range(W - 1))


def test_minibatch_oracle_matches_torch_sequence():
    """The fp64 restatement of pufferl.py:363, 373-375, 408-409 against the
    same lines evaluated with torch in float64."""
    from oracle import puff_oracle
    g = torch.Generator().manual_seed(4)
    S, H, M, beta = 200, 48, 37, 0.4
    adv = torch.randn(S, H, generator=g)
    val = torch.randn(S, H, generator=g)
    probs = torch.rand(S, generator=g).double() + 0.01
    probs = probs / probs.sum()
    idx = torch.multinomial(probs, M, generator=g)
    o_v, o_r, o_n, o_p = puff_oracle.minibatch(adv.numpy(), val.numpy(), probs.numpy(), idx.numpy(), beta)
    a64, v64 = adv.double(), val.double()
    mb_prio = (S * probs[idx, None]) ** -beta
    e = a64[idx]
    e = mb_prio * (e - e.mean()) / (e.std() + 1e-8)
    np.testing.assert_allclose(o_n, e.numpy(), rtol=1e-12, atol=1e-14)
    np.testing.assert_allclose(o_r, (a64[idx] + v64[idx]).numpy(), rtol=0, atol=0)
    np.testing.assert_allclose(o_p, mb_prio.numpy()[:, 0], rtol=1e-13)


def _numpy_restatement(v, r, d, w, gamma, lam, rho_clip, c_clip, sentinel):
    """The recurrence of pufferlib.cpp:28-41 column by column over all rows at
    once, every operation rounded to fp32 in the reference's order."""
    f = np.float32
    S, H = v.shape
    adv = np.full((S, H), sentinel, dtype=np.float32)
    a = np.zeros(S, dtype=np.float32)
    gl = f(f(gamma) * f(lam))
    with np.errstate(all="ignore"):
        for t in range(H - 2, -1, -1):
            nn = (1.0 - d[:, t + 1].astype(np.float64)).astype(np.float32)   # a double subtraction there
            rho = np.minimum(w[:, t], f(rho_clip))
            c = np.minimum(w[:, t], f(c_clip))
            td = (r[:, t + 1] + (f(gamma) * v[:, t + 1]) * nn) - v[:, t]
            delta = rho * td
            a = delta + ((gl * c) * a) * nn
            adv[:, t] = a
    return adv


def test_oracle_matches_a_vectorised_restatement_on_random_shapes():
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=40, deadline=None)
    @given(S=st.integers(1, 40), H=st.integers(1, 70), seed=st.integers(0, 2 ** 16),
           gamma=st.sampled_from([0.0, 0.9, 0.99, 1.0]), lam=st.sampled_from([0.0, 0.5, 0.95, 1.0]),
           rho_clip=st.sampled_from([0.0, 0.5, 1.0, 3.0]), c_clip=st.sampled_from([0.0, 0.9, 1.0, 2.5]),
           done_p=st.sampled_from([0.0, 0.05, 0.5, 1.0]))
    def check(S, H, seed, gamma, lam, rho_clip, c_clip, done_p):
        rng = np.random.default_rng(seed)
        v = rng.standard_normal((S, H)).astype(np.float32)
        r = rng.standard_normal((S, H)).astype(np.float32)
        d = (rng.random((S, H)) < done_p).astype(np.float32)
        w = np.exp(rng.standard_normal((S, H))).astype(np.float32)
        hyper = (gamma, lam, rho_clip, c_clip)
        got = oracle_advantage([v, r, d, w], hyper)
        want = _numpy_restatement(v, r, d, w, *hyper, SENTINEL)
        assert bits_equal(got, want), first_mismatch(got, want)
        # rows are independent: any row block gives the same bits
        if S > 1:
            part = oracle_advantage([a[S // 2:] for a in (v, r, d, w)], hyper)
            assert bits_equal(part, got[S // 2:])
        # scaling values and rewards by a power of two scales the advantages exactly
        scaled = oracle_advantage([v * 4, r * 4, d, w], hyper)
        assert bits_equal(scaled[:, :-1], got[:, :-1] * 4)

    check()
