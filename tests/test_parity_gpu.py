"""GPU parity: every kernel variant against the CPU oracle and the golden
fixtures, through the C ABI and through the torch operator."""
import os

import numpy as np
import pytest
import torch

from helpers import (SENTINEL, bits_equal, first_mismatch, oracle_advantage, sha256_arrays,
                     within_scan_tolerance)
from pufferlib_b200.workloads import WORKLOADS, Workload, make_inputs

pytestmark = pytest.mark.gpu

KEYS = ("values", "rewards", "dones", "importance")
FORCE = {"tma2d": 1, "bulk1d": 2, "scan": 3, "generic": 4}


@pytest.fixture(autouse=True)
def _clear_tuning():
    from pufferlib_b200 import cabi
    cabi.reset_tuning()
    yield
    cabi.reset_tuning()


def run_gpu(inputs, hyper, variant="auto", force=None, epilogue=False, sentinel=SENTINEL, stages=None, flags=0, ws=None,
            warp_teams=None):
    """Launch through the C ABI; returns (advantages, abs_sum or None, kernel name)."""
    from pufferlib_b200 import cabi
    from pufferlib_b200.advantage import launch_raw
    dev = [torch.as_tensor(np.asarray(t)).contiguous().cuda() for t in inputs]
    adv = torch.full_like(dev[0], sentinel)
    abs_sum = torch.full((dev[0].shape[0],), -1.0, device="cuda") if epilogue else None
    # ws: 0 = single-warp tma2d, N = warp-specialised with N stages
    # warp_teams: 0 = the one-stage bulk1d kernel with one tile per CTA, 1 (its default where it fits) one per warp
    cabi.set_tuning(force_kernel=None if force is None else FORCE[force], stages=stages, ws_stages=ws,
                    b1_warp_teams=warp_teams)
    try:
        launch_raw(*dev, adv, *hyper, seg_abs_sum=abs_sum, variant=variant, flags=flags)
        kernel = cabi.last_kernel()
        torch.cuda.synchronize()
    finally:
        cabi.reset_tuning()
    assert cabi.device_status() == 0
    return adv.cpu().numpy(), None if abs_sum is None else abs_sum.cpu().numpy(), kernel


def applicable(force, H):
    if force == "tma2d":
        return H % 4 == 0
    return True


# ---------------------------------------------------------------------------
# golden fixtures (outputs of the reference CPU op)
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("force", ["tma2d", "bulk1d", "generic"])
def test_serial_kernels_match_golden_bitwise(golden_small, force):
    ran = 0
    for name, case in golden_small.items():
        H = case["values"].shape[1]
        if not applicable(force, H):
            continue
        got, _, kernel = run_gpu([case[k] for k in KEYS], case["hyper"], "serial", force)
        if H >= 2:
            assert kernel == force, (name, kernel)
        assert bits_equal(got, case["advantages"]), f"{name}/{force}: {first_mismatch(got, case['advantages'])}"
        ran += 1
    assert ran >= 3


def test_scan_kernel_matches_golden_within_tolerance(golden_small):
    for name, case in golden_small.items():
        if name in ("special", "odd127", "gain_overflow"):
            continue   # non-finite values / |values| ~ 10: outside the scan variant's stated bar
        got, _, kernel = run_gpu([case[k] for k in KEYS], case["hyper"], "scan")
        want = case["advantages"]
        assert np.all(got[:, -1] == np.float32(SENTINEL)), name
        assert within_scan_tolerance(got[:, :-1], want[:, :-1]), name


@pytest.mark.parametrize("name", ["special", "gain_overflow"])
def test_scan_special_values_propagate(golden_small, name):
    """NaN / Inf positions agree with the reference even where values differ in
    rounding; a row whose ((gamma*lambda)*c)*A overflows under nn == 0 is NaN
    from there to its start, as in the reference."""
    case = golden_small[name]
    got, _, kernel = run_gpu([case[k] for k in KEYS], case["hyper"], "scan")
    assert kernel == "scan"
    want = case["advantages"]
    assert np.array_equal(np.isnan(got), np.isnan(want))
    fin = np.isfinite(want)
    np.testing.assert_allclose(got[fin], want[fin], rtol=1e-4, atol=1e-5)


def test_auto_keeps_serial_kernel_when_gain_can_exceed_one():
    """Few long rows take the scan kernel under AUTO only while
    gamma*lambda*c_clip <= 1; otherwise AUTO stays bit-exact."""
    wl = Workload("fewlong", 64, 1024, seed=31, c_clip=3.0, importance_sigma=1.0)
    inputs = [t.numpy() for t in make_inputs(wl)]
    got, _, kernel = run_gpu(inputs, wl.hyper(), "auto")
    assert kernel == "tma2d"
    want = oracle_advantage(inputs, wl.hyper())
    assert bits_equal(got, want), first_mismatch(got, want)
    _, _, kernel = run_gpu(inputs, (0.99, 0.95, 1.0, 1.0), "auto")
    assert kernel == "scan"


# ---------------------------------------------------------------------------
# the five benchmark configurations
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["cfg0", "cfg1", "cfg2", "cfg3", "cfg4"])
def test_config_serial_bitwise(name, config_digests):
    wl = WORKLOADS[name]
    inputs = [t.numpy() for t in make_inputs(wl)]
    got, abs_sum, kernel = run_gpu(inputs, wl.hyper(), "serial", epilogue=True)
    assert kernel == ("bulk1d" if wl.horizon % 4 else "tma2d")
    want = oracle_advantage(inputs, wl.hyper())
    assert bits_equal(got, want), f"{name}: {first_mismatch(got, want)}"
    ref = config_digests["configs"][name]
    if sha256_arrays(*inputs) == ref["inputs_sha256"]:
        assert sha256_arrays(got) == ref["advantages_sha256"]
    exact = np.abs(want[:, :-1].astype(np.float64)).sum(1)
    np.testing.assert_allclose(abs_sum, exact, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("name", ["cfg0", "cfg1", "cfg2", "cfg3"])
def test_config_scan_tolerance(name):
    wl = WORKLOADS[name]
    inputs = [t.numpy() for t in make_inputs(wl)]
    got, abs_sum, kernel = run_gpu(inputs, wl.hyper(), "scan", epilogue=True)
    assert kernel == "scan"
    want = oracle_advantage(inputs, wl.hyper())
    assert np.all(got[:, -1] == np.float32(SENTINEL))
    assert within_scan_tolerance(got[:, :-1], want[:, :-1])
    exact = np.abs(want[:, :-1].astype(np.float64)).sum(1)
    np.testing.assert_allclose(abs_sum, exact, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("S,H", [(3000, 1024), (3500, 512), (700, 2048), (512, 4096), (2048, 4096), (8192, 512),
                                 (1537, 1030), (2999, 515)])
def test_scan_with_many_rows_within_tolerance(S, H):
    """With many rows the launcher gives a row fewer threads (512 down to 64, one or several
    eight- or four-column passes); every such split keeps the tolerance, the untouched last
    column and the fused sums."""
    wl = Workload("scan_rows", S, H, gamma=0.999, lam=0.95, done_p=0.002, seed=S + H)
    inputs = [t.numpy() for t in make_inputs(wl)]
    got, abs_sum, kernel = run_gpu(inputs, wl.hyper(), "scan", epilogue=True)
    assert kernel == "scan"
    want = oracle_advantage(inputs, wl.hyper())
    assert np.all(got[:, -1] == np.float32(SENTINEL))
    assert within_scan_tolerance(got[:, :-1], want[:, :-1])
    exact = np.abs(want[:, :-1].astype(np.float64)).sum(1)
    np.testing.assert_allclose(abs_sum, exact, rtol=1e-5, atol=1e-6)


def test_auto_variant_choices():
    picks = {}
    for name in ("cfg1", "cfg3", "cfg4"):
        wl = WORKLOADS[name]
        inputs = [t.numpy() for t in make_inputs(wl)]
        _, _, picks[name] = run_gpu(inputs, wl.hyper(), "auto")
    assert picks == {"cfg1": "tma2d", "cfg3": "scan", "cfg4": "bulk1d"}


@pytest.mark.parametrize("stages", [2, 3, 4])
def test_tma2d_stage_counts(stages):
    wl = Workload("st", 1000, 200, seed=31, done_p=0.05)
    inputs = [t.numpy() for t in make_inputs(wl)]
    got, abs_sum, kernel = run_gpu(inputs, wl.hyper(), "serial", epilogue=True, stages=stages)
    want = oracle_advantage(inputs, wl.hyper())
    assert kernel == "tma2d" and bits_equal(got, want), first_mismatch(got, want)


# ---------------------------------------------------------------------------
# exhaustive small shapes, ragged tiles, canaries
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("force", ["tma2d", "bulk1d", "scan", "generic"])
def test_small_shape_sweep(force):
    rng_seed = 100
    for S in (1, 2, 31, 32, 33, 65, 70):
        for H in list(range(1, 41)) + [63, 64, 65, 68, 70, 96, 100, 127, 128, 129, 132]:
            if not applicable(force, H):
                continue
            wl = Workload("sweep", S, H, seed=rng_seed, done_p=0.1)
            rng_seed += 1
            inputs = [t.numpy() for t in make_inputs(wl)]
            variant = "scan" if force == "scan" else "serial"
            got, abs_sum, kernel = run_gpu(inputs, wl.hyper(), variant, force, epilogue=True)
            want = oracle_advantage(inputs, wl.hyper())
            if force == "scan":
                assert np.all(got[:, -1] == np.float32(SENTINEL)), (S, H)
                assert within_scan_tolerance(got[:, :-1], want[:, :-1]), (S, H)
            else:
                assert bits_equal(got, want), f"S={S} H={H} {force}: {first_mismatch(got, want)}"
            exact = np.abs(want[:, :-1].astype(np.float64)).sum(1)
            np.testing.assert_allclose(abs_sum, exact, rtol=1e-5, atol=1e-6, err_msg=f"S={S} H={H}")


@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_random_shapes_and_hyperparameters(seed):
    """Seeded random shapes (up to a few thousand segments, horizons up to ~1500), clips, discounts
    and done rates: the automatic choice and every forced serial kernel bit-equal to the oracle."""
    rng = np.random.default_rng(1234 + seed)
    for case in range(10):
        S = int(rng.integers(1, 5000))
        H = int(rng.choice([rng.integers(2, 48), rng.integers(48, 400), rng.integers(400, 1500)]))
        if case % 3 == 0:
            H = (H + 3) // 4 * 4
        wl = Workload("fuzz", S, H, seed=int(rng.integers(1 << 30)), done_p=float(rng.choice([0.0, 0.01, 0.3, 1.0])),
                      gamma=float(rng.uniform(0.8, 1.0)), lam=float(rng.uniform(0.0, 1.0)),
                      rho_clip=float(rng.choice([0.0, 0.5, 1.0, 4.0])), c_clip=float(rng.choice([0.0, 0.9, 1.0, 2.5])),
                      importance_sigma=float(rng.choice([0.1, 1.0])), value_sigma=float(rng.choice([1.0, 10.0])))
        inputs = [t.numpy() for t in make_inputs(wl)]
        want = oracle_advantage(inputs, wl.hyper())
        exact = np.abs(want[:, :-1].astype(np.float64)).sum(1)
        got, abs_sum, kernel = run_gpu(inputs, wl.hyper(), "serial", None, epilogue=True)
        assert bits_equal(got, want), f"auto({kernel}) S={S} H={H}: {first_mismatch(got, want)}"
        np.testing.assert_allclose(abs_sum, exact, rtol=1e-5, atol=1e-6)
        for force, ws in (("tma2d", 0), ("tma2d", 4), ("bulk1d", 0), ("bulk1d", 1), ("generic", None)):
            if not applicable(force, H):
                continue
            got, abs_sum, kernel = run_gpu(inputs, wl.hyper(), "serial", force, epilogue=True, ws=ws)
            assert bits_equal(got, want), f"{force}/{ws} S={S} H={H} {wl}: {first_mismatch(got, want)}"
            np.testing.assert_allclose(abs_sum, exact, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("force,H", [("tma2d", 64), ("tma2d", 36), ("bulk1d", 91), ("bulk1d", 30),
                                     ("scan", 64), ("scan", 333), ("generic", 17)])
def test_canaries_around_buffers(force, H):
    """Inputs and outputs live inside larger canary-filled allocations; nothing
    outside advantages[:, :H-1] may change."""
    from pufferlib_b200.advantage import launch_raw
    S, pad = 77, 256
    wl = Workload("canary", S, H, seed=41 + H)
    host = make_inputs(wl)
    n = S * H
    bufs = [torch.full((n + 2 * pad,), 777.0, device="cuda") for _ in range(5)]
    views = [b[pad:pad + n].view(S, H) for b in bufs]
    for v, h in zip(views[:4], host):
        v.copy_(h)
    views[4].fill_(SENTINEL)
    before = [b.clone() for b in bufs[:4]]
    abs_buf = torch.full((S + 2 * pad,), 777.0, device="cuda")
    from pufferlib_b200 import cabi
    cabi.set_tuning(force_kernel=FORCE[force])
    launch_raw(*views, *wl.hyper(), seg_abs_sum=abs_buf[pad:pad + S], variant="scan" if force == "scan" else "serial")
    torch.cuda.synchronize()
    for b, b0 in zip(bufs[:4], before):
        assert torch.equal(b, b0)
    out = bufs[4].cpu().numpy()
    assert np.all(out[:pad] == 777.0) and np.all(out[pad + n:] == 777.0)
    a = abs_buf.cpu().numpy()
    assert np.all(a[:pad] == 777.0) and np.all(a[pad + S:] == 777.0)
    adv = out[pad:pad + n].reshape(S, H)
    assert np.all(adv[:, -1] == np.float32(SENTINEL))
    want = oracle_advantage([t.numpy() for t in host], wl.hyper())
    if force == "scan":
        assert within_scan_tolerance(adv[:, :-1], want[:, :-1])
    else:
        assert bits_equal(adv, want), first_mismatch(adv, want)


def test_misaligned_base_pointer_uses_generic():
    """A view whose data pointer is only 4-byte aligned still works, bit-exactly."""
    from pufferlib_b200 import cabi
    from pufferlib_b200.advantage import launch_raw
    wl = Workload("mis", 50, 64, seed=77)
    host = make_inputs(wl)
    n = 50 * 64
    views = []
    for h in host:
        b = torch.zeros(n + 8, device="cuda")
        v = b[1:1 + n].view(50, 64)
        v.copy_(h)
        views.append(v)
    out = torch.full((n + 8,), SENTINEL, device="cuda")
    adv = out[3:3 + n].view(50, 64)
    launch_raw(*views, adv, *wl.hyper(), variant="serial")
    assert cabi.last_kernel() == "generic"
    want = oracle_advantage([t.numpy() for t in host], wl.hyper())
    assert bits_equal(adv.cpu().numpy(), want)
    launch_raw(*views, adv, *wl.hyper(), variant="scan")
    assert cabi.last_kernel() == "scan"
    assert within_scan_tolerance(adv.cpu().numpy()[:, :-1], want[:, :-1])


# ---------------------------------------------------------------------------
# size-independent properties at full size
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("name,variant", [("cfg2", "serial"), ("cfg4", "serial"), ("cfg3", "scan")])
def test_power_of_two_scaling_is_exact(name, variant):
    """The op is linear in (values, rewards): scaling both by 4 scales every
    output by exactly 4 (a power of two commutes with fp32 rounding)."""
    wl = WORKLOADS[name]
    v, r, d, w = [t.numpy() for t in make_inputs(wl)]
    base, _, _ = run_gpu([v, r, d, w], wl.hyper(), variant)
    scaled, _, _ = run_gpu([v * 4, r * 4, d, w], wl.hyper(), variant)
    assert bits_equal(scaled[:, :-1], base[:, :-1] * 4)


def test_row_slices_equal_full_result():
    """Rows are independent: any contiguous row block alone reproduces its
    slice of the full result bit for bit (this is what sharding relies on)."""
    wl = WORKLOADS["cfg2"].with_segments(20000)
    inputs = [t.numpy() for t in make_inputs(wl)]
    full, full_abs, _ = run_gpu(inputs, wl.hyper(), "serial", epilogue=True)
    for lo, hi in ((0, 4999), (4999, 12345), (12345, 20000)):
        part, part_abs, _ = run_gpu([a[lo:hi] for a in inputs], wl.hyper(), "serial", epilogue=True)
        assert bits_equal(part, full[lo:hi])
        assert bits_equal(part_abs, full_abs[lo:hi])


def test_hyperparameter_edges():
    wl = Workload("edge", 129, 64, seed=55, importance_sigma=1.0)
    inputs = [t.numpy() for t in make_inputs(wl)]
    for hyper in ((0.99, 0.95, 1.0, 0.0), (1.0, 1.0, 5.0, 5.0), (0.0, 0.95, 1.0, 1.0), (0.99, 0.0, 0.1, 0.1)):
        want = oracle_advantage(inputs, hyper)
        for force in ("tma2d", "bulk1d", "generic"):
            got, _, _ = run_gpu(inputs, hyper, "serial", force)
            assert bits_equal(got, want), (hyper, force, first_mismatch(got, want))
        if hyper[0] * hyper[1] * hyper[3] > 1.0:
            continue   # k_t can exceed 1: the recurrence amplifies rounding, outside the scan variant's bar
        got, _, _ = run_gpu(inputs, hyper, "scan")
        assert within_scan_tolerance(got[:, :-1], want[:, :-1]), hyper
    ones = [inputs[0], inputs[1], np.ones_like(inputs[2]), inputs[3]]
    want = oracle_advantage(ones, wl.hyper())
    for variant in ("serial", "scan"):
        got, _, _ = run_gpu(ones, wl.hyper(), variant)
        assert bits_equal(got, want)   # all episodes end every step: no carry, so scan is exact too


def test_products_near_overflow_follow_the_reference_order():
    """(gamma*lambda*c*A)*nn turns into NaN in the reference when the inner
    product overflows and nn == 0; the kernels must reproduce that, not the
    re-associated (gamma*lambda*c*nn)*A == 0."""
    S, H = 40, 64
    rng = np.random.default_rng(5)
    v = rng.standard_normal((S, H)).astype(np.float32)
    r = rng.standard_normal((S, H)).astype(np.float32)
    d = (rng.random((S, H)) < 0.2).astype(np.float32)
    w = np.full((S, H), 4.0, dtype=np.float32)
    r[:, 40] = 2.5e38          # the advantage at column 39 becomes ~1e38 * rho
    d[:, 39] = 1.0             # and the step at column 38 multiplies its overflowed product by nn = 0
    d[:, 40] = 0.0
    hyper = (1.0, 1.0, 1.0, 4.0)
    want = oracle_advantage([v, r, d, w], hyper)
    assert np.isnan(want[:, 38]).all()
    for force in ("tma2d", "bulk1d", "generic"):
        got, _, _ = run_gpu([v, r, d, w], hyper, "serial", force)
        assert bits_equal(got, want), (force, first_mismatch(got, want))


@pytest.mark.parametrize("H", [64, 256, 127])
def test_huge_gain_overflow_follows_the_reference_order(H):
    """The same overflow reached through the gain instead of the advantage:
    c = min(w, c_clip) = 1e12 (or a hugely negative ratio) against a moderate
    A.  Enough rows that every kernel form is exercised, with and without the
    warp-specialised pipeline."""
    S = 6000
    rng = np.random.default_rng(17)
    v = rng.standard_normal((S, H)).astype(np.float32)
    r = (0.1 * rng.standard_normal((S, H))).astype(np.float32)
    d = (rng.random((S, H)) < 0.05).astype(np.float32)
    w = np.exp(0.3 * rng.standard_normal((S, H))).astype(np.float32)
    rows = np.arange(0, S, 7)
    t0 = H - 10
    r[rows, t0 + 1] = 1e29
    d[rows, t0 + 1] = 0.0
    d[rows, t0] = 1.0
    w[rows, t0 - 1] = 1e12
    rows2 = np.arange(3, S, 11)
    r[rows2, 21] = 1e10
    d[rows2, 21] = 0.0
    d[rows2, 20] = 1.0
    w[rows2, 19] = -1e30
    hyper = (0.99, 0.95, 1.0, 1e12)
    want = oracle_advantage([v, r, d, w], hyper)
    assert np.isnan(want[rows, 0]).all() and np.isnan(want[rows2, 0]).all()
    for force, ws in (("tma2d", 0), ("tma2d", 4), ("bulk1d", 0), ("bulk1d", 1), ("generic", None)):
        if not applicable(force, H):
            continue
        got, _, kernel = run_gpu([v, r, d, w], hyper, "serial", force, ws=ws)
        assert kernel == force
        assert bits_equal(got, want), (force, ws, first_mismatch(got, want))
    got, _, _ = run_gpu([v, r, d, w], hyper, "scan")
    assert np.array_equal(np.isnan(got), np.isnan(want))


def test_non_binary_dones_are_used_arithmetically():
    """dones enter as 1 - d (pufferlib.cpp:34), not as a branch: fractional
    values must give the reference's bits on every serial kernel."""
    wl = Workload("frac", 70, 128, seed=91)
    v, r, d, w = [t.numpy() for t in make_inputs(wl)]
    d = np.random.default_rng(3).random(d.shape).astype(np.float32)
    d[::3] = (d[::3] > 0.5)          # a mix of binary and fractional rows inside every tile
    want = oracle_advantage([v, r, d, w], wl.hyper())
    for force in ("tma2d", "bulk1d", "generic"):
        got, _, _ = run_gpu([v, r, d, w], wl.hyper(), "serial", force)
        assert bits_equal(got, want), (force, first_mismatch(got, want))


@pytest.mark.parametrize("force", ["tma2d", "bulk1d", "scan", "generic"])
def test_zero_last_column_flag(force):
    """PUFF_FLAG_ZERO_LAST_COLUMN: the op owns the output and writes column H-1 = 0,
    i.e. it reproduces the reference called on a zero-filled buffer (pufferl.py:353)
    even when the buffer held garbage."""
    from pufferlib_b200 import cabi
    for S, H in ((70, 64), (33, 36), (5, 1), (9, 2), (300, 91), (64, 256), (20, 1024)):
        if not applicable(force, H):
            continue
        wl = Workload("zl", S, H, seed=300 + H)
        inputs = [t.numpy() for t in make_inputs(wl)]
        variant = "scan" if force == "scan" else "serial"
        got, _, _ = run_gpu(inputs, wl.hyper(), variant, force, flags=cabi.FLAG_ZERO_LAST_COLUMN)
        want = oracle_advantage(inputs, wl.hyper(), sentinel=0.0)
        assert np.all(got[:, -1] == 0.0), (S, H)
        if force == "scan":
            assert within_scan_tolerance(got, want), (S, H)
        else:
            assert bits_equal(got, want), f"S={S} H={H}: {first_mismatch(got, want)}"


def test_large_config_zero_last_column():
    from pufferlib_b200 import cabi
    wl = WORKLOADS["cfg2"].with_segments(40000)
    inputs = [t.numpy() for t in make_inputs(wl)]
    got, abs_sum, kernel = run_gpu(inputs, wl.hyper(), "serial", epilogue=True, flags=cabi.FLAG_ZERO_LAST_COLUMN)
    want = oracle_advantage(inputs, wl.hyper(), sentinel=0.0)
    assert kernel == "tma2d" and bits_equal(got, want), first_mismatch(got, want)


# ---------------------------------------------------------------------------
# both forms of the tma2d kernel (single-warp and warp-specialised) on the
# cases that normally only reach one of them
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("ws", [0, 2, 3, 4, 6])
def test_tma2d_forms_match_golden(golden_small, ws):
    for name, case in golden_small.items():
        H = case["values"].shape[1]
        if H % 4 or H < 2:
            continue
        got, _, kernel = run_gpu([case[k] for k in KEYS], case["hyper"], "serial", "tma2d", ws=ws)
        assert kernel == "tma2d"
        assert bits_equal(got, case["advantages"]), f"{name}/ws={ws}: {first_mismatch(got, case['advantages'])}"


@pytest.mark.parametrize("ws", [0, 4])
def test_tma2d_forms_shape_sweep(ws):
    seed = 500
    for S in (1, 31, 33, 64, 70, 257):
        for H in (4, 8, 28, 32, 36, 60, 64, 68, 96, 128, 132, 256, 260):
            wl = Workload("ws", S, H, seed=seed, done_p=0.1)
            seed += 1
            inputs = [t.numpy() for t in make_inputs(wl)]
            got, abs_sum, _ = run_gpu(inputs, wl.hyper(), "serial", "tma2d", epilogue=True, ws=ws)
            want = oracle_advantage(inputs, wl.hyper())
            assert bits_equal(got, want), f"S={S} H={H} ws={ws}: {first_mismatch(got, want)}"
            exact = np.abs(want[:, :-1].astype(np.float64)).sum(1)
            np.testing.assert_allclose(abs_sum, exact, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("ws", [0, 3, 4])
def test_tma2d_forms_literal_paths(ws):
    """Non-binary dones and products near overflow send a chunk down the
    literal path: from the shared-memory stage in the single-warp form, from
    global memory in the warp-specialised form."""
    wl = Workload("lit", 300, 192, seed=77)
    v, r, d, w = [t.numpy() for t in make_inputs(wl)]
    d = np.random.default_rng(9).random(d.shape).astype(np.float32)
    d[::2] = (d[::2] > 0.7)
    want = oracle_advantage([v, r, d, w], wl.hyper())
    got, _, _ = run_gpu([v, r, d, w], wl.hyper(), "serial", "tma2d", ws=ws)
    assert bits_equal(got, want), first_mismatch(got, want)
    # overflow of (gamma*lambda*c)*A with nn == 0 -> NaN in the reference
    rng = np.random.default_rng(5)
    S, H = 80, 128
    v = rng.standard_normal((S, H)).astype(np.float32)
    r = rng.standard_normal((S, H)).astype(np.float32)
    d = (rng.random((S, H)) < 0.2).astype(np.float32)
    w = np.full((S, H), 4.0, dtype=np.float32)
    r[:, 100] = 2.5e38
    d[:, 99] = 1.0
    d[:, 100] = 0.0
    hyper = (1.0, 1.0, 1.0, 4.0)
    want = oracle_advantage([v, r, d, w], hyper)
    assert np.isnan(want[:, 98]).all()
    got, _, _ = run_gpu([v, r, d, w], hyper, "serial", "tma2d", ws=ws)
    assert bits_equal(got, want), first_mismatch(got, want)


@pytest.mark.parametrize("H,force", [(256, "tma2d"), (127, "bulk1d")])
def test_more_than_2_31_elements(H, force):
    """Element offsets beyond 2^31 (the reference's `int` offsets overflow there,
    cuda/pufferlib.cu:48).  The buffer is a small block of rows repeated, so any
    row block of the result must equal the oracle's result for that block."""
    from pufferlib_b200.advantage import launch_raw
    free, _ = torch.cuda.mem_get_info()
    base_rows = 4096
    reps = (2 ** 31) // (base_rows * H) + 3
    S = base_rows * reps
    need = 5 * S * H * 4 + (2 << 30)
    if free < need:
        pytest.skip(f"needs {need >> 30} GiB of free device memory")
    wl = Workload("huge", base_rows, H, seed=123, done_p=0.02)
    host = make_inputs(wl)
    want = torch.from_numpy(oracle_advantage([t.numpy() for t in host], wl.hyper(), sentinel=SENTINEL)).cuda()
    dev = [t.cuda().repeat(reps, 1) for t in host]
    assert dev[0].numel() > 2 ** 31
    adv = torch.full((S, H), SENTINEL, device="cuda")
    abs_sum = torch.empty(S, device="cuda")
    launch_raw(*dev, adv, *wl.hyper(), seg_abs_sum=abs_sum, variant="serial")
    torch.cuda.synchronize()
    from pufferlib_b200 import cabi
    assert cabi.last_kernel() == force and cabi.device_status() == 0
    for rep in (0, reps // 2, reps - 1):
        got = adv[rep * base_rows:(rep + 1) * base_rows]
        assert torch.equal(got.view(torch.int32), want.view(torch.int32)), rep
    first = abs_sum[:base_rows]
    assert torch.equal(abs_sum[(reps - 1) * base_rows:], first)
    del dev, adv
    torch.cuda.empty_cache()


@pytest.mark.parametrize("ws,warp_teams", [(0, 1), (0, 0), (1, None)],
                         ids=["one_stage_tile_per_warp", "one_stage_tile_per_cta", "pipeline"])
def test_bulk1d_forms(ws, warp_teams, golden_small):
    """The forms of the odd-horizon kernel -- one stage with a tile per warp (H <= 144) or per
    CTA, and the warp-specialised pipeline: golden cases, ragged shapes, many tiles per CTA,
    literal path, fused sums, last column."""
    from pufferlib_b200 import cabi
    import functools
    run = functools.partial(run_gpu, warp_teams=warp_teams)
    for name, case in golden_small.items():
        if case["values"].shape[1] < 2:
            continue
        got, _, kernel = run([case[k] for k in KEYS], case["hyper"], "serial", "bulk1d", ws=ws)
        assert kernel == "bulk1d"
        assert bits_equal(got, case["advantages"]), f"{name}/ws={ws}: {first_mismatch(got, case['advantages'])}"
    seed = 900
    for S, H in ((1, 2), (3, 3), (33, 5), (70, 91), (1000, 127), (9000, 33), (5000, 91), (257, 301), (40, 1101), (64, 64)):
        wl = Workload("b1", S, H, seed=seed, done_p=0.1)
        seed += 1
        inputs = [t.numpy() for t in make_inputs(wl)]
        got, abs_sum, _ = run(inputs, wl.hyper(), "serial", "bulk1d", epilogue=True, ws=ws)
        want = oracle_advantage(inputs, wl.hyper())
        assert bits_equal(got, want), f"S={S} H={H} ws={ws}: {first_mismatch(got, want)}"
        exact = np.abs(want[:, :-1].astype(np.float64)).sum(1)
        np.testing.assert_allclose(abs_sum, exact, rtol=1e-5, atol=1e-6)
        got0, _, _ = run(inputs, wl.hyper(), "serial", "bulk1d", ws=ws, flags=cabi.FLAG_ZERO_LAST_COLUMN)
        assert bits_equal(got0, oracle_advantage(inputs, wl.hyper(), sentinel=0.0)), (S, H, ws)
    wl = Workload("b1frac", 500, 91, seed=77)
    v, r, d, w = [t.numpy() for t in make_inputs(wl)]
    d = np.random.default_rng(2).random(d.shape).astype(np.float32)
    want = oracle_advantage([v, r, d, w], wl.hyper())
    got, _, _ = run([v, r, d, w], wl.hyper(), "serial", "bulk1d", ws=ws)
    assert bits_equal(got, want), first_mismatch(got, want)
