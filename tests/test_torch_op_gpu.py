"""GPU: the torch operator boundary, the host-buffer entry point and the
priority kernels."""
import numpy as np
import pytest
import torch

from helpers import SENTINEL, bits_equal, first_mismatch, oracle_advantage
from pufferlib_b200.workloads import WORKLOADS, Workload, make_inputs

pytestmark = pytest.mark.gpu


def test_op_in_place_contract_and_return():
    import pufferlib_b200
    wl = WORKLOADS["cfg0"]
    host = make_inputs(wl)
    dev = [t.cuda() for t in host]
    adv = torch.full_like(dev[0], SENTINEL)
    out = pufferlib_b200.compute_puff_advantage(*dev, adv, *wl.hyper())
    assert out is adv
    want = oracle_advantage([t.numpy() for t in host], wl.hyper())
    assert bits_equal(adv.cpu().numpy(), want), first_mismatch(adv.cpu().numpy(), want)
    for t, h in zip(dev, host):
        assert torch.equal(t.cpu(), h)   # inputs are not modified despite the (a!) annotations


def test_op_called_like_the_trainer():
    """pufferl.py:352-356: zeros, call through torch.ops with python floats."""
    from pufferlib_b200 import _C  # noqa: F401
    wl = WORKLOADS["cfg1"]
    host = make_inputs(wl)
    values, rewards, terminals, ratio = [t.cuda() for t in host]
    advantages = torch.zeros(values.shape, device="cuda")
    r = torch.ops.pufferlib.compute_puff_advantage(values, rewards, terminals, ratio, advantages,
                                                   0.99, 0.95, 1.0, 1.0)
    assert r is None
    want = oracle_advantage([t.numpy() for t in host], wl.hyper(), sentinel=0.0)
    assert bits_equal(advantages.cpu().numpy(), want)


def test_op_runs_on_the_current_stream():
    import pufferlib_b200
    wl = Workload("stream", 4096, 128, seed=5)
    host = make_inputs(wl)
    want = oracle_advantage([t.numpy() for t in host], wl.hyper())
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        dev = [t.cuda(non_blocking=True) for t in host]
        adv = torch.full_like(dev[0], SENTINEL)
        pufferlib_b200.compute_puff_advantage(*dev, adv, *wl.hyper())
        got = adv.cpu()
    side.synchronize()
    assert bits_equal(got.numpy(), want)


def test_op_rejects_bad_arguments():
    import pufferlib_b200
    wl = Workload("bad", 16, 32)
    v, r, d, w = [t.cuda() for t in make_inputs(wl)]
    adv = torch.zeros_like(v)
    hyper = wl.hyper()
    with pytest.raises(RuntimeError, match="contiguous"):
        pufferlib_b200.compute_puff_advantage(v.t().contiguous().t(), r, d, w, adv, *hyper)
    with pytest.raises(RuntimeError, match="float32"):
        pufferlib_b200.compute_puff_advantage(v, r.double(), d, w, adv, *hyper)
    with pytest.raises(RuntimeError, match="Second dimension"):
        pufferlib_b200.compute_puff_advantage(v, r[:, :16].contiguous(), d, w, adv, *hyper)
    with pytest.raises(RuntimeError, match="First dimension"):
        pufferlib_b200.compute_puff_advantage(v, r, d[:8].contiguous(), w, adv, *hyper)
    with pytest.raises(RuntimeError, match="2D"):
        pufferlib_b200.compute_puff_advantage(v, r, d, w.reshape(-1), adv, *hyper)
    with pytest.raises(RuntimeError, match="same device"):
        pufferlib_b200.compute_puff_advantage(v, r, d, w, adv.cpu(), *hyper)
    with pytest.raises(RuntimeError, match="overlap"):
        pufferlib_b200.compute_puff_advantage(v, r, d, w, v, *hyper)
    with pytest.raises((RuntimeError, NotImplementedError)):
        pufferlib_b200.compute_puff_advantage(v.cpu(), r.cpu(), d.cpu(), w.cpu(), adv.cpu(), *hyper)
    assert torch.all(adv == 0)


def test_op_empty_and_degenerate_shapes():
    import pufferlib_b200
    for shape in ((0, 64), (5, 1), (0, 0), (3, 0)):
        t = [torch.zeros(shape, device="cuda") for _ in range(4)]
        adv = torch.full(shape, SENTINEL, device="cuda")
        pufferlib_b200.compute_puff_advantage(*t, adv, 0.99, 0.95, 1.0, 1.0)
        torch.cuda.synchronize()
        assert torch.all(adv == SENTINEL)
    s = torch.full((5,), 9.0, device="cuda")
    t = [torch.zeros((5, 1), device="cuda") for _ in range(5)]
    pufferlib_b200.compute_puff_advantage_prio(*t, s, 0.99, 0.95, 1.0, 1.0)
    assert torch.all(s == 0)


def test_fill_op_needs_no_zeroed_buffer():
    import pufferlib_b200
    wl = WORKLOADS["cfg1"]
    host = make_inputs(wl)
    dev = [t.cuda() for t in host]
    garbage = torch.full_like(dev[0], float("nan"))
    abs_sum = torch.empty(wl.segments, device="cuda")
    out = pufferlib_b200.compute_puff_advantage_fill(*dev, *wl.hyper(), advantages=garbage, seg_abs_sum=abs_sum)
    assert out is garbage
    want = oracle_advantage([t.numpy() for t in host], wl.hyper(), sentinel=0.0)
    assert bits_equal(out.cpu().numpy(), want)
    fresh = pufferlib_b200.compute_puff_advantage_fill(*dev, *wl.hyper())
    assert bits_equal(fresh.cpu().numpy(), want)
    # identical to the reference sequence zeros -> op
    zeros = torch.zeros_like(dev[0])
    pufferlib_b200.compute_puff_advantage(*dev, zeros, *wl.hyper())
    assert torch.equal(zeros, fresh)


def test_meta_kernel_traces():
    from pufferlib_b200 import _C  # noqa: F401
    t = [torch.empty(8, 16, device="meta") for _ in range(5)]
    torch.ops.pufferlib.compute_puff_advantage(*t, 0.99, 0.95, 1.0, 1.0)


@pytest.mark.parametrize("name", ["cfg0", "cfg4", "cfg1"])
def test_host_entry_point(name):
    import pufferlib_b200
    wl = WORKLOADS[name]
    host = make_inputs(wl, pin=True)
    adv = torch.full(host[0].shape, SENTINEL).pin_memory()
    abs_sum = torch.full((wl.segments,), -1.0).pin_memory()
    pufferlib_b200.compute_puff_advantage_host(*host, adv, *wl.hyper(), seg_abs_sum=abs_sum, variant="serial")
    want = oracle_advantage([t.numpy() for t in host], wl.hyper())
    assert bits_equal(adv.numpy(), want), first_mismatch(adv.numpy(), want)
    exact = np.abs(want[:, :-1].astype(np.float64)).sum(1)
    np.testing.assert_allclose(abs_sum.numpy(), exact, rtol=1e-5, atol=1e-6)


def test_host_entry_point_reports_a_given_up_wait():
    """A bounded wait that gave up inside a kernel leaves the output
    incomplete; the synchronous host entry point must return
    PUFF_ERR_DEVICE_WAIT for it, not success.  The status word is set from the
    host here (no kernel is made to wait)."""
    import pufferlib_b200
    from pufferlib_b200 import cabi
    lib = cabi.load()
    wl = WORKLOADS["cfg0"]
    host = make_inputs(wl)
    adv = torch.zeros_like(host[0])
    assert cabi.device_status() == 0
    assert lib.puff_advantage_sm100_inject_status(cabi.ERR_DEVICE_WAIT) == 0
    with pytest.raises(RuntimeError, match="bounded wait"):
        pufferlib_b200.compute_puff_advantage_host(*host, adv, *wl.hyper())
    assert cabi.device_status() == 0                       # reported once, then cleared
    pufferlib_b200.compute_puff_advantage_host(*host, adv, *wl.hyper())   # and the next call is clean
    want = oracle_advantage([t.numpy() for t in host], wl.hyper(), sentinel=0.0)
    assert bits_equal(adv.numpy(), want)


def test_host_entry_point_many_blocks(monkeypatch):
    """Small row blocks so that the slot ring wraps many times; pageable memory."""
    import pufferlib_b200
    monkeypatch.setenv("PUFF_HOST_BLOCK_BYTES", str(64 * 1024))
    wl = Workload("blocks", 5000, 96, seed=8)
    host = make_inputs(wl)
    adv = torch.full(host[0].shape, SENTINEL)
    pufferlib_b200.compute_puff_advantage_host(*host, adv, *wl.hyper())
    want = oracle_advantage([t.numpy() for t in host], wl.hyper())
    assert bits_equal(adv.numpy(), want), first_mismatch(adv.numpy(), want)
    from pufferlib_b200 import cabi
    assert cabi.load().puff_advantage_sm100_host_release(0) == 0


@pytest.mark.parametrize("alpha", [0.8, 0.0, 1.0, 0.35])
def test_priorities_match_oracle_and_torch(alpha):
    import pufferlib_b200
    from oracle import puff_oracle
    wl = WORKLOADS["cfg4"]
    host = make_inputs(wl)
    dev = [t.cuda() for t in host]
    adv = torch.zeros_like(dev[0])
    adv, probs = pufferlib_b200.prioritized_sample_probs(*dev, adv, *wl.hyper(), alpha)
    want = oracle_advantage([t.numpy() for t in host], wl.hyper(), sentinel=0.0)
    w, p, tot = puff_oracle.priorities(puff_oracle.abs_sum(want), alpha)
    np.testing.assert_allclose(probs.cpu().numpy(), p, rtol=2e-5)
    # and the reference's own eager sequence (pufferl.py:359-361) on the same advantages
    a = adv.abs().sum(axis=1)
    pw = torch.nan_to_num(a ** alpha, 0, 0, 0)
    pp = (pw + 1e-6) / (pw.sum() + 1e-6)
    np.testing.assert_allclose(probs.cpu().numpy(), pp.cpu().numpy(), rtol=2e-5)
    assert abs(float(probs.double().sum()) - 1.0) < 1e-3


def test_priorities_non_finite_sums_become_zero_weight():
    import pufferlib_b200
    s = torch.tensor([1.0, float("nan"), float("inf"), 0.0, 2.0], device="cuda")
    w, tot = pufferlib_b200.priority_weights(s, 0.5)
    assert w.cpu().tolist() == pytest.approx([1.0, 0.0, 0.0, 0.0, 2.0 ** 0.5], rel=1e-6)
    assert float(tot) == pytest.approx(1.0 + 2.0 ** 0.5, rel=1e-6)


def test_standalone_nvcc_harness(tmp_path):
    """A torch-free nvcc program drives the C ABI (the reference's harness style)."""
    import os
    import shutil
    import subprocess
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    libdir = os.path.join(root, "pufferlib_b200")
    exe = str(tmp_path / "harness")
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-o", exe,
                    os.path.join(root, "tests", "harness_puff_advantage.cu"),
                    f"-L{libdir}", "-lpuff_advantage_sm100", "-Xlinker", f"-rpath={libdir}"], check=True)
    out = subprocess.run([exe], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "OK" in out.stdout


@pytest.mark.parametrize("S,H,M", [(8192, 64, 512), (1000, 91, 333), (64, 256, 64), (50, 1, 7), (300, 128, 1),
                                   (8192, 256, 8192), (20000, 512, 12000), (4096, 260, 5000), (3000, 8, 9000)])
def test_minibatch_gather_matches_oracle_and_torch(S, H, M):
    """pufferl.py:363, 373-375, 408-409 fused: against the fp64 oracle and the
    eager torch sequence on the same device."""
    import pufferlib_b200
    from oracle import puff_oracle
    g = torch.Generator().manual_seed(S + H)
    adv = torch.randn(S, H, generator=g)
    adv[:, -1] = 0
    val = torch.randn(S, H, generator=g)
    probs = torch.rand(S, generator=g) + 0.01
    probs = probs / probs.sum()
    idx = torch.multinomial(probs, M, replacement=M > S, generator=g)
    beta = 0.35
    d_adv, d_val, d_probs, d_idx = adv.cuda(), val.cuda(), probs.cuda(), idx.cuda()
    mv, mr, ma, an, mp = pufferlib_b200.minibatch_gather(d_adv, d_val, d_probs, d_idx, beta)
    assert mp.shape == (M, 1)
    # gathers are exact
    assert torch.equal(mv, d_val[d_idx]) and torch.equal(ma, d_adv[d_idx])
    assert torch.equal(mr, d_adv[d_idx] + d_val[d_idx])
    o_v, o_r, o_n, o_p = puff_oracle.minibatch(adv.numpy(), val.numpy(), probs.double().numpy(), idx.numpy(), beta)
    np.testing.assert_allclose(mp.cpu().numpy()[:, 0], o_p, rtol=1e-5)
    if M * H > 1:
        np.testing.assert_allclose(an.cpu().numpy(), o_n, rtol=1e-5, atol=2e-6)
        e_prio = (S * d_probs[d_idx, None]) ** -beta
        e_adv = ma
        e_adv = e_prio * (e_adv - e_adv.mean()) / (e_adv.std() + 1e-8)
        np.testing.assert_allclose(an.cpu().numpy(), e_adv.cpu().numpy(), rtol=1e-4, atol=1e-5)
    else:
        assert torch.isnan(an).all()          # std of one element is NaN in the reference as well
    from pufferlib_b200 import cabi
    assert cabi.load().puff_minibatch_sm100_bad_index() == 0


def test_minibatch_gather_flags_bad_indices():
    import pufferlib_b200
    from pufferlib_b200 import cabi
    adv = torch.randn(16, 32, device="cuda")
    val = torch.randn(16, 32, device="cuda")
    probs = torch.full((16,), 1 / 16, device="cuda")
    idx = torch.tensor([0, 3, 99, -1], device="cuda")
    mv, mr, ma, an, mp = pufferlib_b200.minibatch_gather(adv, val, probs, idx, 0.5)
    assert cabi.load().puff_minibatch_sm100_bad_index() == 1
    assert cabi.load().puff_minibatch_sm100_bad_index() == 0      # cleared by the read
    assert torch.equal(mv[:2], val[idx[:2]]) and torch.all(mv[2:] == 0)
    # a bad index is a zero row with zero weight in every output, never inf or NaN
    assert torch.all(mr[2:] == 0) and torch.all(ma[2:] == 0) and torch.all(an[2:] == 0) and torch.all(mp[2:] == 0)
    assert torch.isfinite(an).all() and torch.isfinite(mp).all()


def test_minibatch_gather_of_a_shard_uses_the_global_segment_count():
    """Rows sharded over ranks, probabilities normalised over all of them: the
    N of (N * p) ** -beta (pufferl.py:363) is the global count, passed apart
    from the local row count that bounds the indices."""
    import pufferlib_b200
    g = torch.Generator().manual_seed(11)
    S_global, S_local, H, M, beta = 4096, 1024, 64, 128, 0.6
    adv = torch.randn(S_local, H, generator=g).cuda()
    val = torch.randn(S_local, H, generator=g).cuda()
    probs = (torch.rand(S_local, generator=g) + 0.01).cuda()
    probs = probs / probs.sum() * (S_local / S_global)       # this shard's slice of a global distribution
    idx = torch.randint(0, S_local, (M,), generator=g).cuda()
    *_, an, mp = pufferlib_b200.minibatch_gather(adv, val, probs, idx, beta, prio_segments=S_global)
    e_prio = (S_global * probs[idx, None]) ** -beta
    np.testing.assert_allclose(mp.cpu().numpy(), e_prio.cpu().numpy(), rtol=1e-5)
    e = adv[idx]
    e = e_prio * (e - e.mean()) / (e.std() + 1e-8)
    np.testing.assert_allclose(an.cpu().numpy(), e.cpu().numpy(), rtol=1e-4, atol=1e-5)
    with pytest.raises(RuntimeError):
        pufferlib_b200.minibatch_gather(adv, val, probs, idx, beta, prio_segments=S_local - 1)


def test_rollout_write_matches_the_trainer_assignments():
    """pufferl.py:275, 294-296 in one launch; then the advantage op on the
    buffers it filled equals the op on buffers filled the reference's way."""
    import pufferlib_b200
    S, H, lo, n = 300, 48, 37, 200
    g = torch.Generator().manual_seed(11)
    bufs = [torch.zeros(S, H, device="cuda") for _ in range(3)]
    refs = [torch.zeros(S, H, device="cuda") for _ in range(3)]
    for col in range(H):
        r = (torch.randn(n, generator=g) * 2).cuda()
        r[3] = float("nan")
        d = (torch.rand(n, generator=g) < 0.1).cuda()
        v = torch.randn(n, 1, generator=g).cuda()
        pufferlib_b200.rollout_write(*bufs, r, d, v, lo, col)
        rows = slice(lo, lo + n)
        rc = torch.clamp(r, -1, 1)
        refs[0][rows, col] = rc
        refs[1][rows, col] = d.float()
        refs[2][rows, col] = v.flatten()
    for b, e in zip(bufs, refs):
        assert torch.equal(torch.nan_to_num(b, 7.0), torch.nan_to_num(e, 7.0))
    with pytest.raises(RuntimeError):
        pufferlib_b200.rollout_write(*bufs, r, d, v, S - 10, 0)       # rows past the end
    with pytest.raises(RuntimeError):
        pufferlib_b200.rollout_write(*bufs, r, d, v, 0, H)            # column past the end


def test_op_replays_from_a_cuda_graph():
    """After one eager call per device the launch path makes no synchronising or
    allocating call, so the op can be captured and replayed."""
    import pufferlib_b200
    for wl in (WORKLOADS["cfg1"], Workload("gws", 20000, 64, seed=3), Workload("godd", 700, 91, seed=4)):
        host = make_inputs(wl)
        dev = [t.cuda() for t in host]
        adv = torch.zeros_like(dev[0])
        sums = torch.empty(wl.segments, device="cuda")
        pufferlib_b200.compute_puff_advantage_prio(*dev, adv, sums, *wl.hyper())     # set-up call
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        g = torch.cuda.CUDAGraph()
        adv.fill_(SENTINEL)
        with torch.cuda.graph(g, stream=side):
            pufferlib_b200.compute_puff_advantage_prio(*dev, adv, sums, *wl.hyper())
        adv.fill_(SENTINEL)
        sums.fill_(-1)
        g.replay()
        torch.cuda.synchronize()
        want = oracle_advantage([t.numpy() for t in host], wl.hyper())
        assert bits_equal(adv.cpu().numpy(), want), wl.name
        exact = np.abs(want[:, :-1].astype(np.float64)).sum(1)
        np.testing.assert_allclose(sums.cpu().numpy(), exact, rtol=1e-5, atol=1e-6)


def test_dependent_launches_back_to_back_keep_stream_order():
    """Every kernel of the sampler sequence is launched with programmatic stream
    serialization and waits for its predecessor before its first global access.  The
    sequence advantage -> weights -> probabilities -> gather, issued many times without
    a synchronise in between (eagerly and from one CUDA graph), gives what the same calls
    give one at a time."""
    import pufferlib_b200
    S, H, M, rounds = 4096, 64, 512, 24
    wl = Workload("chain", S, H, seed=21)
    hyper = wl.hyper()
    gen = torch.Generator().manual_seed(5)
    base = [t.cuda() for t in make_inputs(wl)]
    scales = [1.0 + 0.03125 * i for i in range(rounds)]
    inputs = [[base[0] * sc, base[1] * sc, base[2], base[3]] for sc in scales]
    idx = [torch.randint(0, S, (M,), generator=gen).cuda() for _ in range(rounds)]

    def one(i):
        sums = torch.empty(S, device="cuda")
        adv = pufferlib_b200.compute_puff_advantage_fill(*inputs[i], *hyper, seg_abs_sum=sums)
        w, total = pufferlib_b200.priority_weights(sums, 0.6)
        probs = pufferlib_b200.priority_probs(w, total)
        out = pufferlib_b200.minibatch_gather(adv, inputs[i][0], probs, idx[i], 0.4)
        return [adv, probs] + list(out)

    want = []
    for i in range(rounds):
        want.append([t.clone() for t in one(i)])
        torch.cuda.synchronize()
    got = [one(i) for i in range(rounds)]           # no synchronise between the calls
    torch.cuda.synchronize()
    for i in range(rounds):
        for a, b in zip(got[i], want[i]):
            assert torch.equal(a, b), i
    side = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        got = [one(i) for i in range(rounds)]
    for t in (x for row in got for x in row):
        t.fill_(SENTINEL)
    g.replay()
    torch.cuda.synchronize()
    for i in range(rounds):
        for a, b in zip(got[i], want[i]):
            assert torch.equal(a, b), i


def test_concurrent_launches_from_threads_and_streams():
    """The launcher is re-entrant: per-thread tensor-map caches, one-time device
    set-up behind a lock.  Four threads, each on its own stream and buffers."""
    import threading
    import pufferlib_b200
    cases = [Workload(f"t{i}", 3000 + 517 * i, 64 + 32 * (i % 2), seed=40 + i) for i in range(4)]
    hosts = [make_inputs(wl) for wl in cases]
    wants = [oracle_advantage([t.numpy() for t in h], wl.hyper()) for h, wl in zip(hosts, cases)]
    results = [None] * 4
    errors = []

    def work(i):
        try:
            st = torch.cuda.Stream()
            with torch.cuda.stream(st):
                dev = [t.cuda(non_blocking=True) for t in hosts[i]]
                adv = torch.full_like(dev[0], SENTINEL)
                for _ in range(20):
                    pufferlib_b200.compute_puff_advantage(*dev, adv, *cases[i].hyper())
                results[i] = adv.cpu()
            st.synchronize()
        except Exception as exc:   # surfaced below
            errors.append(exc)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for got, want in zip(results, wants):
        assert bits_equal(got.numpy(), want)
