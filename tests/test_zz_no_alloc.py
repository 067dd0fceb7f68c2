"""GPU: the allocation-free priority-weights entry point.

Some callers of the C ABI cannot hand the library a scratch buffer: they sit
behind an FFI inside a trainer whose device memory is already fully claimed,
or have no allocator to call at all.  `puff_priorities_sm100_weights_noalloc`
serves them from a fixed array inside the library.  This file checks it
against the ordinary entry point (caller-owned scratch) on two calls in a row
that share that array, the second one smaller than the first so that leftovers
of the first call would show, plus the size limit.

The file name sorts last on purpose: with `-x` every other test has already
run by the time this one does.  It passes on its own in a fresh process too.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _weights_with_caller_scratch(lib, s, alpha):
    n = s.numel()
    weights = torch.empty_like(s)
    total = torch.empty(1, device="cuda", dtype=torch.float64)
    nbytes = lib.puff_priorities_sm100_scratch_bytes(n)
    scratch = torch.empty((nbytes + 7) // 8, device="cuda", dtype=torch.float64)
    rc = lib.puff_priorities_sm100_weights(s.data_ptr(), weights.data_ptr(), total.data_ptr(), alpha, n,
                                           scratch.data_ptr(), nbytes, None)
    assert rc == 0
    torch.cuda.synchronize()
    return weights, total


def _weights_noalloc(lib, s, alpha):
    n = s.numel()
    weights = torch.empty_like(s)
    total = torch.full((1,), -1.0, device="cuda", dtype=torch.float64)
    rc = lib.puff_priorities_sm100_weights_noalloc(s.data_ptr(), weights.data_ptr(), total.data_ptr(),
                                                   alpha, n, None)
    assert rc == 0
    torch.cuda.synchronize()
    return weights, total


def test_noalloc_matches_entry_point_with_caller_scratch():
    from pufferlib_b200 import cabi
    lib = cabi.load()
    g = torch.Generator().manual_seed(123)
    alpha = 0.8
    # two calls in a row on the shared array: large first, then small
    for n in (300_000, 5_000):
        s = (torch.rand(n, generator=g) * 40.0).cuda()
        s[::97] = float("nan")          # non-finite sums get weight 0 (pufferl.py:360)
        s[5::113] = 0.0
        want_w, want_t = _weights_with_caller_scratch(lib, s, alpha)
        got_w, got_t = _weights_noalloc(lib, s, alpha)
        np.testing.assert_allclose(got_w.cpu().numpy(), want_w.cpu().numpy(), rtol=1e-6, atol=0.0)
        np.testing.assert_allclose(got_t.cpu().numpy(), want_t.cpu().numpy(), rtol=1e-12)
        # and against torch's own evaluation of the same formula
        ref = torch.nan_to_num(s.double() ** alpha, 0, 0, 0).sum().item()
        assert abs(got_t.item() - ref) <= 2e-5 * ref


def test_noalloc_rejects_sizes_beyond_its_scratch():
    from pufferlib_b200 import cabi
    lib = cabi.load()
    n = cabi.NOALLOC_MAX_SEGMENTS + 1
    s = torch.ones(n, device="cuda")
    weights = torch.zeros_like(s)
    total = torch.full((1,), -1.0, device="cuda", dtype=torch.float64)
    rc = lib.puff_priorities_sm100_weights_noalloc(s.data_ptr(), weights.data_ptr(), total.data_ptr(), 0.5, n, None)
    assert rc == cabi.ERR_SIZE
    assert "size" in cabi.strerror(rc)
    torch.cuda.synchronize()
    assert total.item() == -1.0 and float(weights.abs().sum()) == 0.0     # nothing ran
    # the largest supported size works
    n = cabi.NOALLOC_MAX_SEGMENTS
    rc = lib.puff_priorities_sm100_weights_noalloc(s.data_ptr(), weights.data_ptr(), total.data_ptr(), 0.5, n, None)
    assert rc == 0
    torch.cuda.synchronize()
    assert total.item() == pytest.approx(float(n), rel=1e-12)
