"""GPU: the debug build (-DPUFF_DEBUG_BOUNDS) of the kernel library.

Every global-memory index the kernels form is checked in that build; a bad one
is recorded in the status word and its access skipped, nothing traps.  The
release library is left alone: the debug library is built into a scratch folder
and driven through ctypes.  The sweep shows that no kernel form ever forms an
index outside its arrays on small, ragged and multi-tile shapes (and that the
checks do not change a bit of the results); the self-test shows that a bad index
is in fact caught and skipped.
"""
import ctypes
import os
import shutil

import numpy as np
import pytest
import torch

from helpers import SENTINEL, bits_equal, first_mismatch, oracle_advantage, within_scan_tolerance
from pufferlib_b200.workloads import Workload, make_inputs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def debug_lib(tmp_path_factory):
    from pufferlib_b200 import build, cabi
    if not os.path.exists(build.NVCC) and shutil.which("nvcc") is None:
        pytest.skip("nvcc not available")
    path = str(tmp_path_factory.mktemp("dbg") / "libpuff_advantage_sm100_debug.so")
    build.build_debug_cabi(path)
    lib = ctypes.CDLL(path)
    for name, (res, args) in cabi.SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    lib.puff_advantage_sm100_bounds_selftest.restype = ctypes.c_int
    lib.puff_advantage_sm100_bounds_selftest.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_longlong]
    return lib


def launch(lib, inputs, hyper, variant, epilogue=True, **knobs):
    from pufferlib_b200 import cabi
    dev = [torch.as_tensor(t).contiguous().cuda() for t in inputs]
    adv = torch.full_like(dev[0], SENTINEL)
    sums = torch.full((dev[0].shape[0],), -1.0, device="cuda") if epilogue else None
    for k in cabi.TUNE:
        lib.puff_advantage_sm100_set_tuning(cabi.TUNE[k], -1)
    for k, v in knobs.items():
        lib.puff_advantage_sm100_set_tuning(cabi.TUNE[k], v)
    S, H = dev[0].shape
    rc = lib.puff_advantage_sm100_launch(*[t.data_ptr() for t in dev], adv.data_ptr(),
                                         None if sums is None else sums.data_ptr(), *hyper, S, H,
                                         cabi.VARIANTS[variant], torch.cuda.current_stream().cuda_stream)
    assert rc == 0, rc
    kernel = cabi.KERNEL_NAMES[lib.puff_advantage_sm100_last_kernel()]
    status = lib.puff_advantage_sm100_device_status()
    return adv.cpu().numpy(), kernel, status


FORMS = [("serial", dict(force_kernel=1, ws_stages=0)), ("serial", dict(force_kernel=1, ws_stages=4)),
         ("serial", dict(force_kernel=1, ws_stages=2)), ("serial", dict(force_kernel=2, ws_stages=0)),
         ("serial", dict(force_kernel=2, ws_stages=1)), ("scan", {}), ("generic", {})]


def test_no_kernel_form_leaves_its_arrays(debug_lib):
    seed = 400
    for S, H in ((1, 2), (5, 3), (33, 36), (70, 91), (257, 64), (1000, 127), (2100, 256), (6000, 96), (40, 1100)):
        wl = Workload("dbg", S, H, seed=seed, done_p=0.1)
        seed += 1
        inputs = [t.numpy() for t in make_inputs(wl)]
        want = oracle_advantage(inputs, wl.hyper())
        for variant, knobs in FORMS:
            if knobs.get("force_kernel") == 1 and H % 4:
                continue
            got, kernel, status = launch(debug_lib, inputs, wl.hyper(), variant, **knobs)
            assert status == 0, (S, H, variant, knobs, kernel, status)
            if variant == "scan":
                assert within_scan_tolerance(got[:, :-1], want[:, :-1]), (S, H)
            else:
                assert bits_equal(got, want), (S, H, variant, knobs, first_mismatch(got, want))
    # the literal (overflow / non-binary) paths read global memory directly
    wl = Workload("dbgfrac", 300, 192, seed=77)
    v, r, d, w = [t.numpy() for t in make_inputs(wl)]
    d = np.random.default_rng(9).random(d.shape).astype(np.float32)
    want = oracle_advantage([v, r, d, w], wl.hyper())
    for variant, knobs in FORMS[:5]:
        got, _, status = launch(debug_lib, [v, r, d, w], wl.hyper(), variant, **knobs)
        assert status == 0 and bits_equal(got, want), (variant, knobs)


def test_a_bad_index_is_recorded_and_skipped(debug_lib):
    from pufferlib_b200 import cabi
    buf = torch.zeros(8, device="cuda")
    assert debug_lib.puff_advantage_sm100_bounds_selftest(buf.data_ptr(), 3, 8) == 0
    assert debug_lib.puff_advantage_sm100_device_status() == 0
    assert float(buf[3]) == 1.0
    assert debug_lib.puff_advantage_sm100_bounds_selftest(buf.data_ptr(), 8, 8) == 0      # one past the end
    assert debug_lib.puff_advantage_sm100_device_status() == cabi.ERR_DEVICE_BOUNDS
    assert debug_lib.puff_advantage_sm100_device_status() == 0                           # cleared by the read
    assert float(buf.sum()) == 1.0                                                       # the store was skipped
    assert "out-of-range" in debug_lib.puff_advantage_sm100_strerror(cabi.ERR_DEVICE_BOUNDS).decode()
