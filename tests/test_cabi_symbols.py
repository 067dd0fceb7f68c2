"""CPU: the C-ABI library loads and exports what include/puff_advantage.h declares."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "puff_advantage.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(puff_\w+)\s*\(", text)))


def test_header_symbols_exported():
    from pufferlib_b200 import cabi
    lib = ctypes.CDLL(cabi.LIB_PATH)
    names = declared_functions()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert sorted(cabi.SIGNATURES) == names


def test_error_strings_and_validation_without_gpu():
    from pufferlib_b200 import cabi
    lib = cabi.load()
    assert lib.puff_advantage_sm100_version() == b"0.1"
    for code in range(-10, 1):
        assert cabi.strerror(code) not in ("", "unknown error code")
    # argument validation happens before any CUDA call
    z = ctypes.c_void_p(0)
    f = lib.puff_advantage_sm100_launch
    assert f(z, z, z, z, z, z, .9, .9, 1., 1., -1, 4, 0, z) == cabi.ERR_SHAPE
    assert f(z, z, z, z, z, z, .9, .9, 1., 1., 4, 4, 9, z) == cabi.ERR_VARIANT
    assert f(z, z, z, z, z, z, .9, .9, 1., 1., 0, 4, 0, z) == cabi.OK
    assert f(z, z, z, z, z, z, .9, .9, 1., 1., 4, 4, 0, z) == cabi.ERR_NULL
    buf = (ctypes.c_float * 64)()
    p = ctypes.addressof(buf)
    assert f(p + 2, p, p, p, p, z, .9, .9, 1., 1., 2, 4, 0, z) == cabi.ERR_ALIGN
    assert f(p, p, p, p, p, z, .9, .9, 1., 1., 2, 4, 0, z) == cabi.ERR_ALIAS
    assert lib.puff_priorities_sm100_scratch_bytes(1 << 20) >= 8
    assert lib.puff_priorities_sm100_weights(z, z, z, 0.5, 5, z, 0, z) == cabi.ERR_NULL


def test_device_wait_code_becomes_an_exception():
    """The code a launch path returns for a given-up in-kernel wait is a
    RuntimeError on the Python side, like every other failure."""
    from pufferlib_b200 import cabi
    assert "bounded wait" in cabi.strerror(cabi.ERR_DEVICE_WAIT)
    with pytest.raises(RuntimeError, match="bounded wait"):
        cabi.check(cabi.ERR_DEVICE_WAIT, "puff_advantage_sm100_host")
    cabi.check(cabi.OK)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_no_cpu_fallback():
    """Without a GPU the product refuses to compute instead of falling back."""
    from pufferlib_b200 import cabi
    import pufferlib_b200
    lib = cabi.load()
    a = [torch.zeros(4, 8) for _ in range(5)]
    rc = lib.puff_advantage_sm100_launch(*[t.data_ptr() for t in a], None, .9, .9, 1., 1., 4, 8, 0, None)
    assert rc != cabi.OK
    with pytest.raises((RuntimeError, NotImplementedError)):
        pufferlib_b200.compute_puff_advantage(*a, .9, .9, 1., 1.)
    with pytest.raises(RuntimeError):
        pufferlib_b200.compute_puff_advantage_host(*a, .9, .9, 1., 1.)


def test_schema_is_the_reference_schema():
    from pufferlib_b200 import _C  # noqa: F401
    schema = str(torch.ops.pufferlib.compute_puff_advantage.default._schema)
    assert schema == ("pufferlib::compute_puff_advantage(Tensor(a!) values, Tensor(b!) rewards, "
                      "Tensor(c!) dones, Tensor(d!) importance, Tensor(e!) advantages, float gamma, "
                      "float lambda, float rho_clip, float c_clip) -> ()")


def test_every_op_has_a_shape_kernel():
    """Meta (shape-only) kernels: the whole minibatch sequence traces without a GPU."""
    from pufferlib_b200 import _C  # noqa: F401
    ops = torch.ops.pufferlib
    S, H, M = 64, 32, 8
    t = [torch.empty(S, H, device="meta") for _ in range(5)]
    sums = torch.empty(S, device="meta")
    ops.compute_puff_advantage(*t, 0.99, 0.95, 1.0, 1.0)
    ops.compute_puff_advantage_prio(*t, sums, 0.99, 0.95, 1.0, 1.0)
    ops.compute_puff_advantage_fill(*t, sums, 0.99, 0.95, 1.0, 1.0)
    ops.compute_puff_advantage_fill(*t, None, 0.99, 0.95, 1.0, 1.0)
    w, total = ops.puff_priority_weights(sums, 0.8)
    assert w.shape == (S,) and total.shape == (1,) and total.dtype == torch.float64
    p = ops.puff_priority_probs(w, total)
    assert p.shape == (S,)
    idx = torch.empty(M, dtype=torch.int64, device="meta")
    out = ops.puff_minibatch_gather(t[4], t[0], p, idx, 0.5)
    assert [tuple(o.shape) for o in out] == [(M, H)] * 4 + [(M, 1)]
    step = torch.empty(M, device="meta")
    ops.puff_rollout_write(t[1], t[2], t[0], step, torch.empty(M, dtype=torch.bool, device="meta"), step, 0, 3, 1.0)
