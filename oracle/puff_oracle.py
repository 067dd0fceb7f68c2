"""ctypes front-end of the CPU oracle (test infrastructure, never shipped).

`advantage()` runs oracle/puff_advantage_oracle.c, the plain-C restatement of
the reference CPU op (pufferlib/extensions/pufferlib.cpp:28-41, 63-72).
`load_reference()` loads oracle/_ref/libpufferlib_ref.so -- the reference's own
pufferlib.cpp compiled unmodified with its namespace renamed to
`pufferlib_ref` -- and returns `torch.ops.pufferlib_ref.compute_puff_advantage`
or None when that build is not present.

Only tests/, the smoke check and bench.py's CPU-baseline / reference arms may
import this module.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
# PUFF_ORACLE_LIB names another build of the oracle (a sanitizer build) to load instead
_LIB_PATH = os.environ.get("PUFF_ORACLE_LIB") or os.path.join(_HERE, "libpuff_oracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libpufferlib_ref.so")
_REF_CUDA_PATH = os.path.join(_HERE, "_ref", "libpufferlib_ref_cuda.so")
_lib = None
_ref_loaded = None

_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)


def reference_root():
    """Where the reference checkout is looked for: $PUFFER_REFERENCE_ROOT, else
    a folder `reference` beside this repository.  It need not exist."""
    return os.environ.get("PUFFER_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")


def build(ref=True, ref_cuda=False):
    """Compile the oracle (and, when the reference tree is mounted, the
    reference build under oracle/_ref/).  Existing outputs are kept."""
    targets = ["oracle"]
    ref_root = reference_root()
    have_ref = os.path.isfile(os.path.join(ref_root, "pufferlib", "extensions", "pufferlib.cpp"))
    if ref and have_ref:
        targets.append("ref")
    if ref_cuda and have_ref:
        targets.append("ref_cuda")
    subprocess.run(["make", "-s", "-C", _HERE, f"REF={ref_root}"] + targets, check=True)


def _load():
    global _lib
    if _lib is None:
        if not os.path.isfile(_LIB_PATH):
            build(ref=False)
        lib = ctypes.CDLL(_LIB_PATH)
        lib.puff_oracle_advantage.argtypes = [_f32p] * 5 + [ctypes.c_float] * 4 + [ctypes.c_int64] * 2
        lib.puff_oracle_advantage.restype = None
        lib.puff_oracle_abs_sum.argtypes = [_f32p, _f64p, ctypes.c_int64, ctypes.c_int64]
        lib.puff_oracle_abs_sum.restype = None
        lib.puff_oracle_priorities.argtypes = [_f64p, _f64p, _f64p, ctypes.c_double, ctypes.c_double, ctypes.c_int64]
        lib.puff_oracle_priorities.restype = ctypes.c_double
        _i64p = ctypes.POINTER(ctypes.c_int64)
        lib.puff_oracle_minibatch.argtypes = [_f32p, _f32p, _f64p, _i64p, _f64p, _f64p, _f64p, _f64p,
                                              ctypes.c_double, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64]
        lib.puff_oracle_minibatch.restype = None
        _lib = lib
    return _lib


def _as_f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_f32p)


def advantage(values, rewards, dones, importance, advantages, gamma, lam, rho_clip, c_clip):
    """In-place oracle: fills advantages[:, :H-1], leaves advantages[:, H-1].

    All arrays are C-contiguous float32 numpy arrays of shape [S, H];
    `advantages` is modified and returned.  ctypes releases the GIL during the
    call, so disjoint row slices may be processed from several threads."""
    lib = _load()
    assert advantages.dtype == np.float32 and advantages.flags.c_contiguous
    S, H = values.shape
    for a in (values, rewards, dones, importance, advantages):
        assert a.shape == (S, H) and a.dtype == np.float32 and a.flags.c_contiguous
    lib.puff_oracle_advantage(
        values.ctypes.data_as(_f32p), rewards.ctypes.data_as(_f32p),
        dones.ctypes.data_as(_f32p), importance.ctypes.data_as(_f32p),
        advantages.ctypes.data_as(_f32p),
        np.float32(gamma), np.float32(lam), np.float32(rho_clip), np.float32(c_clip), S, H)
    return advantages


def abs_sum(advantages):
    """float64 per-segment sum of |advantages[:, :H-1]|."""
    lib = _load()
    adv, p = _as_f32(advantages)
    S, H = adv.shape
    out = np.empty(S, dtype=np.float64)
    lib.puff_oracle_abs_sum(p, out.ctypes.data_as(_f64p), S, H)
    return out


def priorities(abs_sums, alpha, total_w=None):
    """(weights, probs, local_sum) of pufferl.py:359-361 in float64."""
    lib = _load()
    a = np.ascontiguousarray(abs_sums, dtype=np.float64)
    w = np.empty_like(a)
    p = np.empty_like(a)
    local = lib.puff_oracle_priorities(
        a.ctypes.data_as(_f64p), w.ctypes.data_as(_f64p), p.ctypes.data_as(_f64p),
        float(alpha), -1.0 if total_w is None else float(total_w), a.shape[0])
    return w, p, local


def minibatch(advantages, values, prio_probs, idx, beta):
    """float64 (mb_values, mb_returns, mb_adv_norm, mb_prio) of pufferl.py:363,
    373-375, 408-409 for int64 segment indices `idx`."""
    lib = _load()
    adv, pa = _as_f32(advantages)
    val, pv = _as_f32(values)
    probs = np.ascontiguousarray(prio_probs, dtype=np.float64)
    ix = np.ascontiguousarray(idx, dtype=np.int64)
    S, H = adv.shape
    M = ix.shape[0]
    out = [np.empty((M, H), dtype=np.float64) for _ in range(3)] + [np.empty(M, dtype=np.float64)]
    lib.puff_oracle_minibatch(pa, pv, probs.ctypes.data_as(_f64p), ix.ctypes.data_as(ctypes.POINTER(ctypes.c_int64)),
                              *[o.ctypes.data_as(_f64p) for o in out], float(beta), S, H, M)
    return tuple(out)


def load_reference(cuda=False):
    """torch.ops.pufferlib_ref.compute_puff_advantage from the reference build,
    or None when oracle/_ref/ has not been built (e.g. the reference tree was
    never mounted on this machine).  With cuda=True the build that also holds
    the reference CUDA kernel is preferred."""
    global _ref_loaded
    import torch
    if _ref_loaded is None:
        path = None
        if cuda and os.path.isfile(_REF_CUDA_PATH):
            path = _REF_CUDA_PATH
        elif os.path.isfile(_REF_PATH):
            path = _REF_PATH
        elif os.path.isfile(_REF_CUDA_PATH):
            path = _REF_CUDA_PATH
        if path is None:
            return None
        torch.ops.load_library(path)
        _ref_loaded = path
    return torch.ops.pufferlib_ref.compute_puff_advantage


def reference_has_cuda():
    return _ref_loaded == _REF_CUDA_PATH
