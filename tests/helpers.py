"""Shared checks for the parity tests (the oracle is the checker here)."""
import hashlib

import numpy as np

SENTINEL = 12345.0


def oracle_advantage(inputs, hyper, sentinel=SENTINEL):
    """Reference result from the CPU oracle for numpy/torch CPU inputs."""
    from oracle import puff_oracle
    arrs = [np.ascontiguousarray(np.asarray(t), dtype=np.float32) for t in inputs]
    adv = np.full(arrs[0].shape, sentinel, dtype=np.float32)
    puff_oracle.advantage(*arrs, adv, *hyper)
    return adv


def bits_equal(a, b):
    """Bitwise equality, except that any NaN matches any NaN (x86 and the GPU
    propagate different NaN payloads)."""
    a = np.asarray(a, dtype=np.float32)
    b = np.asarray(b, dtype=np.float32)
    if a.shape != b.shape:
        return False
    nan = np.isnan(a) & np.isnan(b)
    return bool(np.all((a.view(np.uint32) == b.view(np.uint32)) | nan))


def first_mismatch(a, b):
    a = np.asarray(a, dtype=np.float32)
    b = np.asarray(b, dtype=np.float32)
    bad = (a.view(np.uint32) != b.view(np.uint32)) & ~(np.isnan(a) & np.isnan(b))
    idx = np.argwhere(bad)
    if idx.size == 0:
        return None
    i = tuple(idx[0])
    return f"{int(bad.sum())} mismatches, first at {i}: got {a[i]!r} want {b[i]!r}"


def within_scan_tolerance(a, b, floor=1e-6, rel=1e-5):
    """|a-b| <= max(1e-6, 1e-5*|b|) elementwise: the stated bar for the scan
    variant (max relative error 1e-5 with an absolute floor of 1e-6)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return bool(np.all(np.abs(a - b) <= np.maximum(floor, rel * np.abs(b))))


def sha256_arrays(*arrs):
    h = hashlib.sha256()
    for a in arrs:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()
