"""Generate the committed golden fixtures for the advantage path.

Run in a container where the reference tree is mounted and `make -C oracle ref`
has produced oracle/_ref/libpufferlib_ref.so (the reference's own
pufferlib/extensions/pufferlib.cpp, compiled unmodified).  Every output below
comes from torch.ops.pufferlib_ref.compute_puff_advantage, i.e. from the
reference CPU implementation (pufferlib.cpp:75-85), never from this repo's
oracle or kernels.

    python tests/golden/make_golden.py

Writes
  tests/golden/small_cases.npz    inputs + reference outputs of small cases
  tests/golden/config_digests.json  sha256 / samples of the reference output on
                                    the five benchmark configurations (inputs
                                    are regenerated from the seed)
"""
import hashlib
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import puff_oracle  # noqa: E402
from pufferlib_b200.workloads import WORKLOADS, Workload, make_inputs  # noqa: E402

SENTINEL = 12345.0

# (name, workload) -- small enough to commit inputs and outputs verbatim
SMALL = [
    ("h1", Workload("h1", 5, 1)),
    ("h2", Workload("h2", 7, 2, seed=1)),
    ("h3", Workload("h3", 9, 3, seed=2)),
    ("s1", Workload("s1", 1, 64, seed=3)),
    ("tile", Workload("tile", 32, 32, seed=4)),
    ("ragged", Workload("ragged", 37, 45, seed=5, done_p=0.1)),
    ("odd127", Workload("odd127", 33, 127, seed=6, c_clip=0.9, done_p=0.2,
                        importance_sigma=1.0, value_sigma=10.0)),
    ("drive91", Workload("drive91", 40, 91, seed=7, gamma=0.98, lam=0.95)),
    ("cclip0", Workload("cclip0", 16, 64, seed=8, c_clip=0.0)),
    ("rho_hi", Workload("rho_hi", 16, 64, seed=9, rho_clip=3.5, c_clip=2.25, importance_sigma=1.0)),
    ("all_done", Workload("all_done", 8, 36, seed=10, done_p=1.1)),
    ("long", Workload("long", 3, 700, seed=11, gamma=0.999, done_p=0.002)),
]


def run_reference(ref, inputs, hyper):
    v, r, d, w = inputs
    adv = torch.full_like(v, SENTINEL)
    ref(v, r, d, w, adv, *hyper)
    return adv


def main():
    ref = puff_oracle.load_reference()
    if ref is None:
        raise SystemExit("oracle/_ref/libpufferlib_ref.so missing: run `make -C oracle ref`")
    out_dir = os.path.dirname(os.path.abspath(__file__))

    arrays = {}
    meta = {}
    for name, wl in SMALL:
        inputs = make_inputs(wl)
        adv = run_reference(ref, inputs, wl.hyper())
        for key, t in zip(("values", "rewards", "dones", "importance"), inputs):
            arrays[f"{name}.{key}"] = t.numpy()
        arrays[f"{name}.advantages"] = adv.numpy()
        meta[name] = {"hyper": list(wl.hyper()), "segments": wl.segments, "horizon": wl.horizon}
    # non-binary dones and non-finite values: the op uses dones arithmetically
    wl = Workload("special", 12, 40, seed=12)
    v, r, d, w = make_inputs(wl)
    d = torch.rand(d.shape, generator=torch.Generator().manual_seed(99))
    v[3, 17] = float("inf")
    v[5, 5] = float("nan")
    r[7, 30] = -float("inf")
    w[9, 12] = float("nan")
    adv = run_reference(ref, (v, r, d, w), wl.hyper())
    for key, t in zip(("values", "rewards", "dones", "importance"), (v, r, d, w)):
        arrays[f"special.{key}"] = t.numpy()
    arrays["special.advantages"] = adv.numpy()
    meta["special"] = {"hyper": list(wl.hyper()), "segments": 12, "horizon": 40}
    # ((gamma*lambda)*c)*A overflows to inf while nn == 0: the reference then carries inf*0 = NaN
    # to the start of the row, whereas (((gamma*lambda)*c)*nn)*A would be 0.  Rows 0..15 get there
    # through a huge clip and ratio (c = 1e12 against A ~ 1e29), rows 16..31 through a hugely
    # negative ratio (c = min(w, c_clip) = -1e30 against A ~ 1e10); the rest stay finite.
    wl = Workload("gain_overflow", 48, 96, seed=13, done_p=0.05, rho_clip=1.0, c_clip=1e12)
    v, r, d, w = make_inputs(wl)
    r[0:16, 70] = 1e29
    d[0:16, 70] = 0.0
    d[0:16, 69] = 1.0
    w[0:16, 68] = 1e12
    r[16:32, 40] = 1e10
    d[16:32, 40] = 0.0
    d[16:32, 39] = 1.0
    w[16:32, 38] = -1e30
    adv = run_reference(ref, (v, r, d, w), wl.hyper())
    assert torch.isnan(adv[0:32, 0]).all() and torch.isfinite(adv[32:, :-1]).all()
    for key, t in zip(("values", "rewards", "dones", "importance"), (v, r, d, w)):
        arrays[f"gain_overflow.{key}"] = t.numpy()
    arrays["gain_overflow.advantages"] = adv.numpy()
    meta["gain_overflow"] = {"hyper": list(wl.hyper()), "segments": 48, "horizon": 96}
    arrays["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(out_dir, "small_cases.npz"), **arrays)

    digests = {"sentinel": SENTINEL, "torch": torch.__version__, "configs": {}}
    for name, wl in WORKLOADS.items():
        inputs = make_inputs(wl)
        adv = run_reference(ref, inputs, wl.hyper()).numpy()
        in_sha = hashlib.sha256(b"".join(t.numpy().tobytes() for t in inputs)).hexdigest()
        flat = adv.reshape(-1)
        idx = np.linspace(0, flat.size - 1, 64).astype(np.int64)
        body = adv[:, :-1].astype(np.float64)
        digests["configs"][name] = {
            "segments": wl.segments, "horizon": wl.horizon, "hyper": list(wl.hyper()),
            "inputs_sha256": in_sha,
            "advantages_sha256": hashlib.sha256(adv.tobytes()).hexdigest(),
            "sample_index": idx.tolist(),
            "sample_bits": flat[idx].view(np.uint32).tolist(),
            "abs_sum_total": float(np.abs(body).sum()),
            "max_abs": float(np.abs(body).max()),
        }
        print(name, digests["configs"][name]["advantages_sha256"][:16], digests["configs"][name]["max_abs"])
    with open(os.path.join(out_dir, "config_digests.json"), "w") as f:
        json.dump(digests, f, indent=1)


if __name__ == "__main__":
    main()
