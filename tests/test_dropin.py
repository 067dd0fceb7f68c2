"""The drop-in claim, checked with the reference's own text and build recipe.

* The wrapper `compute_puff_advantage` is read out of the reference checkout's
  pufferlib/pufferl.py at test time (never copied into this repository) and
  executed unchanged against the operator this repository registers.
* The `CUDAExtension("pufferlib._C", ...)` block that INTEGRATION.md gives as
  the replacement of setup.py:237-258 is taken from INTEGRATION.md itself and
  built once; the resulting module must import as `pufferlib._C` and register
  the reference's schema with CUDA and Meta kernels.
"""
import ast
import os
import re
import shutil
import subprocess
import sys
import textwrap

import numpy as np
import pytest
import torch

from helpers import bits_equal, first_mismatch, oracle_advantage
from pufferlib_b200.workloads import WORKLOADS, make_inputs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def reference_wrapper():
    """The function object compiled from the reference's own source text, with
    ADVANTAGE_CUDA = True (pufferl.py:49-55: a CUDA toolchain was found)."""
    from oracle import puff_oracle
    path = os.path.join(puff_oracle.reference_root(), "pufferlib", "pufferl.py")
    if not os.path.isfile(path):
        pytest.skip("no reference checkout on this machine")
    tree = ast.parse(open(path).read(), filename=path)
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "compute_puff_advantage")
    module = ast.Module(body=[fn], type_ignores=[])
    scope = {"torch": torch, "ADVANTAGE_CUDA": True}
    exec(compile(module, path, "exec"), scope)
    return scope["compute_puff_advantage"]


def test_reference_wrapper_text_calls_the_op_unchanged():
    """Shape-only run on meta tensors: argument order, keyword-free call and
    return value of pufferl.py:660-680 fit the registered operator."""
    from pufferlib_b200 import _C  # noqa: F401
    wrapper = reference_wrapper()
    t = [torch.empty(64, 32, device="meta") for _ in range(5)]
    out = wrapper(*t, 0.99, 0.95, 1.0, 1.0)
    assert out is t[4]


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["cfg0", "cfg4"])
def test_reference_wrapper_text_on_the_gpu(name):
    from pufferlib_b200 import _C  # noqa: F401
    wrapper = reference_wrapper()
    wl = WORKLOADS[name]
    host = make_inputs(wl)
    dev = [t.cuda() for t in host]
    adv = torch.zeros_like(dev[0])
    out = wrapper(*dev, adv, *wl.hyper())
    assert out is adv
    want = oracle_advantage([t.numpy() for t in host], wl.hyper(), sentinel=0.0)
    assert bits_equal(adv.cpu().numpy(), want), first_mismatch(adv.cpu().numpy(), want)


def test_integration_recipe_builds_pufferlib_C(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    blocks = re.findall(r"```python\n(.*?)```", text, flags=re.S)
    recipe = next(b for b in blocks if 'CUDAExtension(' in b and '"pufferlib._C"' in b)
    pkg = tmp_path / "pufferlib"
    pkg.mkdir()
    (pkg / "__init__.py").write_text("")
    os.symlink(os.path.join(ROOT, "pufferlib_b200"), tmp_path / "pufferlib_b200")
    os.symlink(os.path.join(ROOT, "include"), tmp_path / "include")
    (tmp_path / "setup.py").write_text(
        "from setuptools import setup\n"
        "from torch.utils.cpp_extension import BuildExtension, CUDAExtension\n"
        + textwrap.dedent(recipe) +
        "\nsetup(name='pufferlib', packages=['pufferlib'], ext_modules=torch_extensions,\n"
        "      cmdclass={'build_ext': BuildExtension})\n")
    env = dict(os.environ, TORCH_CUDA_ARCH_LIST="10.0a", MAX_JOBS="8", CUDA_HOME=os.path.dirname(os.path.dirname(nvcc)))
    for var in ("CC", "CXX"):      # a compiler wrapper that links a static libstdc++ breaks python modules
        env.pop(var, None)
    out = subprocess.run([sys.executable, "setup.py", "build_ext", "--inplace"], cwd=tmp_path, env=env,
                         capture_output=True, text=True, timeout=1500)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    built = [f for f in os.listdir(pkg) if f.startswith("_C") and f.endswith(".so")]
    assert built, os.listdir(pkg)
    # a fresh interpreter: this process may already hold pufferlib_b200._C, and a second
    # definition of the same operator library in one process is an error
    check = textwrap.dedent("""
        import sys, torch
        sys.path.insert(0, sys.argv[1])
        from pufferlib import _C
        op = torch.ops.pufferlib.compute_puff_advantage
        schema = str(op.default._schema)
        assert schema == ("pufferlib::compute_puff_advantage(Tensor(a!) values, Tensor(b!) rewards, "
                          "Tensor(c!) dones, Tensor(d!) importance, Tensor(e!) advantages, float gamma, "
                          "float lambda, float rho_clip, float c_clip) -> ()"), schema
        has = torch._C._dispatch_has_kernel_for_dispatch_key
        assert has("pufferlib::compute_puff_advantage", "CUDA")
        assert has("pufferlib::compute_puff_advantage", "Meta")
        assert not has("pufferlib::compute_puff_advantage", "CPU")
        t = [torch.empty(8, 16, device="meta") for _ in range(5)]
        op(*t, 0.99, 0.95, 1.0, 1.0)
        print("recipe ok")
    """)
    run = subprocess.run([sys.executable, "-c", check, str(tmp_path)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0 and "recipe ok" in run.stdout, run.stdout[-2000:] + run.stderr[-2000:]
