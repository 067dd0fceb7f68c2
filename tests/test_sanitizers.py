"""CPU: the host side of the launcher and the CPU oracle under AddressSanitizer
and UndefinedBehaviorSanitizer.

Mirrors the reference's DEBUG=1 build, which adds
`-fsanitize=address,undefined,...` to its C extensions and is run with
LD_PRELOAD=libasan (setup.py:1-3, 29-30, 88-106).  The kernel library's host
code (argument validation, kernel selection, tensor-map cache, tuning knobs,
error strings) and the oracle are compiled with the sanitizers into a scratch
folder, and the symbol / validation tests and the oracle tests run against those
builds in a child interpreter.  Device code is not instrumented; nothing here
needs a GPU.
"""
import os
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SAN = "-fsanitize=address,undefined"


def test_host_launcher_and_oracle_under_asan_ubsan(tmp_path):
    from pufferlib_b200 import build
    gcc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else shutil.which("gcc")
    if gcc is None or not os.path.exists(build.NVCC):
        pytest.skip("gcc / nvcc not available")
    libasan = subprocess.run([gcc, "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
    if not os.path.isabs(libasan) or not os.path.exists(libasan):
        pytest.skip("libasan not installed")
    adv_lib = str(tmp_path / "libpuff_advantage_sm100_asan.so")
    oracle_lib = str(tmp_path / "libpuff_oracle_asan.so")
    sources = [os.path.join(build.CSRC, s) for s in build.CU_SOURCES]
    # nvcc splits -Xcompiler arguments at commas: one sanitizer per flag
    flags = [f for f in build.NVCC_FLAGS if f != "-O3"] + [
        "-O1", "-g", "-ccbin", gcc.replace("gcc", "g++"), "-Xcompiler", "-fsanitize=address",
        "-Xcompiler", "-fsanitize=undefined", "-Xcompiler", "-fno-omit-frame-pointer"]
    subprocess.run([build.NVCC] + flags + ["-o", adv_lib] + sources + ["-Xlinker", "-lasan", "-Xlinker", "-lubsan"],
                   check=True, capture_output=True)
    subprocess.run([gcc, "-O1", "-g", "-ffp-contract=off", "-fPIC", "-shared", SAN, "-fno-omit-frame-pointer",
                    "-o", oracle_lib, os.path.join(ROOT, "oracle", "puff_advantage_oracle.c"), "-lm"], check=True)
    env = dict(os.environ, LD_PRELOAD=libasan, PUFF_ADV_LIB=adv_lib, PUFF_ORACLE_LIB=oracle_lib,
               ASAN_OPTIONS="detect_leaks=0:abort_on_error=1:halt_on_error=1",
               UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1", PYTHONPATH=ROOT)
    out = subprocess.run(
        [sys.executable, "-m", "pytest", "-x", "-q", "-p", "no:cacheprovider",
         os.path.join(ROOT, "tests", "test_oracle.py"), os.path.join(ROOT, "tests", "test_cabi_symbols.py"),
         "-k", "not schema and not shape_kernel and not no_cpu_fallback"],
        env=env, capture_output=True, text=True, timeout=1200, cwd=ROOT)
    tail = out.stdout[-3000:] + out.stderr[-3000:]
    assert out.returncode == 0, tail
    assert "passed" in out.stdout and "AddressSanitizer" not in tail and "runtime error" not in tail, tail
