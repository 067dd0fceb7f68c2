"""In-tree build of the native libraries (sm_100a only).

Plays the part of the reference's `build_torch` step (setup.py:170-178,
237-258: CUDAExtension("pufferlib._C", [pufferlib.cpp, cuda/pufferlib.cu]) with
nvcc flags `-O3`), with the flags this implementation needs instead:

  libpuff_advantage_sm100.so   nvcc, -gencode arch=compute_100a,code=sm_100a,
                               no fast-math, no FTZ, no torch headers: the
                               kernels and their C ABI (include/puff_advantage.h)
  _C.so                        g++, torch headers: the TORCH_LIBRARY operator
                               registration, linked against the library above

Both land next to this file so that the package works from the source tree.
Outputs are rebuilt only when a source is newer.
"""
import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")

CABI_LIB = os.path.join(HERE, "libpuff_advantage_sm100.so")
TORCH_EXT = os.path.join(HERE, "_C.so")

CU_SOURCES = ["puff_advantage_sm100.cu", "puff_priorities_sm100.cu", "puff_minibatch_sm100.cu",
              "puff_rollout_sm100.cu", "puff_host_pipeline.cu"]

# --fmad=true leaves nvcc free to contract a*b+c into an FMA.  One such contraction in the
# recurrence changes the last bit of about half of the outputs, so every kernel that must be
# bit-exact (tma2d, bulk1d, generic, and the replay step of scan) spells its arithmetic with
# __fmul_rn / __fadd_rn / __fsub_rn and their f32x2 forms, which are never contracted.  Only code
# that is checked against a tolerance (the scan kernel's carry composition, the minibatch
# normalisation, the priority weights) is written with plain operators and may be fused.
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--ftz=false", "--prec-div=true", "--prec-sqrt=true", "--fmad=true",
    "-Xcompiler", "-fPIC", "-shared",
]


def _host_cxx():
    """The system g++.  A compiler wrapper that points the linker at a static
    libstdc++ (as the CXX of some build images does) would embed a second,
    uninitialised copy of the C++ runtime in the module; its iostreams crash
    the first time an error message formats a number."""
    override = os.environ.get("PUFF_CXX")
    if override:
        return override
    for cand in ("/usr/bin/g++", shutil.which("g++"), os.environ.get("CXX")):
        if cand and os.path.exists(cand):
            return cand
    return "g++"


def _stale(target, sources):
    if not os.path.isfile(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)


def build_debug_cabi(out_path, verbose=False):
    """The kernel library with -DPUFF_DEBUG_BOUNDS: every global-memory index
    the kernels form is checked, a bad one sets PUFF_ERR_DEVICE_BOUNDS in the
    status word and its access is skipped (nothing traps).  Slower; for tests
    and debugging.  Written to `out_path`, never over the release library."""
    sources = [os.path.join(CSRC, s) for s in CU_SOURCES]
    _run([NVCC] + NVCC_FLAGS + ["-DPUFF_DEBUG_BOUNDS", "-o", out_path] + sources, verbose)
    return out_path


def build_cabi(force=False, verbose=False, ptxas_info=False):
    sources = [os.path.join(CSRC, s) for s in CU_SOURCES]
    headers = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith(".cuh")]
    deps = sources + headers + [os.path.join(INCLUDE, "puff_advantage.h")]
    if force or _stale(CABI_LIB, deps):
        flags = list(NVCC_FLAGS)
        if ptxas_info:
            flags += ["-Xptxas", "-v"]
        _run([NVCC] + flags + ["-o", CABI_LIB] + sources, verbose)
    return CABI_LIB


def build_torch_ext(force=False, verbose=False):
    import torch
    from torch.utils.cpp_extension import include_paths, library_paths
    src = os.path.join(CSRC, "torch_binding.cpp")
    deps = [src, os.path.join(INCLUDE, "puff_advantage.h"), CABI_LIB]
    if force or _stale(TORCH_EXT, deps):
        cxx = _host_cxx()
        inc = [f"-I{p}" for p in include_paths()]
        inc += [f"-I{os.path.join(CUDA_HOME, 'include')}", f"-I{sysconfig.get_paths()['include']}"]
        libdir = library_paths()[0]
        cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared",
               f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
               "-DTORCH_EXTENSION_NAME=_C"] + inc + [
               "-o", TORCH_EXT, src,
               f"-L{HERE}", "-lpuff_advantage_sm100", "-Wl,-rpath,$ORIGIN",
               f"-L{libdir}", f"-Wl,-rpath,{libdir}",
               "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch"]
        _run(cmd, verbose)
    return TORCH_EXT


def build_all(force=False, verbose=False):
    build_cabi(force=force, verbose=verbose)
    build_torch_ext(force=force, verbose=verbose)


if __name__ == "__main__":
    if "--debug-bounds" in sys.argv:
        build_debug_cabi(os.path.join(HERE, "libpuff_advantage_sm100_debug.so"), verbose=True)
    else:
        build_all(force="--force" in sys.argv, verbose=True)
