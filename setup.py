"""Build entry point in the place of the reference's setup.py.

The reference builds `pufferlib._C` with torch's CUDAExtension and nvcc flags
`-O3` for whatever architectures torch lists (setup.py:83-120, 237-258), and
falls back to a CPU-only CppExtension when no CUDA toolkit is found.  Here
`build_ext` compiles for sm_100a only (`-gencode arch=compute_100a,code=sm_100a`,
no fast-math, no FTZ), there is no Triton and no CPU fallback: without nvcc the
build fails.  The actual commands live in pufferlib_b200/build.py, which is
also what `python -m pufferlib_b200.build` runs.
"""
import os
import sys

from setuptools import Command, find_packages, setup

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


class build_ext(Command):
    description = "compile libpuff_advantage_sm100.so and the torch operator module in-tree"
    user_options = [("force", "f", "rebuild even when outputs are newer than sources"),
                    ("inplace", "i", "accepted for compatibility; the build is always in-tree")]
    boolean_options = ["force", "inplace"]

    def initialize_options(self):
        self.force = False
        self.inplace = True

    def finalize_options(self):
        pass

    def run(self):
        from pufferlib_b200 import build
        build.build_all(force=bool(self.force), verbose=True)


setup(
    name="pufferlib_b200",
    version="0.1",
    description="B200-native (sm_100a) compute_puff_advantage for PufferLib",
    packages=find_packages(include=["pufferlib_b200"]),
    package_data={"pufferlib_b200": ["*.so", "csrc/*"]},
    cmdclass={"build_ext": build_ext},
)
