"""Build and install the sm_100a gdn_chunk library.

    python setup.py build_ext --inplace      # same as: python -m gdn_qsa_sm80_b200.build

The CUDA sources are compiled by nvcc for sm_100a only (-gencode arch=compute_100a,code=sm_100a) into
gdn_qsa_sm80_b200/lib/libgdn_chunk_sm100.so, a plain C-ABI shared library that Python loads with ctypes;
there is no other architecture, no op selection and no fallback target (the reference's setup.py builds
five sm_80 extensions selected by environment variables, setup.py:9-33).
"""

import os
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_ext import build_ext

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


class BuildCudaLibrary(build_ext):
    def run(self):
        from gdn_qsa_sm80_b200 import build as b
        print(b.build(force=True))


setup(
    name="gdn_qsa_sm80_b200",
    version="0.1.0",
    description="gdn_chunk forward for NVIDIA B200 (sm_100a): TMA + tcgen05/TMEM kernels behind a C ABI",
    packages=find_packages(include=["gdn_qsa_sm80", "gdn_qsa_sm80_b200"]),
    package_data={"gdn_qsa_sm80_b200": ["lib/*.so", "csrc/*"]},
    cmdclass={"build_ext": BuildCudaLibrary},
    python_requires=">=3.10",
)
