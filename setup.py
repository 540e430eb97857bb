"""Packaging for deepep_ascend_b200 (sm_100a only).

    python setup.py build_ext --inplace      # compile the CUDA / C++ sources into deepep_ascend_b200/_ext
    python -m pip install --no-build-isolation .

There is one build path: the ``build_ext`` command calls ``deepep_ascend_b200._native.build`` (nvcc with
``-gencode arch=compute_100a,code=sm_100a``), the same function the package uses to refresh a stale binary, and the shared
object is then shipped as package data.  ``EP_NUM_TOPK_IDX_BITS`` (64 or 32) is read at import time, not at build time.
Parity: setup.py of the reference (CUDA path), without its NVSHMEM / NCCL link steps: this library links neither.
"""
import importlib.util
import os

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


def _native():
    spec = importlib.util.spec_from_file_location('_ep_native_build', os.path.join(ROOT, 'deepep_ascend_b200', '_native.py'))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class BuildExt(Command):
    description = 'compile the sm_100a extension in-tree'
    user_options = [('inplace', 'i', 'accepted for compatibility: the build is always in-tree')]

    def initialize_options(self):
        self.inplace = True

    def finalize_options(self):
        pass

    def run(self):
        _native().build(verbose=bool(os.environ.get('EP_BUILD_VERBOSE')))


class BuildPy(build_py):
    def run(self):
        self.run_command('build_ext')
        super().run()


setup(
    name='deepep_ascend_b200',
    version='0.1.0',
    description='Expert-parallel dispatch / combine, low-latency decode, fused MoE and TP GEMM kernels for 8xB200 (sm_100a)',
    packages=find_packages(include=['deepep_ascend_b200', 'deepep_ascend_b200.*']),
    package_data={'deepep_ascend_b200': ['_ext/*.so', '_ext/sources.sha256', 'csrc/**/*']},
    python_requires='>=3.10',
    install_requires=['torch'],
    cmdclass={'build_ext': BuildExt, 'build_py': BuildPy},
)
