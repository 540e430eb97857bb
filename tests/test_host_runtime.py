"""Compiles the host-only C++ probe (life-cycle coordinator, overflow-checked region layout) with the system C++
compiler and runs it: no GPU, no torch."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cuda_include():
    for cand in (os.environ.get('CUDA_HOME'), '/usr/local/cuda'):
        if cand and os.path.exists(os.path.join(cand, 'include', 'cuda_runtime_api.h')):
            return os.path.join(cand, 'include')
    return None


@pytest.mark.parametrize('sanitize', [False, True])
def test_host_runtime_probe(tmp_path, sanitize):
    cxx = shutil.which('g++') or shutil.which('c++')
    inc = _cuda_include()
    if cxx is None or inc is None:
        pytest.skip('needs a C++ compiler and the CUDA headers')
    exe = str(tmp_path / 'probe')
    flags = ['-std=c++17', '-O1', '-pthread', '-I', os.path.join(ROOT, 'deepep_ascend_b200', 'csrc'), '-I', inc]
    if sanitize:
        flags += ['-fsanitize=address,undefined', '-fno-omit-frame-pointer']
    build = subprocess.run([cxx, *flags, os.path.join(ROOT, 'tests', 'probes', 'host_runtime_probe.cpp'), '-o', exe],
                           capture_output=True, text=True)
    if build.returncode != 0 and sanitize:
        pytest.skip('sanitizer runtime not available: ' + build.stderr[-200:])
    assert build.returncode == 0, build.stderr
    run = subprocess.run([exe], capture_output=True, text=True)
    assert run.returncode == 0, run.stdout + run.stderr
    assert 'all checks passed' in run.stdout
