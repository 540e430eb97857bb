"""Builds and loads the native extension (C++ runtime + sm_100a kernels).

The extension is built ahead of time into ``deepep_ascend_b200/_ext`` (in-tree, next to the sources) with
``nvcc -gencode arch=compute_100a,code=sm_100a``; importing the package only loads the shared object.  If the
object is missing and ``nvcc`` is available it is built on first use.  There is no runtime JIT of kernels:
shapes are runtime arguments (the reference compiles each shape with nvcc at run time, csrc/jit/compiler.hpp:22-267).
"""
import glob
import importlib.util
import os
import threading
from typing import Optional

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_PKG_DIR, 'csrc')
_EXT_DIR = os.path.join(_PKG_DIR, '_ext')
_NAME = 'deepep_b200_C'
_lock = threading.Lock()
_module = None

NVCC_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-O3', '-std=c++17', '-lineinfo',
              '--expt-relaxed-constexpr', '-Xptxas', '-v']
CXX_FLAGS = ['-O2', '-std=c++17']


def sources():
    srcs = [os.path.join(_CSRC, 'python_api.cpp')]
    srcs += sorted(glob.glob(os.path.join(_CSRC, 'kernels', '*.cu')))
    return srcs


def extra_include_paths():
    return [_CSRC]


def shared_object() -> Optional[str]:
    hits = glob.glob(os.path.join(_EXT_DIR, _NAME + '*.so'))
    return hits[0] if hits else None


def build(verbose: bool = False):
    """Compile every source for sm_100a into ``_ext/`` (incremental through ninja) and load the result."""
    global _module
    from torch.utils import cpp_extension
    os.makedirs(_EXT_DIR, exist_ok=True)
    os.environ.setdefault('MAX_JOBS', str(os.cpu_count() or 4))
    # Link with the distribution's g++: a toolchain whose libstdc++.so is missing falls back to the static
    # archive, and a second private copy of libstdc++ inside the extension breaks iostreams at run time.
    for var, path in (('CXX', '/usr/bin/g++'), ('CC', '/usr/bin/gcc')):
        if os.path.exists(path):
            os.environ[var] = path
    with _lock:
        _module = cpp_extension.load(
            name=_NAME, sources=sources(), extra_cflags=CXX_FLAGS, extra_cuda_cflags=NVCC_FLAGS,
            extra_include_paths=extra_include_paths(), extra_ldflags=['-lcuda'],
            build_directory=_EXT_DIR, verbose=verbose, with_cuda=True)
        with open(os.path.join(_EXT_DIR, 'sources.sha256'), 'w') as fh:
            fh.write(_source_digest())
        _capture_persistent_envs()
    return _module


# Settings that must be the same when the package runs as when it was built: they are captured at build time and applied
# at import unless the process sets them itself (the reference writes them into deep_ep/envs.py, setup.py:31,91-110, and
# re-applies them in deep_ep/__init__.py:13-20).  EP_NUM_TOPK_IDX_BITS selects the dtype of ``topk_idx_t``.
PERSISTENT_ENVS = ('EP_NUM_TOPK_IDX_BITS',)
_PERSISTENT_FILE = 'persistent_envs.json'


def _capture_persistent_envs() -> None:
    import json
    found = {k: os.environ[k] for k in PERSISTENT_ENVS if k in os.environ}
    with open(os.path.join(_EXT_DIR, _PERSISTENT_FILE), 'w') as fh:
        json.dump(found, fh)


def apply_persistent_envs(directory: Optional[str] = None) -> dict:
    """Set every captured variable that the process has not set itself; returns what was captured."""
    import json
    path = os.path.join(directory or _EXT_DIR, _PERSISTENT_FILE)
    if not os.path.exists(path):
        return {}
    try:
        with open(path) as fh:
            found = json.load(fh)
    except (OSError, ValueError):
        return {}
    for k, v in found.items():
        if k in PERSISTENT_ENVS:
            os.environ.setdefault(k, str(v))
    return found


def _source_digest() -> str:
    import hashlib
    h = hashlib.sha256()
    for root, dirs, files in os.walk(_CSRC):
        dirs.sort()
        for f in sorted(files):
            h.update(f.encode())
            with open(os.path.join(root, f), 'rb') as fh:
                h.update(fh.read())
    return h.hexdigest()


def _stale(so: str) -> bool:
    """The shared object is stale when the digest recorded at build time differs from the sources'
    (file times do not survive copying the tree to another machine)."""
    stamp = os.path.join(_EXT_DIR, 'sources.sha256')
    if not os.path.exists(stamp):
        return True
    with open(stamp) as fh:
        return fh.read().strip() != _source_digest()


def load(required: bool = True):
    """Return the extension module; build it if it is missing or older than its sources and nvcc exists.
    With ``required=False`` returns ``None`` instead of raising (CPU-only use of the package)."""
    global _module
    if _module is not None:
        return _module
    import torch  # noqa: F401  (the extension links against libtorch)
    so = shared_object()
    from torch.utils.cpp_extension import CUDA_HOME
    have_nvcc = CUDA_HOME is not None and os.path.exists(os.path.join(CUDA_HOME, 'bin', 'nvcc'))
    try:
        if so is not None and not (have_nvcc and _stale(so) and os.environ.get('EP_NO_REBUILD', '0') != '1'):
            with _lock:
                spec = importlib.util.spec_from_file_location(_NAME, so)
                mod = importlib.util.module_from_spec(spec)
                spec.loader.exec_module(mod)
                _module = mod
            return _module
        if have_nvcc:
            return build()
    except Exception:
        if required:
            raise
        return None
    if required:
        raise ImportError('deepep_ascend_b200: the native extension is not built and nvcc is not available; build it on a '
                          'machine with CUDA 12.9 (`python setup.py build_ext --inplace`, or `deepep_ascend_b200._native.build()`)')
    return None


def is_available() -> bool:
    return load(required=False) is not None
