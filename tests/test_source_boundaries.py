"""Source-level rules of this code base, checked by reading the files (no GPU, no compiler):

* no bulk / tensor copy with a cluster-multicast qualifier anywhere (loads from peer memory with it are not allowed on
  multi-GPU machines, and the library has to run unchanged on 1 to 8 GPUs),
* none of the batched memcpy entry points of the CUDA runtime / driver,
* device code never traps, never uses a failing device assert and never spins without a bound: every spin-wait goes through
  `bounded_wait` / `wait_bar` / `mbar_wait_bounded`,
* nothing under the package imports from the working directories.
The forbidden names are assembled from pieces so that this file does not contain them either.
"""
import re
from pathlib import Path

REPO = Path(__file__).resolve().parents[1]
SRC_SUFFIXES = {'.cu', '.cuh', '.h', '.hpp', '.cpp', '.py'}


def _sources():
    for base in (REPO / 'deepep_ascend_b200', REPO / 'tests'):
        for p in base.rglob('*'):
            if p.suffix in SRC_SUFFIXES and '_ext' not in p.parts and '__pycache__' not in p.parts:
                yield p
    for name in ('bench.py', 'bench_extras.py', '__graft_entry__.py', 'setup.py'):
        yield REPO / name


def test_no_forbidden_constructs():
    multicast = '.multi' + 'cast::' + 'cluster'
    batched = [a + 'Batch' + 'Async' for a in ('cudaMemcpy', 'cudaMemcpy3D', 'cuMemcpy', 'cuMemcpy3D')]
    trap = re.compile(r'__tr' + r'ap\s*\(|\basm\s*(volatile)?\s*\(\s*"tr' + 'ap')
    bad = []
    for p in _sources():
        text = p.read_text(encoding='utf-8', errors='replace')
        if multicast in text:
            bad.append((p, 'cluster multicast'))
        for b in batched:
            if b in text:
                bad.append((p, 'batched memcpy'))
        if p.suffix in ('.cu', '.cuh') and trap.search(text):
            bad.append((p, 'trap'))
        if p.suffix in ('.cu', '.cuh') and re.search(r'^\s*assert\s*\(', text, re.M):
            bad.append((p, 'device assert'))
        if p.suffix == '.py' and re.search(r'(^|[^A-Za-z0-9])_wo' + r'rk(/|[\'"])', text):
            bad.append((p, 'reference to the working directory'))
    assert not bad, bad


def test_every_device_spin_is_bounded():
    """A `while` whose condition polls memory (ld_acquire / ld_relaxed / mbar_try_wait / volatile) must sit in one of the bounded
    helpers or carry its own time limit."""
    kernels = REPO / 'deepep_ascend_b200' / 'csrc' / 'kernels'
    polls = re.compile(r'while\s*\(.*(ld_acquire|ld_relaxed|mbar_try_wait|volatile)')
    offenders = []
    for p in list(kernels.glob('*.cu')) + list(kernels.glob('*.cuh')):
        lines = p.read_text().split('\n')
        for i, line in enumerate(lines):
            if polls.search(line):
                window = '\n'.join(lines[max(0, i - 6):i + 8])
                if not re.search(r'timeout_ns|kWaitLimitNs|globaltimer|gemm_timer|limit', window):
                    offenders.append('%s:%d' % (p.name, i + 1))
    assert not offenders, offenders
