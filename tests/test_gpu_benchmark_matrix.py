"""The 144-case API mode matrix (handle copy x alignment x precision x biases x stream plumbing) through the benchmark runner on
real GPUs: every received row bit for bit against its source token, counts, cached re-dispatch, zero padding, combine sums."""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
REPO = Path(__file__).resolve().parents[1]


def _run(tmp_path, world, cases):
    out = tmp_path / ('w%d' % world)
    cmd = [sys.executable, '-m', 'deepep_ascend_b200.benchmark.run_ep', '--backend', 'cuda', '--profile', 'smoke', '--world-size', str(world),
           '--cases', cases, '--num-sms', '8', '--output-dir', str(out)]
    res = subprocess.run(cmd, cwd=REPO, capture_output=True, text=True, timeout=900)
    log = (out / 'run.log').read_text()[-3000:] if (out / 'run.log').exists() else ''
    assert res.returncode == 0, res.stderr[-3000:] + log
    return json.loads((out / 'benchmark.json').read_text())


def test_mode_matrix_one_gpu(tmp_path):
    rep = _run(tmp_path, 1, 'all')
    assert rep['summary'] == {'total': 144, 'passed': 144, 'failed': 0}


def test_mode_matrix_all_visible_gpus(tmp_path):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip('needs at least two GPUs')
    world = 8 if n >= 8 else (4 if n >= 4 else 2)
    rep = _run(tmp_path, world, 'all')
    assert rep['summary'] == {'total': 144, 'passed': 144, 'failed': 0}
