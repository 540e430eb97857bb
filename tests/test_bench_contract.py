"""The benchmark entry point's contract that can be checked without a GPU: the reference arm answers with one JSON line saying why
it is unavailable, and exits 0."""
import json
import subprocess
import sys
from pathlib import Path

REPO = Path(__file__).resolve().parents[1]


def test_reference_arm_reports_unavailable():
    res = subprocess.run([sys.executable, 'bench.py', '--impl', 'reference', '--gpus', '1', '--steps', '2', '--warmup', '1'], cwd=REPO,
                         capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line['impl'] == 'reference' and isinstance(line['unavailable'], str) and len(line['unavailable']) > 10


def test_entry_points_exist():
    sys.path.insert(0, str(REPO))
    import __graft_entry__ as entry
    assert callable(entry.build) and callable(entry.smoke)
