"""Compare two ``benchmark.json`` files made from the same workload.

    python -m deepep_ascend_b200.benchmark.compare_ep --left out/a/benchmark.json --right out/b/benchmark.json --output cmp.md

Refuses (exit code 2 with a message) when the reports differ in profile, world size or workload fingerprint, when either fails
the schema check, or when ``--output`` names one of the inputs.  Parity: tests/benchmark/compare_ep.py of the reference.
"""
import argparse
import json
from pathlib import Path
from typing import List, Optional

from .report import compare_reports
from .workload import write_text_atomic


def _same_file(a: Path, b: Path) -> bool:
    if a == b:
        return True
    try:
        return a.samefile(b)
    except FileNotFoundError:
        return False


def main(argv: Optional[List[str]] = None) -> int:
    p = argparse.ArgumentParser()
    p.add_argument('--left', required=True, type=Path)
    p.add_argument('--right', required=True, type=Path)
    p.add_argument('--output', required=True, type=Path)
    args = p.parse_args(argv)
    try:
        left, right, out = args.left.resolve(), args.right.resolve(), args.output.resolve()
        if _same_file(out, left) or _same_file(out, right):
            raise ValueError('--output must not be one of the inputs')
        reports = []
        for path in (left, right):
            with open(path, encoding='utf-8') as f:
                reports.append(json.load(f))
        write_text_atomic(out, compare_reports(reports[0], reports[1]))
    except (OSError, json.JSONDecodeError, ValueError) as e:
        p.error(str(e))
    return 0


if __name__ == '__main__':
    raise SystemExit(main())
