"""Benchmark automation for the expert-parallel dispatch / combine API.

* ``cases``     - the matrix of API modes every backend is run through (144 of them),
* ``workload``  - a seeded routing workload with a SHA-256 fingerprint, stored as ``workload.json``,
* ``traffic``   - byte counts behind the reported GB/s,
* ``profiles``  - named workload sizes (smoke / canonical / headline),
* ``report``    - schema check, markdown rendering and comparison of two ``benchmark.json`` files,
* ``run_ep``    - ``python -m deepep_ascend_b200.benchmark.run_ep --backend cuda|cpu --profile smoke --output-dir out``,
* ``compare_ep``- ``python -m deepep_ascend_b200.benchmark.compare_ep --left a/benchmark.json --right b/benchmark.json --output cmp.md``.

Parity: tests/benchmark/{run_ep,compare_ep,report_markdown,profiles}.py and tests/utils/ep_benchmark_{core,manifest}.py of the reference.
"""
