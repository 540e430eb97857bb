"""Benchmark automation: mode matrix, workload manifest + fingerprint, traffic formulas, report schema, comparison, and one
command-line run on the gloo backend (two CPU ranks, smoke profile, four cases)."""
import copy
import json
import subprocess
import sys
from pathlib import Path

import pytest

from deepep_ascend_b200.benchmark import cases, profiles, report, traffic, workload

REPO = Path(__file__).resolve().parents[1]


def test_mode_matrix_is_144_distinct_cases():
    cs = cases.enumerate_mode_cases()
    assert len(cs) == 144 and len({c.case_id for c in cs}) == 144
    assert all(c.allocate_on_comm_stream for c in cs if c.with_previous_event)
    perf = cases.select_cases('performance')
    assert len(perf) == 24 and all(not (c.with_previous_event or c.async_with_compute_stream or c.allocate_on_comm_stream) for c in perf)
    assert len(cases.select_cases('functional')) == 120
    one = cs[17]
    assert cases.select_cases(one.case_id) == (one,)
    with pytest.raises(ValueError):
        cases.select_cases('ep-nope')


def test_manifest_is_deterministic_and_tamper_evident(tmp_path):
    spec = profiles.profile_spec(profiles.PROFILES['smoke'], 4)
    a, b = workload.build_manifest(spec), workload.build_manifest(spec)
    assert a.fingerprint == b.fingerprint and a.ranks == b.ranks
    assert [r.num_tokens for r in a.ranks] == [16, 15, 14, 13]
    assert all(len(set(e for e in row if e >= 0)) == len([e for e in row if e >= 0]) for r in a.ranks for row in r.topk_idx)
    other = workload.build_manifest(workload.WorkloadSpec(4, 16, 128, 2, 8, seed=1))
    assert other.fingerprint != a.fingerprint
    path = tmp_path / 'workload.json'
    workload.write_manifest(path, a)
    assert workload.load_manifest(path).fingerprint == a.fingerprint
    d = json.loads(path.read_text())
    d['ranks'][0]['topk_idx'][0][0] = (d['ranks'][0]['topk_idx'][0][0] + 1) % 8
    path.write_text(json.dumps(d))
    with pytest.raises(ValueError, match='fingerprint'):
        workload.load_manifest(path)
    for bad in (dict(world_size=3, num_experts=8), dict(num_topk=9), dict(masked_ratio=1.5), dict(unbalanced_ratio=0.5)):
        kw = dict(world_size=2, num_tokens=4, hidden=8, num_topk=2, num_experts=8)
        kw.update(bad)
        with pytest.raises(ValueError):
            workload.WorkloadSpec(**kw)


def test_masked_and_unbalanced_workloads():
    m = workload.build_manifest(workload.WorkloadSpec(2, 200, 8, 2, 8, masked_ratio=0.5, unbalanced_ratio=4.0))
    flat = [e for r in m.ranks for row in r.topk_idx for e in row]
    masked = sum(e < 0 for e in flat) / len(flat)
    assert 0.4 < masked < 0.6
    to_rank0 = sum(0 <= e < 4 for e in flat) / sum(e >= 0 for e in flat)
    assert to_rank0 > 0.6          # the experts of rank 0 are favoured


def test_traffic_formulas():
    t = traffic.dispatch_row_tensors(7168, 8, use_fp8=True)
    per = 7168 + 4 * 56 + 64 + 32 + 8
    d = traffic.dispatch_traffic(t, num_recv_rows=1000, num_local_rows=125)
    assert d.bytes_per_token == per and d.logical_bytes == 1000 * per and d.nvlink_bytes == 875 * per
    assert traffic.dispatch_traffic(traffic.dispatch_row_tensors(128, 2, False), 10, 10).nvlink_bytes == 0
    c = traffic.combine_traffic(num_rows=1000, num_local_rows=125, num_tokens=200, hidden=7168, num_bias=2)
    assert c.logical_bytes == 1000 * 14336 and c.nvlink_bytes == 875 * 14336 and c.reduction_bytes == (1000 + 400 + 200) * 14336
    with pytest.raises(ValueError):
        traffic.dispatch_traffic(t, 10, 11)
    with pytest.raises(ValueError):
        traffic.TensorBytes(-1, 4)
    routes = [[0, 1, 9, -1], [8, 8, 8, 8], [-1, -1, -1, -1]]
    assert traffic.count_unique_destinations(routes) == 3 + 1
    assert traffic.count_unique_destinations(routes, divisor=8) == 2 + 1
    assert traffic.count_unique_destinations(routes, divisor=8, ignored_range=(0, 1)) == 1 + 1
    with pytest.raises(ValueError):
        traffic.count_unique_destinations(routes, divisor=0)


def _fake_report(case_ids, fingerprint='ab' * 32, profile='smoke', world=2, scale=1.0):
    p = profiles.PROFILES[profile]
    known = {c.case_id: c for c in cases.enumerate_mode_cases()}
    t = lambda: {'avg_us': 10.0 * scale, 'min_us': 9.0 * scale, 'max_us': 12.0 * scale, 'logical_gbs': 1.0, 'nvlink_gbs': 0.5}
    cs = [{'case_id': cid, 'suite': known[cid].suite, 'status': 'passed', 'correctness': {op: True for op in cases.CORRECTNESS_OPERATIONS},
           'performance': {op: t() for op in cases.PERFORMANCE_OPERATIONS}} for cid in case_ids]
    return {'schema_version': 1, 'backend': 'cpu', 'device': 'cpu (gloo)', 'world_size': world, 'workload_fingerprint': fingerprint,
            'profile': {k: getattr(p, k) for k in ('name', 'num_tokens', 'hidden', 'num_topk', 'num_experts', 'seed', 'warmups', 'iterations')},
            'cases': cs, 'summary': {'total': len(cs), 'passed': len(cs), 'failed': 0}}


def test_report_schema_and_markdown():
    ids = [c.case_id for c in cases.select_cases('performance')][:3]
    r = _fake_report(ids)
    report.validate_report(r)
    md = report.render_markdown(r)
    assert ids[0] in md and 'fingerprint' in md
    with pytest.raises(ValueError, match='covers'):
        report.validate_report(r, require_all_cases=True)
    for mutate, what in [
        (lambda x: x.pop('summary'), 'lacks'),
        (lambda x: x.update(workload_fingerprint='xyz'), 'SHA-256'),
        (lambda x: x['cases'].append(copy.deepcopy(x['cases'][0])), 'twice'),
        (lambda x: x['cases'][0]['performance']['dispatch'].update(avg_us=-1.0), 'nonnegative'),
        (lambda x: x['cases'][0]['performance']['combine'].update(min_us=99.0), 'min <= avg'),
        (lambda x: x['cases'][0]['correctness'].update(combine=False), 'marked passed'),
        (lambda x: x['summary'].update(passed=0), 'summary'),
        (lambda x: x['profile'].update(hidden=64), 'profile field'),
        (lambda x: x['cases'][0].update(suite='functional'), 'suite'),
    ]:
        bad = copy.deepcopy(r)
        mutate(bad)
        with pytest.raises(ValueError, match=what):
            report.validate_report(bad)


def test_compare_refuses_reports_that_are_not_comparable(tmp_path):
    ids = [c.case_id for c in cases.select_cases('performance')][:2]
    a, b = _fake_report(ids), _fake_report(ids, scale=0.5)
    md = report.compare_reports(a, b)
    assert '2.00x' in md
    with pytest.raises(ValueError, match='fingerprints'):
        report.compare_reports(a, _fake_report(ids, fingerprint='cd' * 32))
    with pytest.raises(ValueError, match='world sizes'):
        report.compare_reports(a, _fake_report(ids, world=4))
    with pytest.raises(ValueError, match='profiles'):
        report.compare_reports(a, _fake_report(ids, profile='canonical'))
    # command line: output must not be one of the inputs, mismatches exit with code 2
    pa, pb = tmp_path / 'a.json', tmp_path / 'b.json'
    pa.write_text(json.dumps(a))
    pb.write_text(json.dumps(_fake_report(ids, fingerprint='cd' * 32)))
    run = lambda *args: subprocess.run([sys.executable, '-m', 'deepep_ascend_b200.benchmark.compare_ep', *args], cwd=REPO, capture_output=True, text=True)
    assert run('--left', str(pa), '--right', str(pb), '--output', str(tmp_path / 'c.md')).returncode == 2
    assert run('--left', str(pa), '--right', str(pa), '--output', str(pa)).returncode == 2
    ok = run('--left', str(pa), '--right', str(pa), '--output', str(tmp_path / 'c.md'))
    assert ok.returncode == 0 and (tmp_path / 'c.md').read_text().startswith('# EP benchmark comparison')


def test_run_ep_command_line_on_two_gloo_ranks(tmp_path):
    cs = cases.enumerate_mode_cases()
    picked = [c for c in cs if c.do_handle_copy and c.expert_alignment == 128 and c.num_bias == 2 and not c.with_previous_event
              and c.async_with_compute_stream == c.allocate_on_comm_stream]
    assert len(picked) == 4          # fp8 / bf16, with and without stream plumbing
    out = tmp_path / 'run'
    cmd = [sys.executable, '-m', 'deepep_ascend_b200.benchmark.run_ep', '--backend', 'cpu', '--profile', 'smoke', '--world-size', '2',
           '--cases', ','.join(c.case_id for c in picked), '--output-dir', str(out)]
    res = subprocess.run(cmd, cwd=REPO, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:] + (out / 'run.log').read_text()[-2000:]
    assert sorted(p.name for p in out.iterdir()) == ['benchmark.json', 'benchmark.md', 'run.log', 'workload.json']
    rep = json.loads((out / 'benchmark.json').read_text())
    report.validate_report(rep)
    assert rep['summary'] == {'total': 4, 'passed': 4, 'failed': 0}
    assert rep['workload_fingerprint'] == workload.load_manifest(out / 'workload.json').fingerprint
    # the same workload can be handed to a second run; a workload of another size is refused
    res2 = subprocess.run(cmd[:-2] + ['--output-dir', str(tmp_path / 'run2'), '--workload-manifest', str(out / 'workload.json')],
                          cwd=REPO, capture_output=True, text=True, timeout=600)
    assert res2.returncode == 0, res2.stderr[-2000:]
    assert json.loads((tmp_path / 'run2' / 'benchmark.json').read_text())['workload_fingerprint'] == rep['workload_fingerprint']
    other = tmp_path / 'w4.json'
    workload.write_manifest(other, profiles.profile_manifest(profiles.PROFILES['smoke'], 4))
    res3 = subprocess.run(cmd[:-2] + ['--output-dir', str(tmp_path / 'run3'), '--workload-manifest', str(other)],
                          cwd=REPO, capture_output=True, text=True, timeout=600)
    assert res3.returncode == 2 and not (tmp_path / 'run3' / 'benchmark.json').exists()
