"""``benchmark.json`` schema check, markdown rendering and the comparison of two reports.

A report is comparable with another one only if both were produced from the same workload (equal fingerprints) and the
same profile; ``compare_reports`` refuses anything else.
Parity: tests/benchmark/report_markdown.py and compare_ep.py of the reference.
"""
from typing import Any, Dict, List

from .cases import CORRECTNESS_OPERATIONS, PERFORMANCE_OPERATIONS, enumerate_mode_cases
from .profiles import PROFILES

REPORT_SCHEMA_VERSION = 1
_TOP_KEYS = ('schema_version', 'backend', 'device', 'profile', 'world_size', 'workload_fingerprint', 'cases', 'summary')
_TIMING_KEYS = ('avg_us', 'min_us', 'max_us', 'logical_gbs', 'nvlink_gbs')


def _fail(msg: str) -> None:
    raise ValueError(msg)


def identify_profile(report: Dict[str, Any]):
    p = report.get('profile')
    if not isinstance(p, dict) or p.get('name') not in PROFILES:
        _fail('report names no known profile')
    prof = PROFILES[p['name']]
    for key in ('num_tokens', 'hidden', 'num_topk', 'num_experts', 'seed', 'warmups', 'iterations'):
        if p.get(key) != getattr(prof, key):
            _fail('profile field %s does not match profile %s' % (key, prof.name))
    return prof


def validate_report(report: Dict[str, Any], require_all_cases: bool = False) -> None:
    """Raise ``ValueError`` naming the first thing that is wrong with ``report``."""
    if not isinstance(report, dict):
        _fail('report must be a JSON object')
    for k in _TOP_KEYS:
        if k not in report:
            _fail('report lacks ' + k)
    if report['schema_version'] != REPORT_SCHEMA_VERSION:
        _fail('unsupported report schema_version')
    if report['backend'] not in ('cuda', 'cpu'):
        _fail('unknown backend')
    identify_profile(report)
    fp = report['workload_fingerprint']
    if not (isinstance(fp, str) and len(fp) == 64 and all(c in '0123456789abcdef' for c in fp)):
        _fail('workload_fingerprint must be a SHA-256 hex digest')
    known = {c.case_id: c for c in enumerate_mode_cases()}
    seen = set()
    passed = failed = 0
    for case in report['cases']:
        cid = case.get('case_id')
        if cid not in known:
            _fail('unknown case id %r' % (cid,))
        if cid in seen:
            _fail('case %s is listed twice' % cid)
        seen.add(cid)
        if case.get('suite') != known[cid].suite:
            _fail('case %s has the wrong suite' % cid)
        if case.get('status') not in ('passed', 'failed'):
            _fail('case %s has no status' % cid)
        corr = case.get('correctness', {})
        for op in CORRECTNESS_OPERATIONS:
            if not isinstance(corr.get(op), bool):
                _fail('case %s lacks the correctness result of %s' % (cid, op))
        if case['status'] == 'passed' and not all(corr[op] for op in CORRECTNESS_OPERATIONS):
            _fail('case %s is marked passed with a failed operation' % cid)
        perf = case.get('performance', {})
        for op in PERFORMANCE_OPERATIONS:
            t = perf.get(op)
            if not isinstance(t, dict):
                _fail('case %s lacks the timing of %s' % (cid, op))
            for k in _TIMING_KEYS:
                v = t.get(k)
                if not isinstance(v, (int, float)) or v < 0 or v != v:
                    _fail('case %s, %s: %s must be a nonnegative number' % (cid, op, k))
            if not t['min_us'] <= t['avg_us'] <= t['max_us']:
                _fail('case %s, %s: min <= avg <= max does not hold' % (cid, op))
        passed += case['status'] == 'passed'
        failed += case['status'] == 'failed'
    if require_all_cases and seen != set(known):
        _fail('report covers %d of %d cases' % (len(seen), len(known)))
    s = report['summary']
    if s.get('total') != len(seen) or s.get('passed') != passed or s.get('failed') != failed:
        _fail('summary does not match the cases')


def _fmt(v: float) -> str:
    return '%.1f' % v


def render_markdown(report: Dict[str, Any]) -> str:
    validate_report(report)
    p = report['profile']
    out: List[str] = ['# EP benchmark - %s on %s' % (report['backend'], report['device']), '',
                      'Profile `%s`: %d ranks, %d tokens/rank, hidden %d, top-%d of %d experts, %d warm-up + %d timed iterations.'
                      % (p['name'], report['world_size'], p['num_tokens'], p['hidden'], p['num_topk'], p['num_experts'], p['warmups'],
                         p['iterations']),
                      'Workload fingerprint `%s`.' % report['workload_fingerprint'],
                      'Cases: %d run, %d passed, %d failed.' % (report['summary']['total'], report['summary']['passed'],
                                                                report['summary']['failed']), '',
                      '| case | suite | status | ' + ' | '.join('%s us (GB/s)' % op for op in PERFORMANCE_OPERATIONS) + ' |',
                      '|---|---|---|' + '---|' * len(PERFORMANCE_OPERATIONS)]
    for case in report['cases']:
        cells = ['%s (%s)' % (_fmt(case['performance'][op]['avg_us']), _fmt(case['performance'][op]['logical_gbs']))
                 for op in PERFORMANCE_OPERATIONS]
        out.append('| %s | %s | %s | %s |' % (case['case_id'], case['suite'], case['status'], ' | '.join(cells)))
    return '\n'.join(out) + '\n'


def compare_reports(left: Dict[str, Any], right: Dict[str, Any]) -> str:
    """Markdown table of ``right`` against ``left`` for the performance suite; refuses reports that are not comparable."""
    validate_report(left)
    validate_report(right)
    if identify_profile(left).name != identify_profile(right).name:
        _fail('the reports were made with different profiles')
    if left['world_size'] != right['world_size']:
        _fail('the reports were made with different world sizes')
    if left['workload_fingerprint'] != right['workload_fingerprint']:
        _fail('the reports were made from different workloads (fingerprints differ)')
    lcases = {c['case_id']: c for c in left['cases'] if c['suite'] == 'performance'}
    rcases = {c['case_id']: c for c in right['cases'] if c['suite'] == 'performance'}
    common = [cid for cid in lcases if cid in rcases]
    if not common:
        _fail('the reports share no performance case')
    out = ['# EP benchmark comparison: %s (%s) vs %s (%s)' % (right['backend'], right['device'], left['backend'], left['device']), '',
           'Workload fingerprint `%s`, profile `%s`.' % (left['workload_fingerprint'], left['profile']['name']), '',
           '| case | operation | left us | right us | right / left speed |', '|---|---|---|---|---|']
    for cid in common:
        for op in PERFORMANCE_OPERATIONS:
            a, b = lcases[cid]['performance'][op]['avg_us'], rcases[cid]['performance'][op]['avg_us']
            out.append('| %s | %s | %s | %s | %s |' % (cid, op, _fmt(a), _fmt(b), ('%.2fx' % (a / b)) if b > 0 else 'n/a'))
    return '\n'.join(out) + '\n'
