"""Run the API-mode matrix of expert-parallel dispatch / combine on one backend and write the benchmark artifacts.

    python -m deepep_ascend_b200.benchmark.run_ep --backend cuda --profile canonical --output-dir out/cuda
    python -m deepep_ascend_b200.benchmark.run_ep --backend cpu --profile smoke --world-size 2 --cases performance --output-dir out/cpu

``cuda`` runs one process per GPU (NCCL for the plumbing, this library's kernels for the data), ``cpu`` runs the gloo backend
of the same API.  Artifacts in ``--output-dir``: ``workload.json`` (the routing, with its fingerprint), ``benchmark.json``
(written to ``benchmark.staging.json`` first and renamed when complete), ``benchmark.md`` and ``run.log``.
Every case runs six operations (dispatch, expanded dispatch, cached dispatch, cached expanded dispatch with zero padding, combine,
reduced combine); each is checked against what the workload says must arrive (row counts per rank and per expert, every received
row bit for bit against its source token, the combined tokens against the sum their routing implies) and five are timed.
Parity: tests/benchmark/run_ep.py and the benchmark mode of tests/elastic/test_ep.py of the reference.
"""
import argparse
import json
import os
import socket
import sys
import time
import traceback
from pathlib import Path
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from .cases import CORRECTNESS_OPERATIONS, PERFORMANCE_OPERATIONS, ModeCase, select_cases
from .profiles import PROFILES, Profile, profile_spec
from .report import REPORT_SCHEMA_VERSION, render_markdown, validate_report
from .traffic import combine_traffic, dispatch_row_tensors, dispatch_traffic
from .workload import Manifest, build_manifest, load_manifest, write_manifest, write_text_atomic


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def rank_inputs(manifest: Manifest, rank: int):
    """(x bf16 [T, H], topk_idx int64 [T, K], topk_weights fp32 [T, K]) of one rank, on the CPU.  The activations come from a
    generator seeded by (seed, rank), so any process can rebuild any rank's tokens."""
    spec, rw = manifest.spec, manifest.ranks[rank]
    g = torch.Generator().manual_seed(1000003 * (spec.seed + 1) + rank)
    x = torch.randn(rw.num_tokens, spec.hidden, generator=g).bfloat16()
    idx = torch.tensor(rw.topk_idx, dtype=torch.int64).reshape(rw.num_tokens, spec.num_topk)
    w = torch.tensor(rw.topk_weights, dtype=torch.float32).reshape(rw.num_tokens, spec.num_topk)
    return x, idx, w


class Expectation:
    """What the workload says this rank must receive, derived from the manifest alone."""

    def __init__(self, manifest: Manifest, rank: int, device):
        from ..utils.math import per_token_cast_back, per_token_cast_to_fp8
        spec = manifest.spec
        R, E = spec.world_size, spec.num_experts
        El = E // R
        self.recv_rows = 0
        self.local_rows = 0
        self.per_expert = torch.zeros(El, dtype=torch.int64)
        xs, qs, sfs = [], [], []
        for s in range(R):
            x, idx, _ = rank_inputs(manifest, s)
            valid = idx >= 0
            dest = torch.where(valid, idx // El, torch.full_like(idx, -1))
            hits_me = (dest == rank).any(dim=1)
            self.recv_rows += int(hits_me.sum())
            if s == rank:
                self.local_rows = int(hits_me.sum())
                self.num_dest = torch.stack([(dest == d).any(dim=1) for d in range(R)]).sum(0)       # distinct ranks per token
                self.num_lanes = valid.sum(dim=1)                                                       # valid selections per token
            mine = idx[(dest == rank)] - rank * El
            self.per_expert += torch.bincount(mine, minlength=El)
            q, sf = per_token_cast_to_fp8(x)
            xs.append(x)
            qs.append(q)
            sfs.append(sf)
        self.max_tokens = spec.num_tokens
        # all ranks' tokens stacked with a fixed stride, so that `src_rank * max_tokens + token` indexes them
        pad = lambda t: torch.cat([t, torch.zeros((self.max_tokens - t.shape[0],) + t.shape[1:], dtype=t.dtype)])
        self.all_x = torch.cat([pad(x) for x in xs]).to(device)
        self.all_q = torch.cat([pad(q.view(torch.uint8)) for q in qs]).to(device)
        self.all_sf = torch.cat([pad(sf) for sf in sfs]).to(device)
        self.own_x = xs[rank].to(device)
        self.own_xq = per_token_cast_back(qs[rank], sfs[rank]).to(device)      # what an identity expert sends back under FP8
        self.num_dest = self.num_dest.to(device)
        self.num_lanes = self.num_lanes.to(device)


def _valid_rows(handle, rows: int, device) -> torch.Tensor:
    """Rows of the expand layout that hold a token (the others are alignment padding)."""
    ends = handle.psum_num_recv_tokens_per_expert.to(torch.int64).to(device)
    a = max(1, handle.expert_alignment)
    aligned = (ends + a - 1) // a * a
    starts = torch.cat([torch.zeros(1, dtype=torch.int64, device=device), aligned[:-1]])
    r = torch.arange(rows, device=device).unsqueeze(1)
    return ((r >= starts.unsqueeze(0)) & (r < ends.unsqueeze(0))).any(dim=1)


class CaseRunner:
    def __init__(self, buf, manifest: Manifest, rank: int, exp: Expectation, profile: Profile, backend: str, num_sms: int, group):
        self.buf, self.manifest, self.rank, self.exp, self.profile, self.backend = buf, manifest, rank, exp, profile, backend
        self.num_sms, self.group = num_sms, group
        self.device = 'cuda' if backend == 'cuda' else 'cpu'
        x, idx, w = rank_inputs(manifest, rank)
        self.x, self.idx, self.w = x.to(self.device), idx.to(self.device), w.to(self.device)
        g = torch.Generator().manual_seed(77 + rank)
        self.bias = [torch.randn(x.shape, generator=g).bfloat16().to(self.device) for _ in range(2)]

    # ---------------------------------------------------------------- API calls
    def _plumbing(self, case: ModeCase) -> Dict[str, Any]:
        kw = dict(async_with_compute_stream=case.async_with_compute_stream, allocate_on_comm_stream=case.allocate_on_comm_stream,
                  num_sms=self.num_sms)
        if case.with_previous_event:
            kw['previous_event'] = self.buf.capture()
        return kw

    def _finish(self, case: ModeCase, event) -> None:
        if case.async_with_compute_stream and event is not None:
            event.current_stream_wait()

    def dispatch(self, case: ModeCase, do_expand: bool, handle=None, zero_padding: bool = False):
        spec = self.manifest.spec
        kw = self._plumbing(case)
        if handle is None:
            out = self.buf.dispatch(self.x, self.idx, self.w, num_experts=spec.num_experts, expert_alignment=case.expert_alignment,
                                    do_handle_copy=case.do_handle_copy, do_expand=do_expand,
                                    use_tma_aligned_col_major_sf=do_expand and case.use_fp8_dispatch, **kw)
        else:
            out = self.buf.dispatch(self.x, handle=handle, topk_weights=self.w, do_zero_padding=zero_padding,
                                    use_tma_aligned_col_major_sf=handle.do_expand and case.use_fp8_dispatch, **kw)
        self._finish(case, out[4])
        return out

    def combine(self, case: ModeCase, y, handle, with_bias: bool, recv_w=None):
        bias = None
        if with_bias and case.num_bias == 1:
            bias = self.bias[0]
        elif with_bias and case.num_bias == 2:
            bias = (self.bias[0], self.bias[1])
        out = self.buf.combine(y, handle, topk_weights=recv_w, bias=bias, **self._plumbing(case))
        self._finish(case, out[2])
        return out

    # ---------------------------------------------------------------- checks
    def _rows_of(self, recv_x, case: ModeCase):
        from ..utils.math import per_token_cast_back
        if case.use_fp8_dispatch:
            q, sf = recv_x
            return per_token_cast_back(q, sf.contiguous() if sf.stride(-1) != 1 else sf)
        return recv_x

    def check_dispatch(self, out, case: ModeCase, do_expand: bool) -> bool:
        recv_x, recv_idx, recv_w, handle, _ = out
        exp = self.exp
        ok = handle.num_unaligned_recv_tokens_per_expert.cpu().to(torch.int64).tolist() == exp.per_expert.tolist()
        rows = handle.num_rows
        if do_expand:
            valid = _valid_rows(handle, rows, self.device)
            ok &= int(valid.sum()) == int(exp.per_expert.sum())
        else:
            ok &= rows == exp.recv_rows == int(handle.psum_num_recv_tokens_per_scaleup_rank[-1])
            valid = torch.ones(rows, dtype=torch.bool, device=self.device)
        src = handle.recv_src_metadata[:rows, 0].to(torch.int64)
        buf_max = handle.num_max_tokens_per_rank
        src = (src // buf_max) * exp.max_tokens + src % buf_max            # the buffer may have been sized for more tokens
        src = torch.where(valid, src, torch.zeros_like(src))
        if case.use_fp8_dispatch:
            q, sf = recv_x
            ok &= bool(torch.equal(q[:rows].view(torch.uint8)[valid], exp.all_q[src][valid]))
            ok &= bool(torch.equal(sf[:rows][valid].float(), exp.all_sf[src][valid]))
        else:
            ok &= bool(torch.equal(recv_x[:rows][valid].view(torch.int16), exp.all_x[src][valid].view(torch.int16)))
        return bool(ok)

    def check_same_payload(self, a, b, case: ModeCase, handle, zero_padding: bool) -> bool:
        xa = a[0][0] if case.use_fp8_dispatch else a[0]
        xb = b[0][0] if case.use_fp8_dispatch else b[0]
        rows = handle.num_rows
        valid = _valid_rows(handle, rows, self.device) if handle.do_expand else torch.ones(rows, dtype=torch.bool, device=self.device)
        ua, ub = xa[:rows].view(torch.uint8), xb[:rows].view(torch.uint8)
        ok = bool(torch.equal(ua[valid], ub[valid]))
        if zero_padding and handle.do_expand:
            ok &= not bool(ub[~valid].any())
        return ok

    def check_combine(self, out, case: ModeCase, count: torch.Tensor, with_bias: bool, back_w=None) -> bool:
        base = self.exp.own_xq if case.use_fp8_dispatch else self.exp.own_x
        want = base.float() * count.unsqueeze(1).float()
        nb = case.num_bias if with_bias else 0
        for b in self.bias[:nb]:
            want = want + b.float()
        got = out[0].float()
        if nb == 0:
            ok = bool(torch.equal(out[0].view(torch.int16), want.bfloat16().view(torch.int16)))
        else:
            ok = bool(torch.allclose(got, want, rtol=2e-2, atol=2e-2))
        if back_w is not None:
            v = self.idx >= 0
            ok &= bool(torch.equal(out[1][v], self.w[v]))
        return ok

    # ---------------------------------------------------------------- timing
    def _time(self, fn) -> Dict[str, float]:
        """avg / min / max microseconds over the profile's iterations, max over ranks of each."""
        p = self.profile
        for _ in range(p.warmups):
            fn()
        samples = []
        if self.backend == 'cuda':
            evs = []
            for _ in range(p.iterations):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                evs.append((a, b))
            torch.cuda.synchronize()
            samples = [a.elapsed_time(b) * 1e3 for a, b in evs]
        else:
            for _ in range(p.iterations):
                t0 = time.perf_counter()
                fn()
                samples.append((time.perf_counter() - t0) * 1e6)
        t = torch.tensor([sum(samples) / len(samples), -min(samples), max(samples)], dtype=torch.float64, device=self.device)
        if self.group is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        avg, neg_min, mx = t.tolist()
        return {'avg_us': avg, 'min_us': min(-neg_min, avg), 'max_us': max(mx, avg)}

    @staticmethod
    def _with_rates(t: Dict[str, float], logical: int, nvlink: int) -> Dict[str, float]:
        secs = max(t['avg_us'], 1e-3) * 1e-6
        return dict(t, logical_gbs=logical / secs / 1e9, nvlink_gbs=nvlink / secs / 1e9)

    # ---------------------------------------------------------------- one case
    def run(self, case: ModeCase) -> Dict[str, Any]:
        spec, exp = self.manifest.spec, self.exp
        corr: Dict[str, bool] = {}
        d = self.dispatch(case, False)
        corr['dispatch'] = self.check_dispatch(d, case, False)
        e = self.dispatch(case, True)
        corr['expanded_dispatch'] = self.check_dispatch(e, case, True)
        # the cached calls land in other receive slots: take copies of what they are compared with
        keep = lambda o: (tuple(t.clone() for t in o[0]) if isinstance(o[0], tuple) else o[0].clone(),)
        d_keep, e_keep = keep(d), keep(e)
        y = self._rows_of(d[0], case).clone()
        recv_w = d[2].clone()
        ye = self._rows_of(e[0], case).clone()
        ye = torch.where(_valid_rows(e[3], e[3].num_rows, self.device).unsqueeze(1), ye[:e[3].num_rows], torch.zeros_like(ye[:e[3].num_rows]))
        cd = self.dispatch(case, False, handle=d[3])
        corr['cached_dispatch'] = self.check_same_payload(d_keep, cd, case, d[3], False)
        ce = self.dispatch(case, True, handle=e[3], zero_padding=True)
        corr['cached_expanded_padding'] = self.check_same_payload(e_keep, ce, case, e[3], True)
        c = self.combine(case, y, d[3], True, recv_w=recv_w)
        corr['combine'] = self.check_combine(c, case, exp.num_dest, True, back_w=True)
        rc = self.combine(case, ye, e[3], False)
        corr['reduced_combine'] = self.check_combine(rc, case, exp.num_lanes, False)
        if self.backend == 'cuda':
            torch.cuda.synchronize()
            self.buf.check_status()

        tensors = dispatch_row_tensors(spec.hidden, spec.num_topk, case.use_fp8_dispatch)
        dt = dispatch_traffic(tensors, exp.recv_rows, exp.local_rows)
        lanes_here = int(exp.per_expert.sum())
        et = dispatch_traffic(tensors[:2] if case.use_fp8_dispatch else tensors[:1], lanes_here, 0)
        ct = combine_traffic(exp.recv_rows, exp.local_rows, self.x.shape[0], spec.hidden, case.num_bias)
        rt = combine_traffic(lanes_here, 0, self.x.shape[0], spec.hidden, 0)
        perf = {
            'dispatch': self._with_rates(self._time(lambda: self.dispatch(case, False)), dt.logical_bytes, dt.nvlink_bytes),
            'expanded_dispatch': self._with_rates(self._time(lambda: self.dispatch(case, True)), et.logical_bytes, et.logical_bytes),
            'cached_dispatch': self._with_rates(self._time(lambda: self.dispatch(case, False, handle=d[3])), dt.logical_bytes, dt.nvlink_bytes),
            'combine': self._with_rates(self._time(lambda: self.combine(case, y, d[3], True, recv_w=recv_w)), ct.logical_bytes, ct.nvlink_bytes),
            'reduced_combine': self._with_rates(self._time(lambda: self.combine(case, ye, e[3], False)), rt.logical_bytes, rt.logical_bytes),
        }
        ok = torch.tensor([int(all(corr.values()))], device=self.device)
        if self.group is not None:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        for op in CORRECTNESS_OPERATIONS:
            flag = torch.tensor([int(corr[op])], device=self.device)
            if self.group is not None:
                dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
            corr[op] = bool(flag.item())
        return {'case_id': case.case_id, 'suite': case.suite, 'status': 'passed' if ok.item() else 'failed', 'correctness': corr,
                'performance': {op: perf[op] for op in PERFORMANCE_OPERATIONS}}


def _worker(rank: int, world: int, port: int, backend: str, profile_name: str, manifest_path: str, case_spec: str,
            staging: str, log_path: str, num_sms: int) -> None:
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    log = open(log_path, 'a', encoding='utf-8') if rank == 0 else None

    def say(msg: str) -> None:
        if log is not None:
            log.write(msg + '\n')
            log.flush()
    if backend == 'cuda':
        torch.cuda.set_device(rank)
        dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    else:
        dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        from .. import ElasticBuffer
        profile = PROFILES[profile_name]
        manifest = load_manifest(manifest_path)
        spec = manifest.spec
        group = dist.new_group(list(range(world)))
        device = 'cuda' if backend == 'cuda' else 'cpu'
        exp = Expectation(manifest, rank, device)
        cases = select_cases(case_spec)
        results: List[Dict[str, Any]] = []
        for fp8 in (True, False):
            todo = [c for c in cases if c.use_fp8_dispatch == fp8]
            if not todo:
                continue
            buf = ElasticBuffer(group, num_max_tokens_per_rank=spec.num_tokens, hidden=spec.hidden, num_topk=spec.num_topk,
                                use_fp8_dispatch=fp8, enable_expand=True, num_experts=spec.num_experts, expert_alignment=128,
                                num_recv_slots=4)
            runner = CaseRunner(buf, manifest, rank, exp, profile, backend, num_sms, group)
            for case in todo:
                try:
                    res = runner.run(case)
                except Exception:       # a failing case must not take the other cases' results with it
                    say('case %s raised on rank %d:\n%s' % (case.case_id, rank, traceback.format_exc()))
                    raise
                results.append(res)
                bad = [op for op in CORRECTNESS_OPERATIONS if not res['correctness'][op]]
                say('%s %s dispatch %.1f us combine %.1f us%s' % (res['case_id'], res['status'], res['performance']['dispatch']['avg_us'],
                                                                 res['performance']['combine']['avg_us'],
                                                                 (' wrong: ' + ', '.join(bad)) if bad else ''))
            buf.destroy()
        if rank == 0:
            order = {c.case_id: i for i, c in enumerate(cases)}
            results.sort(key=lambda r: order[r['case_id']])
            passed = sum(r['status'] == 'passed' for r in results)
            report = {
                'schema_version': REPORT_SCHEMA_VERSION, 'backend': backend,
                'device': torch.cuda.get_device_name(0) if backend == 'cuda' else 'cpu (gloo)',
                'profile': {k: getattr(profile, k) for k in ('name', 'num_tokens', 'hidden', 'num_topk', 'num_experts', 'seed', 'warmups',
                                                             'iterations')},
                'world_size': world, 'workload_fingerprint': manifest.fingerprint, 'num_sms': num_sms, 'cases': results,
                'summary': {'total': len(results), 'passed': passed, 'failed': len(results) - passed},
            }
            write_text_atomic(staging, json.dumps(report, indent=1, sort_keys=True) + '\n')
    finally:
        if log is not None:
            log.close()
        dist.destroy_process_group()


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description='Run the EP API-mode matrix on one backend and write benchmark artifacts')
    p.add_argument('--backend', choices=('cuda', 'cpu'), required=True)
    p.add_argument('--profile', choices=tuple(PROFILES), default='smoke')
    p.add_argument('--world-size', type=int, default=0, help='ranks (default: the profile\'s, capped by the visible GPUs for cuda)')
    p.add_argument('--cases', default='all', help='all | performance | functional | comma-separated case ids')
    p.add_argument('--num-sms', type=int, default=64)
    p.add_argument('--output-dir', type=Path, required=True)
    p.add_argument('--workload-manifest', type=Path, help='reuse this workload.json instead of generating one')
    return p


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    profile = PROFILES[args.profile]
    world = args.world_size or profile.world_size
    if args.backend == 'cuda':
        if not torch.cuda.is_available():
            print('the cuda backend needs GPUs', file=sys.stderr)
            return 2
        world = min(world, torch.cuda.device_count()) if not args.world_size else world
        if world > torch.cuda.device_count():
            print('world size %d exceeds the %d visible GPUs' % (world, torch.cuda.device_count()), file=sys.stderr)
            return 2
    select_cases(args.cases)          # fail early on unknown ids
    out = args.output_dir
    out.mkdir(parents=True, exist_ok=True)
    manifest_path = out / 'workload.json'
    if args.workload_manifest is not None:
        manifest = load_manifest(args.workload_manifest)
        if manifest.spec != profile_spec(profile, manifest.spec.world_size) or manifest.spec.world_size != world:
            print('the workload manifest does not belong to profile %s at world size %d' % (profile.name, world), file=sys.stderr)
            return 2
    else:
        manifest = build_manifest(profile_spec(profile, world))
    write_manifest(manifest_path, manifest)
    staging, final, md, log = out / 'benchmark.staging.json', out / 'benchmark.json', out / 'benchmark.md', out / 'run.log'
    for stale in (staging, final, md):
        if stale.exists():
            stale.unlink()
    log.write_text('backend %s profile %s world %d cases %s fingerprint %s\n' % (args.backend, profile.name, world, args.cases,
                                                                               manifest.fingerprint), encoding='utf-8')
    try:
        mp.spawn(_worker, args=(world, _free_port(), args.backend, profile.name, str(manifest_path), args.cases, str(staging), str(log),
                                args.num_sms), nprocs=world, join=True)
    except Exception as e:          # the staging file is never promoted after a failed run
        with open(log, 'a', encoding='utf-8') as f:
            f.write('run failed: %r\n' % (e,))
        print('benchmark run failed, see %s' % log, file=sys.stderr)
        return 1
    report = json.loads(staging.read_text(encoding='utf-8'))
    validate_report(report)
    write_text_atomic(md, render_markdown(report))
    os.replace(staging, final)
    print(json.dumps({'output_dir': str(out), 'summary': report['summary'], 'workload_fingerprint': report['workload_fingerprint']}))
    return 0 if report['summary']['failed'] == 0 else 1


if __name__ == '__main__':
    raise SystemExit(main())
