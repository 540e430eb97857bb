"""Benchmark helpers: L2 flush, CUDA-event timing, per-kernel timing through the profiler, and
percentile summaries (parity: deep_ep/utils/testing.py:12-219)."""
import os
from typing import Callable, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch
import torch.distributed as dist

L2_FLUSH_BYTES = 256 * 1024 * 1024   # > 126 MB of B200 L2
_flush_buffers: Dict[int, torch.Tensor] = {}


def flush_l2_cache(enabled: bool = True) -> None:
    """Overwrite a 256 MB scratch tensor so nothing of the previous iteration stays in L2."""
    if not enabled:
        return
    dev = torch.cuda.current_device()
    buf = _flush_buffers.get(dev)
    if buf is None:
        buf = _flush_buffers[dev] = torch.empty(L2_FLUSH_BYTES // 4, dtype=torch.int32, device='cuda')
    buf.zero_()


def bench(fn: Callable, num_warmups: int = 5, num_tests: int = 20, post_fn: Optional[Callable] = None,
          flush_l2: bool = True, barrier_group: Optional[dist.ProcessGroup] = None) -> Tuple[float, float, float]:
    """Time ``fn`` with CUDA events on the current stream; returns (mean, min, max) seconds.
    With ``barrier_group`` every sample is preceded by a group barrier so ranks start together."""
    torch.cuda.synchronize()
    for _ in range(num_warmups):
        fn()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(num_tests)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(num_tests)]
    for i in range(num_tests):
        flush_l2_cache(flush_l2)
        if barrier_group is not None:
            dist.barrier(group=barrier_group)
        starts[i].record()
        fn()
        ends[i].record()
        if post_fn is not None:
            post_fn()
    torch.cuda.synchronize()
    times = np.array([s.elapsed_time(e) / 1e3 for s, e in zip(starts, ends)])
    return float(times.mean()), float(times.min()), float(times.max())


def bench_samples(fn: Callable, num_warmups: int, num_tests: int, flush_l2: bool = True,
                  pre_fn: Optional[Callable] = None) -> np.ndarray:
    """Like :func:`bench` but returns every sample (seconds) for percentile reports."""
    torch.cuda.synchronize()
    for _ in range(num_warmups):
        if pre_fn is not None:
            pre_fn()
        fn()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(num_tests)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(num_tests)]
    for i in range(num_tests):
        flush_l2_cache(flush_l2)
        if pre_fn is not None:
            pre_fn()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    return np.array([s.elapsed_time(e) / 1e3 for s, e in zip(starts, ends)])


def percentiles(samples: Sequence[float], qs: Sequence[float] = (50, 95, 99)) -> Dict[str, float]:
    arr = np.asarray(samples, dtype=np.float64)
    out = {'mean': float(arr.mean()), 'min': float(arr.min()), 'max': float(arr.max())}
    for q in qs:
        out[f'p{int(q)}'] = float(np.percentile(arr, q))
    return out


def max_over_ranks(value: float, group: Optional[dist.ProcessGroup] = None) -> float:
    """Slowest rank's value; multi-GPU timings are reported as the max over ranks."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device='cuda' if torch.cuda.is_available() else 'cpu')
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def bench_kineto(fn: Callable, kernel_names: Union[str, Sequence[str]], num_tests: int = 20,
                 flush_l2: bool = True, barrier_group: Optional[dist.ProcessGroup] = None,
                 trace_path: Optional[str] = None) -> Union[float, List[float]]:
    """Average device time (seconds) of the kernels whose name contains each entry of ``kernel_names``,
    measured with ``torch.profiler``.  Before each sample the GPU is kept busy for a few ms and the ranks
    meet at a barrier so launch skew is not counted as kernel time.  ``EP_USE_NVIDIA_TOOLS=1`` skips the
    profiler (one plain run) so an outer ncu capture is not disturbed."""
    single = isinstance(kernel_names, str)
    names = [kernel_names] if single else list(kernel_names)
    if int(os.environ.get('EP_USE_NVIDIA_TOOLS', '0')):
        fn()
        return 0.0 if single else [0.0] * len(names)
    fn()
    torch.cuda.synchronize()
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA]) as prof:
        for _ in range(num_tests):
            flush_l2_cache(flush_l2)
            if barrier_group is not None:
                torch.cuda._sleep(int(2e7))
                dist.barrier(group=barrier_group)
            fn()
        torch.cuda.synchronize()
    if trace_path is not None:
        prof.export_chrome_trace(trace_path)
    totals = {n: [0.0, 0] for n in names}
    for evt in prof.key_averages():
        for n in names:
            if n in evt.key:
                totals[n][0] += evt.device_time_total * 1e-6
                totals[n][1] += evt.count
    out = [totals[n][0] / max(totals[n][1], 1) for n in names]
    return out[0] if single else out
