"""Byte counts behind the GB/s a benchmark reports (one NVLink domain: "scale-up" traffic only).

``logical`` bytes follow the reference's convention (tests/elastic/test_ep.py:443-568, tests/utils/ep_benchmark_core.py:126-198):
all rows a rank receives (dispatch) or contributes (combine) times the row size, local rows included; ``nvlink`` bytes leave out
the rows that stay on the rank.
"""
from dataclasses import dataclass
from typing import Iterable, Optional, Sequence, Tuple


@dataclass(frozen=True)
class TensorBytes:
    rows: int
    row_bytes: int

    def __post_init__(self) -> None:
        if self.rows < 0 or self.row_bytes < 0:
            raise ValueError('tensor byte dimensions must be nonnegative')


@dataclass(frozen=True)
class DispatchTraffic:
    bytes_per_token: int
    logical_bytes: int
    nvlink_bytes: int


@dataclass(frozen=True)
class CombineTraffic:
    logical_bytes: int
    nvlink_bytes: int
    reduction_bytes: int


def dispatch_row_tensors(hidden: int, num_topk: int, use_fp8: bool, idx_bytes: int = 8) -> Tuple[TensorBytes, ...]:
    """What travels with one dispatched row: payload, 1x128 scales (FP8), expert ids, weights, source metadata."""
    parts = [TensorBytes(1, hidden if use_fp8 else 2 * hidden)]
    if use_fp8:
        parts.append(TensorBytes(1, 4 * ((hidden + 127) // 128)))
    parts += [TensorBytes(1, idx_bytes * num_topk), TensorBytes(1, 4 * num_topk), TensorBytes(1, 8)]
    return tuple(parts)


def dispatch_traffic(tensors: Iterable[TensorBytes], num_recv_rows: int, num_local_rows: int) -> DispatchTraffic:
    tensors = tuple(tensors)
    if num_recv_rows < 0 or num_local_rows < 0 or num_local_rows > num_recv_rows:
        raise ValueError('row counts must satisfy 0 <= local <= received')
    if any(t.rows != tensors[0].rows for t in tensors[1:]):
        raise ValueError('dispatch tensors must have matching row counts')
    per = sum(t.row_bytes for t in tensors)
    return DispatchTraffic(per, per * num_recv_rows, per * (num_recv_rows - num_local_rows))


def combine_traffic(num_rows: int, num_local_rows: int, num_tokens: int, hidden: int, num_bias: int = 0) -> CombineTraffic:
    if min(num_rows, num_local_rows, num_tokens, hidden, num_bias) < 0 or num_local_rows > num_rows:
        raise ValueError('combine traffic inputs must be nonnegative with local <= rows')
    row = 2 * hidden
    return CombineTraffic(row * num_rows, row * (num_rows - num_local_rows), row * (num_rows + num_bias * num_tokens + num_tokens))


def count_unique_destinations(routes: Sequence[Sequence[int]], divisor: int = 1,
                              ignored_range: Optional[Tuple[int, int]] = None) -> int:
    """Rows a rank sends in the non-expand layout: distinct ``route // divisor`` per token, ``-1`` skipped, destinations in
    ``ignored_range`` (for example the sender itself) left out."""
    if divisor <= 0:
        raise ValueError('divisor must be positive')
    if ignored_range is not None and ignored_range[0] > ignored_range[1]:
        raise ValueError('ignored destination range must be ordered')
    n = 0
    for row in routes:
        dests = {r // divisor for r in row if r >= 0}
        if ignored_range is not None:
            dests = {d for d in dests if not ignored_range[0] <= d < ignored_range[1]}
        n += len(dests)
    return n
